"""Typed configuration records.

Two levels are kept apart on purpose:

* an *architecture configuration* (a subclass of :class:`TypedConfig`) is the
  typed image of one architecture's own ``config.json`` keys; and
* a :class:`ModelSpec` is the architecture-neutral description that the
  framework builds from: a list of layers, each naming its mixer, feed-forward,
  norms and block arrangement with their sizes and constants as parameters, and
  a schedule (the order in which layers run, as data).

Nothing below this level reads ``config.json`` keys, and nothing in the parts
knows which architecture it sits in.  The reference keeps the same split between
metadata parsing (src/model.c:2309-2521) and the per-layer op list
(src/models/lfm.c:7-62, src/recipe/builders.c:47-69).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields, MISSING
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """A configuration that cannot be used; the message names the key."""


_REQUIRED = object()


def cfg(default: Any = _REQUIRED, *, key: Optional[str] = None, doc: str = ""):
    """Declare one config.json key of a :class:`TypedConfig`.

    ``default`` left out means the key is required.  ``key`` is the JSON key if
    it differs from the attribute name.
    """
    meta = {"json_key": key, "doc": doc, "required": default is _REQUIRED}
    if default is _REQUIRED:
        return field(default=None, metadata=meta)
    if isinstance(default, (list, dict)):
        return field(default_factory=lambda: type(default)(default), metadata=meta)
    return field(default=default, metadata=meta)


def _coerce(name: str, value: Any, typ: Any) -> Any:
    """Check ``value`` against the annotated type ``typ`` (int, float, bool, str,
    List[str], List[int], Optional[...])."""
    origin = getattr(typ, "__origin__", None)
    args = getattr(typ, "__args__", ())
    if origin is not None and type(None) in args:  # Optional[T]
        if value is None:
            return None
        inner = [a for a in args if a is not type(None)][0]
        return _coerce(name, value, inner)
    if origin in (list, List):
        if not isinstance(value, (list, tuple)):
            raise ConfigError(f"config key '{name}': expected a list, got {type(value).__name__}")
        return [_coerce(f"{name}[{i}]", v, args[0]) for i, v in enumerate(value)]
    if typ is bool:
        if isinstance(value, bool):
            return value
        raise ConfigError(f"config key '{name}': expected true/false, got {value!r}")
    if typ is int:
        if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value:
            raise ConfigError(f"config key '{name}': expected an integer, got {value!r}")
        return int(value)
    if typ is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config key '{name}': expected a number, got {value!r}")
        return float(value)
    if typ is str:
        if not isinstance(value, str):
            raise ConfigError(f"config key '{name}': expected a string, got {value!r}")
        return value
    return value


@dataclass
class TypedConfig:
    """Base of every architecture configuration.

    Subclasses are dataclasses whose fields are declared with :func:`cfg`.
    Unknown keys in the JSON are ignored (the reference ignores metadata keys
    it does not read); a missing required key is an error that names the key
    (src/model.c:98-104).
    """

    @classmethod
    def from_dict(cls, d: Dict[str, Any]):
        import typing

        hints = typing.get_type_hints(cls)
        kwargs = {}
        for f in fields(cls):
            k = f.metadata.get("json_key") or f.name
            if k in d and d[k] is not None:
                kwargs[f.name] = _coerce(k, d[k], hints[f.name])
            elif f.metadata.get("required"):
                raise ConfigError(f"config.json: missing required key '{k}'")
        obj = cls(**kwargs)
        obj.validate()
        return obj

    def to_dict(self) -> Dict[str, Any]:
        out = {}
        for f in fields(self):
            k = f.metadata.get("json_key") or f.name
            out[k] = getattr(self, f.name)
        return out

    def validate(self) -> None:  # overridden
        pass


# --------------------------------------------------------------------------
# Architecture-neutral description
# --------------------------------------------------------------------------

@dataclass
class PartSpec:
    """One part of a layer: its registry ``kind``, its sizes and constants
    (``params``), the prefix of its tensor names in the weight file and an
    optional renaming of the part's local tensor names to the file's."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""
    rename: Dict[str, str] = field(default_factory=dict)


@dataclass
class LayerSpec:
    """A block: the arrangement (``block``) of a mixer, a feed-forward and the
    norms it needs.  Chosen layer by layer."""

    mixer: PartSpec
    ffn: Optional[PartSpec]
    mixer_norm: Optional[PartSpec]
    ffn_norm: Optional[PartSpec]
    block: str = "prenorm_residual"


@dataclass
class ScheduleEntry:
    """One run of a layer.  ``layer`` indexes :attr:`ModelSpec.layers` (a layer
    may be named by several entries: its weights are then shared and every entry
    gets a cache of its own).  ``cache_of`` names an earlier schedule entry whose
    cache this run reads instead of keeping one (it then writes nothing)."""

    layer: int
    cache_of: Optional[int] = None


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: Optional[PartSpec]
    head: PartSpec
    eos_token_id: Optional[int] = None

    def validate(self) -> None:
        if self.hidden_size < 1 or self.vocab_size < 1:
            raise ConfigError("hidden_size and vocab_size must be positive")
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.layers)):
                raise ConfigError(f"schedule[{i}] names layer {e.layer}, model has {len(self.layers)}")
            if e.cache_of is not None:
                if not (0 <= e.cache_of < i):
                    raise ConfigError(f"schedule[{i}].cache_of={e.cache_of} must name an earlier entry")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ConfigError(f"schedule[{i}].cache_of names an entry that itself borrows a cache")


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no such file")
    with open(path, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d
