"""One registry from an architecture's name to its model.

The key is ``config.json``'s ``architectures[0]``.  The reference keeps two
tables (arch flags by GGUF name, src/arch.c:12-114, and constructor-registered
layer builders, src/recipe.h:577-580, src/recipe/build.c:14-42); here one entry
carries both: the typed configuration class and the function that turns a
configuration into a :class:`~kappai_b200.config.schema.ModelSpec`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Type

from .schema import ConfigError, ModelSpec, TypedConfig, read_config_json


@dataclass
class Architecture:
    name: str
    config_cls: Type[TypedConfig]
    build_spec: Callable[[Any], ModelSpec]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: Type[TypedConfig],
                          build_spec: Callable[[Any], ModelSpec], *, replace: bool = False) -> Architecture:
    if name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture '{name}' is already registered")
    arch = Architecture(name, config_cls, build_spec)
    _ARCHITECTURES[name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def lookup_architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        known = ", ".join(sorted(_ARCHITECTURES)) or "(none)"
        # src/arch.c:133-137 — an unknown architecture is an error that names it
        raise ConfigError(f"unsupported architecture '{name}' (known: {known})") from None


def architecture_names():
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def architecture_of(config_dict: Dict[str, Any]) -> Architecture:
    archs = config_dict.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: missing required key 'architectures' (a list with one name)")
    return lookup_architecture(archs[0])


def config_from_dict(config_dict: Dict[str, Any]):
    """Return ``(architecture, typed config)`` for a parsed config.json."""
    arch = architecture_of(config_dict)
    return arch, arch.config_cls.from_dict(config_dict)


def load_config(model_dir: str):
    return config_from_dict(read_config_json(model_dir))


_builtin_loaded = False


def _ensure_builtin() -> None:
    global _builtin_loaded
    if not _builtin_loaded:
        _builtin_loaded = True
        from .. import models  # noqa: F401  (registers the built-in architectures)
