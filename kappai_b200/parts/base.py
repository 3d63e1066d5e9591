"""Interfaces of the parts a layer is put together from, and their registry.

A part is built from a :class:`~kappai_b200.config.schema.PartSpec` (its
registry kind plus sizes and constants) and a :class:`BuildEnv` (device, the
compute dtype, the longest position the engine will run).  It declares the
tensors it binds under local names, gets them at load, and runs on the rows of
a step.  No part knows which model it is in; the architecture file chooses the
parts layer by layer.

Categories and what each must offer
-----------------------------------
any             optionally ``step_tables_key`` and ``step_tables(segs)``: int32
                  tables built on the host for every step (see :class:`Part`).
``mixer``         ``cache_spec()`` -> PagedKVSpec | StateSpec | None;
                  ``forward(h, residual, ctx, cache)`` adds its output (float32)
                  into ``residual`` in place.  It must restart at every
                  segment of the batch, read its request's cache/state at the
                  segment's head and leave it updated at its end, and accept
                  segments of one row.
``feed_forward``  ``forward(h, residual, ctx)`` adds into ``residual``.
``norm``          ``forward(x, rows=None)`` -> normalised rows in the compute
                  dtype (``rows`` picks rows of ``x`` first).
``position``      either ``fused_rotary()`` -> (cos, sin, rotary_dim,
                  interleaved) for the fused q/k kernel, or ``apply(q, k, ctx)``.
``block``         ``forward(x, ctx, cache)``: the arrangement of the above
                  around the float32 residual ``x``.
``embedding`` / ``head``  token ids -> residual rows; selected rows -> logits.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Optional, Tuple

import torch

from ..config.schema import ConfigError, PartSpec


@dataclass
class WeightSpec:
    """One tensor a part binds.  ``role`` picks the random-weights
    distribution and the storage dtype of a written model folder:
    ``matrix`` / ``embedding`` (bfloat16), ``norm`` / ``conv`` / ``bias``
    (float32)."""

    shape: Tuple[int, ...]
    role: str = "matrix"
    optional: bool = False


@dataclass
class BuildEnv:
    device: torch.device
    dtype: torch.dtype                  # compute dtype: torch.bfloat16 or torch.float32
    max_positions: int                  # positions 0..max_positions-1 may be run
    shared: Dict[Any, Any] = field(default_factory=dict)   # tables shared between parts (e.g. rotary)


class Part:
    category = "part"
    # True if forward() reads the step's tables from the device tensors of the context only (never from
    # its host_* lists or other host values that change from step to step): such a part can be captured
    # in a CUDA graph.  Parts registered from outside are not assumed to be.
    graph_safe = False

    def __init__(self, params: Dict[str, Any], env: BuildEnv):
        self.params = dict(params)
        self.env = env

    # Step tables.  A part whose kernels need host-built int32 tables for every step (tile lists, scan
    # boundaries, rows per expert...) names them here: ``step_tables_key`` (hashable; parts with equal keys
    # share one set of tables) and ``step_tables(segs)``, which gets the step's segments on the host
    # (``engine.batch.StepSegments``) and returns an ``engine.batch.PartTables`` (or None for a step that
    # needs none).  The arrays travel in the step's one upload and show up as ``ctx.tables[key].<name>``.
    # In a captured decode step the arrays live in the graph's static buffer and are refilled before every
    # replay; their sizes must then depend on the number of requests only.
    step_tables_key = None

    def step_tables(self, segs):
        return None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {}

    def bind(self, w: Dict[str, torch.Tensor]) -> None:
        """Receive the tensors named by :meth:`weight_specs` (on the device, in
        the compute dtype for 16-bit stored tensors, float32 for 32-bit ones)."""

    # helpers for subclasses
    def _p(self, name: str, default: Any = ...):
        if name in self.params:
            return self.params[name]
        if default is ...:
            raise ConfigError(f"part '{type(self).__name__}': missing parameter '{name}'")
        return default


_REGISTRY: Dict[Tuple[str, str], Callable[..., Part]] = {}
CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")


def register_part(category: str, kind: str, factory: Callable[..., Part], *, replace: bool = False) -> None:
    if category not in CATEGORIES:
        raise ConfigError(f"unknown part category '{category}' (one of {', '.join(CATEGORIES)})")
    if (category, kind) in _REGISTRY and not replace:
        raise ConfigError(f"{category} '{kind}' is already registered")
    _REGISTRY[(category, kind)] = factory


def unregister_part(category: str, kind: str) -> None:
    _REGISTRY.pop((category, kind), None)


def make_part(category: str, spec: PartSpec, env: BuildEnv) -> Part:
    _ensure_builtin()
    try:
        factory = _REGISTRY[(category, spec.kind)]
    except KeyError:
        known = ", ".join(sorted(k for c, k in _REGISTRY if c == category)) or "(none)"
        raise ConfigError(f"no {category} of kind '{spec.kind}' is registered (known: {known})") from None
    return factory(spec.params, env)


def part_kinds(category: str):
    _ensure_builtin()
    return sorted(k for c, k in _REGISTRY if c == category)


_builtin = False


def _ensure_builtin() -> None:
    global _builtin
    if not _builtin:
        _builtin = True
        from . import norm, position, attention, shortconv, ffn, block, embedding  # noqa: F401
