"""kappai_b200 — a small, whole inference engine for one GPU (B200, sm_100a).

Everything between a request's tokens and its next token: typed configuration
and an architecture registry, weights from safetensors, layers put together
from parts, a paged cache manager with per-request state slots, one step
function for mixed batches, a scheduler, samplers, and hand-written CUDA
kernels below.

Entry points: :class:`Engine` / :class:`EngineArgs` (Python),
``engine_init`` / ``engine_run`` / ``engine_shutdown`` and
``python -m kappai_b200.cli`` (command line), ``bin/trace_run`` (trace replay).
"""
__version__ = "0.1.0"

_LAZY = {
    "Engine": ("kappai_b200.engine.engine", "Engine"),
    "EngineArgs": ("kappai_b200.engine.engine", "EngineArgs"),
    "ModelRunner": ("kappai_b200.engine.runner", "ModelRunner"),
    "StepEntry": ("kappai_b200.engine.runner", "StepEntry"),
    "SamplingParams": ("kappai_b200.sampling.params", "SamplingParams"),
    "engine_init": ("kappai_b200.cli", "engine_init"),
    "engine_run": ("kappai_b200.cli", "engine_run"),
    "engine_shutdown": ("kappai_b200.cli", "engine_shutdown"),
    "write_random_model": ("kappai_b200.weights.random_init", "write_random_model"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib

        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod), attr)
    raise AttributeError(f"module 'kappai_b200' has no attribute '{name}'")
