"""kappai_b200 — a small, whole inference engine for one GPU (B200, sm_100a).

Everything between a request's tokens and its next token: typed configuration
and an architecture registry, weights from safetensors, layers put together
from parts, a paged cache manager with per-request state slots, one step
function for mixed batches, a scheduler, samplers, and hand-written CUDA
kernels below.
"""
__version__ = "0.1.0"
