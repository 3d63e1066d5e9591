"""Sampling of a batch of rows on the device."""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from ..ops import kernels as K
from ..ops.build import load_library
from .params import SamplingParams
from .rng import uniform


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Greedy tokens, int32 [n] on the device (lowest index on ties,
    src/sampler.c:125-136).  Nothing is copied from the host."""
    K._need(logits, "logits", torch.float32)
    n, V = logits.shape
    if out is None:
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
    lib = load_library("sampling")
    scratch = torch.empty(n * 64, dtype=torch.int32, device=logits.device) if V >= 8192 else None
    K._run("argmax_rows", lib.kp_argmax_rows, K._ptr(logits), n, V, K._ptr(out), K._ptr(scratch), K.STREAM)
    return out


def sample(logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int], indices: Sequence[int],
           recent: Optional[Sequence[Sequence[int]]] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of ``logits`` [n, vocab] (float32, on the device).

    ``seeds[i]`` and ``indices[i]`` fix row i's uniform number (the request's
    resolved seed and how many tokens it has sampled before); ``recent[i]``
    holds the request's last tokens for the repeat penalty.  Returns int32 [n]
    on the device (``out`` if given).  ``logits`` is changed in place where a
    penalty applies.
    """
    K._need(logits, "logits", torch.float32)
    n, V = logits.shape
    if not (len(params) == len(seeds) == len(indices) == n):
        raise K.KernelError("sample: one SamplingParams, seed and index per row")
    for p in params:
        p.validate(V)
    penalised = recent is not None and any(p.repeat_penalty != 1.0 for p in params)
    if not penalised and all(p.greedy for p in params):
        return argmax(logits, out)
    lib = load_library("sampling")
    dev = logits.device
    # one pinned staging buffer: [n,5] floats, [n] top_k, then the recent tokens
    width = 0
    if penalised:
        width = max(1, max(min(p.repeat_last_n, len(r)) for p, r in zip(params, recent)))
    host = torch.empty(n * (6 + width), dtype=torch.int32, pin_memory=True)
    h = host.numpy()
    f = h[:n * 5].view(np.float32).reshape(5, n)
    for i, p in enumerate(params):
        f[0, i], f[1, i], f[2, i], f[3, i] = p.temperature, p.top_p, p.min_p, p.repeat_penalty
        f[4, i] = 0.0 if p.greedy else uniform(seeds[i], indices[i])
        h[n * 5 + i] = p.top_k
    if penalised:
        rec = h[n * 6:].reshape(n, width)
        rec[:] = -1
        for i, (p, r) in enumerate(zip(params, recent)):
            m = min(p.repeat_last_n, len(r))
            if m > 0 and p.repeat_penalty != 1.0:
                rec[i, :m] = np.asarray(r[len(r) - m:], dtype=np.int64)
    d = host.to(dev, non_blocking=True)
    fl = d[:n * 5].view(torch.float32)
    col = lambda j: K._ptr(fl[j * n:(j + 1) * n])
    if penalised:
        K._run("repeat_penalty", lib.kp_repeat_penalty, K._ptr(logits), n, V, K._ptr(d[n * 6:]), width, col(3), K.STREAM)
    if out is None:
        out = torch.empty(n, dtype=torch.int32, device=dev)
    K._need(out, "out", torch.int32)
    K._run("sample_rows", lib.kp_sample_rows, K._ptr(logits), n, V, col(0), K._ptr(d[n * 5:n * 6]), col(1), col(2), col(4),
           K._ptr(out), K.STREAM)
    out._staging = host           # keep the pinned buffer alive until the copy has run
    return out
