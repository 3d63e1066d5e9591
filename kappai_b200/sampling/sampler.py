"""Sampling of a batch of rows on the device."""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..ops import kernels as K
from ..ops.build import load_library
from .params import SamplingParams
from .rng import uniform


def sample(logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int], indices: Sequence[int],
           recent: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
    """One token per row of ``logits`` [n, vocab] (float32, on the device).

    ``seeds[i]`` and ``indices[i]`` fix row i's uniform number (the request's
    resolved seed and how many tokens it has sampled before); ``recent[i]``
    holds the request's last tokens for the repeat penalty.  Returns int32 [n]
    on the device.  ``logits`` is changed in place where a penalty applies.
    """
    K._need(logits, "logits", torch.float32)
    n, V = logits.shape
    if not (len(params) == len(seeds) == len(indices) == n):
        raise K.KernelError("sample: one SamplingParams, seed and index per row")
    lib = load_library("sampling")
    dev = logits.device
    stream = K._stream()
    if any(p.repeat_penalty != 1.0 for p in params) and recent is not None:
        width = max(1, max(min(p.repeat_last_n, len(r)) for p, r in zip(params, recent)))
        rec = np.full((n, width), -1, np.int32)
        for i, (p, r) in enumerate(zip(params, recent)):
            m = min(p.repeat_last_n, len(r))
            if m > 0 and p.repeat_penalty != 1.0:
                rec[i, :m] = np.asarray(r[len(r) - m:], dtype=np.int64)
        rec_d = torch.from_numpy(rec).to(dev)
        pen_d = torch.tensor([p.repeat_penalty for p in params], dtype=torch.float32, device=dev)
        K._check(lib.kp_repeat_penalty(K._ptr(logits), n, V, K._ptr(rec_d), width, K._ptr(pen_d), stream),
                 "repeat_penalty")
    host = np.empty((n, 5), np.float32)
    for i, p in enumerate(params):
        p.validate(V)
        host[i] = (p.temperature, 0.0, p.top_p, p.min_p, 0.0 if p.greedy else uniform(seeds[i], indices[i]))
    f = torch.from_numpy(host).to(dev)
    topk = torch.tensor([p.top_k for p in params], dtype=torch.int32, device=dev)
    cols = f.t().contiguous()
    out = torch.empty(n, dtype=torch.int32, device=dev)
    K._check(lib.kp_sample_rows(K._ptr(logits), n, V, K._ptr(cols[0]), K._ptr(topk), K._ptr(cols[2]),
                                K._ptr(cols[3]), K._ptr(cols[4]), K._ptr(out), stream), "sample_rows")
    return out


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """Greedy tokens (lowest index on ties, src/sampler.c:125-136)."""
    n = logits.shape[0]
    g = SamplingParams(temperature=0.0)
    return sample(logits, [g] * n, [1] * n, [0] * n)
