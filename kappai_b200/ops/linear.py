"""Matrix products ``out = a @ w.T (+ bias)`` with W row-major [out, in].

One door for every product of the model; it picks the kernel by dtype and
shape: float32 operands always run the CUDA-core float32 kernel (the true
32-bit path); bfloat16 products of up to 64 rows run the weight-streaming
kernel (decode steps).  The product is this package's own kernel in every case; no
library matrix product is called.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import kernels as K


def linear(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
           accumulate: bool = False) -> torch.Tensor:
    """``out_dtype`` defaults to ``a.dtype``; ``accumulate`` adds into the
    float32 ``out`` (the residual sum stays in 32-bit)."""
    M, N = a.shape[0], w.shape[0]
    if out is None:
        if accumulate:
            raise K.KernelError("linear: accumulate needs an output")
        out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
    if w.dtype != a.dtype:
        # a weight stored in 32-bit stays so: run that product in float32
        if w.dtype == torch.float32 and a.dtype == torch.bfloat16:
            a32 = K.cast(a.contiguous(), torch.empty(a.shape, dtype=torch.float32, device=a.device))
            if out.dtype == torch.float32:
                return K.gemm_nt_simt(a32, w, out, bias, accumulate)
            tmp = K.gemm_nt_simt(a32, w, torch.empty((M, N), dtype=torch.float32, device=a.device), bias)
            return K.cast(tmp, out)
        raise K.KernelError(f"linear: operand dtypes {a.dtype} and {w.dtype} do not go together")
    if K.skinny_ok(a, w):
        return K.gemm_skinny(a, w, out, bias, accumulate)
    return K.gemm_nt_simt(a, w, out, bias, accumulate)


def linear_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(a @ Wg.T) * (a @ Wu.T)`` with ``w_gate_up = [Wg; Wu]``; one fused
    kernel where there is one for the shape, else product then activation.
    Gate and up are rounded to the storage type before the activation either way."""
    ff = w_gate_up.shape[0] // 2
    act = torch.empty((a.shape[0], ff), dtype=a.dtype, device=a.device)
    if K.skinny_ok(a, w_gate_up):
        return K.gemm_skinny(a, w_gate_up, act, bias, swiglu=True)
    gu = linear(a, w_gate_up, bias)
    return K.swiglu(gu, act)
