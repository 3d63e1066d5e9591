"""Matrix products ``out = a @ w.T (+ bias)`` with W row-major [out, in].

One door for every product of the model; it picks the kernel by dtype and
shape: float32 operands always run the CUDA-core float32 kernel (the true
32-bit path); bfloat16 products of up to 16 rows run the weight-streaming
kernels (decode steps) except where the tcgen05 kernel was measured faster
(``kernels.tc_pays_for_few_rows``), larger ones the tcgen05 tensor-core kernel
(decode steps of 17 rows and more, where it cuts the product along K, and
prompt portions).  The product is this package's own kernel in every case;
no library matrix product is called.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import kernels as K


def linear(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
           accumulate: bool = False) -> torch.Tensor:
    """``out_dtype`` defaults to the operand dtype; ``accumulate`` adds into the
    float32 ``out`` (the residual sum stays in 32-bit)."""
    M, N = a.shape[0], w.shape[0]
    a_dtype = a.dtype
    if out is None:
        if accumulate:
            raise K.KernelError("linear: accumulate needs an output")
        out = torch.empty((M, N), dtype=out_dtype or a_dtype, device=a.device)
    if w.dtype != a.dtype:
        # a weight stored in 32-bit stays so: run that product in float32
        if w.dtype == torch.float32 and a.dtype == torch.bfloat16:
            a32 = K.cast(a.contiguous(), torch.empty(a.shape, dtype=torch.float32, device=a.device))
            if out.dtype == torch.float32:
                return K.gemm_nt_simt(a32, w, out, bias, accumulate)
            tmp = K.gemm_nt_simt(a32, w, torch.empty((M, N), dtype=torch.float32, device=a.device), bias)
            return K.cast(tmp, out)
        raise K.KernelError(f"linear: operand dtypes {a.dtype} and {w.dtype} do not go together")
    tc = K.tc_ok(a, w) and out.stride(1) == 1
    if K.skinny_ok(a, w) and not (tc and K.tc_pays_for_few_rows(M, N, False)):
        return K.gemm_skinny(a, w, out, bias, accumulate)
    if tc:
        return K.gemm_tc(a, w, out, bias, accumulate)
    return K.gemm_nt_simt(a, w, out, bias, accumulate)


def linear_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(a @ Wg.T) * (a @ Wu.T)`` with ``w_gate_up = [Wg; Wu]``; one fused
    kernel where there is one for the shape, else product then activation.
    Gate and up are rounded to the storage type before the activation either way."""
    ff = w_gate_up.shape[0] // 2
    act = torch.empty((a.shape[0], ff), dtype=a.dtype, device=a.device)
    tc = K.tc_ok(a, w_gate_up)
    if K.skinny_ok(a, w_gate_up) and not (tc and K.tc_pays_for_few_rows(a.shape[0], w_gate_up.shape[0], True)):
        return K.gemm_skinny(a, w_gate_up, act, bias, swiglu=True)
    if tc:
        return K.gemm_tc(a, w_gate_up, act, bias, swiglu=True)
    gu = linear(a, w_gate_up, bias)
    return K.swiglu(gu, act)
