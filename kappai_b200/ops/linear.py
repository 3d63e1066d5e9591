"""Matrix products ``out = a @ w.T (+ bias)`` with W row-major [out, in].

One door for every product of the model; it picks the kernel by dtype and
shape: float32 operands always run the CUDA-core float32 kernel (the true
32-bit path); bfloat16 products of up to 64 rows run the weight-streaming
kernels (decode steps) except where the tcgen05 kernel was measured faster
(``kernels.tc_pays_for_few_rows``), larger ones the tcgen05 tensor-core kernel
(prompt portions).  The product is this package's own kernel in every case;
no library matrix product is called.

The left operand may be a :class:`NormedRows`: "the RMSNorm of these float32
rows", not yet computed.  Where a kernel can take the norm in front of the
product (few rows, bfloat16) nothing is materialised; otherwise the normalised
rows are computed once, kept, and used as an ordinary operand.
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from . import kernels as K


class NormedRows:
    """RMSNorm of (some rows of) the float32 residual, computed when needed."""

    def __init__(self, x: torch.Tensor, weight: torch.Tensor, eps: float, dtype: torch.dtype,
                 rows: Optional[torch.Tensor] = None):
        self.x, self.weight, self.eps, self.dtype, self.rows = x, weight, eps, dtype, rows
        self._h: Optional[torch.Tensor] = None

    @property
    def shape(self):
        return (self.x.shape[0] if self.rows is None else self.rows.numel(), self.x.shape[1])

    @property
    def device(self):
        return self.x.device

    def tensor(self) -> torch.Tensor:
        """The normalised rows as a tensor of the compute dtype (computed once)."""
        if self._h is None:
            out = torch.empty(self.shape, dtype=self.dtype, device=self.x.device)
            self._h = K.rmsnorm_rows(self.x, self.weight, self.eps, out, self.rows)
        return self._h


Operand = Union[torch.Tensor, NormedRows]


def as_tensor(a: Operand) -> torch.Tensor:
    return a.tensor() if isinstance(a, NormedRows) else a


# Whether few-row products take the norm in front of them.  Every CTA of the fused kernel recomputes the
# rows' scales, which on B200 costs more than the separate norm kernel it saves once a product has more
# than a few hundred CTAs (measured: in_proj 9.7 us fused against 4.3 + 5.3 us, the head 82 against 48 us),
# so it is off; the path stays for shapes where it pays and is covered by the kernel tests.
FUSE_NORM = False


def _fusable(a: Operand, w: torch.Tensor) -> bool:
    return (FUSE_NORM and isinstance(a, NormedRows) and a._h is None and a.dtype == torch.bfloat16
            and K.skinny_norm_ok(a.x, a.shape[0], w))


def linear(a: Operand, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
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
    if _fusable(a, w):
        return K.gemm_skinny_norm(a.x, a.weight, a.eps, a.rows, w, out, bias, accumulate)
    a = as_tensor(a)
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


def linear_swiglu(a: Operand, w_gate_up: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(a @ Wg.T) * (a @ Wu.T)`` with ``w_gate_up = [Wg; Wu]``; one fused
    kernel where there is one for the shape, else product then activation.
    Gate and up are rounded to the storage type before the activation either way."""
    ff = w_gate_up.shape[0] // 2
    act = torch.empty((a.shape[0], ff), dtype=a.dtype, device=a.device)
    if _fusable(a, w_gate_up):
        return K.gemm_skinny_norm(a.x, a.weight, a.eps, a.rows, w_gate_up, act, bias, swiglu=True)
    a = as_tensor(a)
    tc = K.tc_ok(a, w_gate_up)
    if K.skinny_ok(a, w_gate_up) and not (tc and K.tc_pays_for_few_rows(a.shape[0], w_gate_up.shape[0], True)):
        return K.gemm_skinny(a, w_gate_up, act, bias, swiglu=True)
    if tc:
        return K.gemm_tc(a, w_gate_up, act, bias, swiglu=True)
    gu = linear(a, w_gate_up, bias)
    return K.swiglu(gu, act)
