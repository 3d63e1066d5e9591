"""Gated short convolution (the LFM2 conv mixer).

``p = h Win^T`` split as B | C | X (each hidden_size wide, in this order:
src/backend/cpu/common.c:2401-2403); ``bx = B*X``; a causal depthwise
convolution of length ``kernel_size`` over ``bx`` along the sequence whose last
tap multiplies the current token; ``out = C * y``; ``a = out Wout^T`` added to
the residual (src/models/lfm.c:7-21, src/backend/cpu/common.c:2393-2431).  The
previous ``kernel_size - 1`` values of ``bx`` are the request's state, zero at
a sequence's start (src/recipe/ops_hybrid.c:353-354).  With ``bias`` the two
products and the convolution each add a bias (the convolution's before the C
gate).

Params: hidden_size, kernel_size, bias.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache.spec import StateSpec
from ..config.schema import ConfigError
from ..ops import kernels as K
from ..ops.linear import linear
from .base import Part, WeightSpec, register_part

MAX_KERNEL = 16


class ShortConv(Part):
    category = "mixer"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.d = int(self._p("hidden_size"))
        self.K = int(self._p("kernel_size"))
        self.bias = bool(self._p("bias", False))
        self.fuse_step = True           # decode steps of few rows: conv step in in_proj's epilogue where the kernel takes it
        if not (2 <= self.K <= MAX_KERNEL):
            raise ConfigError(f"shortconv: kernel_size={self.K} outside 2..{MAX_KERNEL}")

    def weight_specs(self) -> Dict[str, WeightSpec]:
        d = self.d
        s = {"in_proj.weight": WeightSpec((3 * d, d)), "conv.weight": WeightSpec((d, 1, self.K), "conv"),
             "out_proj.weight": WeightSpec((d, d))}
        if self.bias:
            s["in_proj.bias"] = WeightSpec((3 * d,), "bias")
            s["conv.bias"] = WeightSpec((d,), "bias")
            s["out_proj.bias"] = WeightSpec((d,), "bias")
        return s

    def bind(self, w):
        self.w_in = w["in_proj.weight"].contiguous()
        self.w_out = w["out_proj.weight"].contiguous()
        self.w_conv = w["conv.weight"].float().reshape(self.d, self.K).contiguous()
        self.b_in = self.b_conv = self.b_out = None
        if self.bias:
            self.b_in = w["in_proj.bias"].float().contiguous()
            self.b_conv = w["conv.bias"].float().contiguous()
            self.b_out = w["out_proj.bias"].float().contiguous()

    def cache_spec(self):
        return StateSpec((self.K - 1, self.d), "float32")

    def forward(self, h, residual, ctx, cache):
        """``cache``: a :class:`~kappai_b200.cache.storage.StateView` with tensor
        [n_slots, kernel_size - 1, hidden_size] float32."""
        if (ctx.decode_only and cache.writes and h.dtype == torch.bfloat16 and self.fuse_step
                and K.conv_step_fusable(h, self.w_in, self.K)):
            # a decode step of few rows: the conv step runs in in_proj's epilogue (one launch less a layer)
            y = torch.empty((ctx.n_rows, self.d), dtype=h.dtype, device=h.device)
            K.gemm_stream_conv_step(h, self.w_in, self.b_in, self.w_conv, self.b_conv, cache.tensor, ctx.seg_pos,
                                    ctx.seg_slot, y)
            linear(y, self.w_out, self.b_out, out=residual, accumulate=True)
            return
        p = linear(h, self.w_in, self.b_in)
        y = torch.empty((ctx.n_rows, self.d), dtype=p.dtype, device=p.device)
        if ctx.decode_only and cache.writes:
            K.shortconv_decode(p, self.w_conv, self.b_conv, cache.tensor, ctx.seg_pos, ctx.seg_slot, y)
        else:
            K.shortconv_forward(p, self.w_conv, self.b_conv, cache.tensor, ctx.row_seg, ctx.cu_rows, ctx.seg_pos,
                                ctx.seg_slot, y)
            if cache.writes:
                K.shortconv_update_state(p, cache.tensor, ctx.cu_rows, ctx.seg_pos, ctx.seg_slot, ctx.n_seg)
        linear(y, self.w_out, self.b_out, out=residual, accumulate=True)


register_part("mixer", "shortconv", ShortConv)
