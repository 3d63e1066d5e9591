"""SwiGLU feed-forward.

``f = (silu(h Wg^T) * (h Wu^T)) Wd^T`` added to the residual; gate and up run
as one product against [Wg; Wu], gate rows first (src/recipe/builders.c:344-388,
src/model.c:1575-1610); ``silu(g) = g / (1 + exp(-g))``
(src/backend/cpu/quants.h:369-371).

Params: hidden_size, intermediate_size, bias.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels as K
from ..ops.linear import linear, linear_swiglu
from .base import Part, WeightSpec, register_part


class SwiGLU(Part):
    category = "feed_forward"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.d = int(self._p("hidden_size"))
        self.ff = int(self._p("intermediate_size"))
        self.bias = bool(self._p("bias", False))

    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = {"gate_proj.weight": WeightSpec((self.ff, self.d)), "up_proj.weight": WeightSpec((self.ff, self.d)),
             "down_proj.weight": WeightSpec((self.d, self.ff))}
        if self.bias:
            s["gate_proj.bias"] = WeightSpec((self.ff,), "bias")
            s["up_proj.bias"] = WeightSpec((self.ff,), "bias")
            s["down_proj.bias"] = WeightSpec((self.d,), "bias")
        return s

    def bind(self, w):
        self.w_gu = torch.cat([w["gate_proj.weight"], w["up_proj.weight"]], 0).contiguous()
        self.w_down = w["down_proj.weight"].contiguous()
        self.b_gu = self.b_down = None
        if self.bias:
            self.b_gu = torch.cat([w["gate_proj.bias"].float(), w["up_proj.bias"].float()]).contiguous()
            self.b_down = w["down_proj.bias"].float().contiguous()

    def forward(self, h, residual, ctx):
        act = linear_swiglu(h, self.w_gu, self.b_gu)
        linear(act, self.w_down, self.b_down, out=residual, accumulate=True)


register_part("feed_forward", "swiglu", SwiGLU)
