"""RMSNorm over the rows of the residual.

``y = (x * rsqrt(mean(x^2) + eps)) * w`` with float32 statistics
(src/backend/cpu/scalar/quants.c:1489-1512).  The input is the float32
residual; the output has the compute dtype (it feeds a matrix product).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import kernels as K
from .base import Part, WeightSpec, register_part


class RMSNorm(Part):
    category = "norm"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.size = int(self._p("size"))
        self.eps = float(self._p("eps"))
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.size,), "norm")}

    def bind(self, w):
        self.weight = w["weight"].to(torch.float32).contiguous()

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=self.env.dtype, device=x.device)
        return K.rmsnorm_rows(x, self.weight, self.eps, out, rows)


register_part("norm", "rmsnorm", RMSNorm)
