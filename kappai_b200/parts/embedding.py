"""Token embedding and the output head.

``x[r,:] = E[token[r],:]`` (times ``scale`` if the architecture has one;
src/recipe/scratch.c:195-235), into the float32 residual.  The head computes
``logits = h W^T`` in float32 output; when tied, W is the embedding table
(src/model.c:2562-2572).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels as K
from ..ops.linear import linear
from .base import Part, WeightSpec, register_part


class TokenEmbedding(Part):
    category = "embedding"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.V = int(self._p("vocab_size"))
        self.d = int(self._p("hidden_size"))
        s = self._p("scale", None)
        self.scale = 1.0 if s is None else float(s)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.V, self.d), "embedding")}

    def bind(self, w):
        self.weight = w["weight"].contiguous()

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        x = torch.empty((token_ids.numel(), self.d), dtype=torch.float32, device=token_ids.device)
        return K.embed_rows(self.weight, token_ids, x, self.scale)


class LMHead(Part):
    category = "head"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.V = int(self._p("vocab_size"))
        self.d = int(self._p("hidden_size"))
        self.tied = bool(self._p("tied", True))
        self.weight = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {} if self.tied else {"weight": WeightSpec((self.V, self.d), "matrix")}

    def bind(self, w):
        if not self.tied:
            self.weight = w["weight"].contiguous()

    def tie(self, embedding: TokenEmbedding) -> None:
        self.weight = embedding.weight

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return linear(h, self.weight, out_dtype=torch.float32)


register_part("embedding", "embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
