"""Arrangements of a mixer, a feed-forward and their norms around the residual.

``prenorm_residual``: ``x += mixer(norm1(x)); x += ffn(norm2(x))``
(src/models/lfm.c:7-53 followed by src/recipe/builders.c:378-388).  The
residual ``x`` is float32 and is updated in place.
"""
from __future__ import annotations

from .base import Part, register_part


class PreNormResidualBlock(Part):
    category = "block"
    graph_safe = True

    def assemble(self, mixer, ffn, mixer_norm, ffn_norm):
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm = mixer, ffn, mixer_norm, ffn_norm
        return self

    def forward(self, x, ctx, cache):
        self.mixer.forward(self.mixer_norm.forward(x) if self.mixer_norm is not None else x, x, ctx, cache)
        if self.ffn is not None:
            self.ffn.forward(self.ffn_norm.forward(x) if self.ffn_norm is not None else x, x, ctx)


register_part("block", "prenorm_residual", PreNormResidualBlock)
