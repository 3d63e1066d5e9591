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

    @staticmethod
    def _normed(norm, part, x):
        """A part that says it feeds its input straight into ``linear`` gets the
        norm as a lazy operand (it may then run inside the product kernel);
        any other part gets the normalised tensor."""
        if norm is None:
            return x
        if getattr(part, "accepts_normed_rows", False) and hasattr(norm, "lazy"):
            return norm.lazy(x)
        return norm.forward(x)

    def forward(self, x, ctx, cache):
        self.mixer.forward(self._normed(self.mixer_norm, self.mixer, x), x, ctx, cache)
        if self.ffn is not None:
            self.ffn.forward(self._normed(self.ffn_norm, self.ffn, x), x, ctx)


register_part("block", "prenorm_residual", PreNormResidualBlock)
