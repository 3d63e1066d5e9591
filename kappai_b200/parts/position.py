"""Position encodings of a mixer.

``rope``: rotary encoding.  The angle table is built on the host in double
precision, ``angle = pos * theta^(-2j/rotary_dim)``, and stored as float32
cos/sin ``[max_positions, rotary_dim/2]`` (src/compute.c:22-65; the reference
shares one table between all layers with the same sizes, src/compute.c:80-102,
and so does this).  ``pairing`` is ``neox`` (j, j + rotary_dim/2) or
``interleaved`` (2j, 2j+1) (src/backend/cpu/scalar/core.c:66-84); ``rotary_dim``
may be smaller than the head size (the rest of the head is left as it is).

``none``: no rotation.
"""
from __future__ import annotations

import numpy as np
import torch

from ..config.schema import ConfigError
from .base import Part, register_part


class RotaryEncoding(Part):
    category = "position"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.rotary_dim = int(self._p("rotary_dim"))
        self.theta = float(self._p("theta"))
        pairing = self._p("pairing", "neox")
        if pairing not in ("neox", "interleaved"):
            raise ConfigError(f"rope: pairing '{pairing}' (expected 'neox' or 'interleaved')")
        if self.rotary_dim < 2 or self.rotary_dim % 2:
            raise ConfigError(f"rope: rotary_dim={self.rotary_dim} must be even and positive")
        self.interleaved = pairing == "interleaved"
        key = ("rope", self.rotary_dim, self.theta, env.max_positions)
        if key not in env.shared:
            half = self.rotary_dim // 2
            inv = np.power(self.theta, -2.0 * np.arange(half, dtype=np.float64) / self.rotary_dim)
            ang = np.arange(env.max_positions, dtype=np.float64)[:, None] * inv[None, :]
            env.shared[key] = (torch.from_numpy(np.cos(ang).astype(np.float32)).to(env.device),
                               torch.from_numpy(np.sin(ang).astype(np.float32)).to(env.device))
        self.cos, self.sin = env.shared[key]

    def fused_rotary(self):
        return self.cos, self.sin, self.rotary_dim, self.interleaved


class NoPosition(Part):
    category = "position"
    graph_safe = True

    def fused_rotary(self):
        return None, None, 0, False


register_part("position", "rope", RotaryEncoding)
register_part("position", "none", NoPosition)
