"""The random numbers of sampling.

The reference gives each session a generator seeded by splitmix64 and draws a
24-bit uniform per sampled token (src/sampler.c:13-32).  Here the uniform of a
request's ``i``-th sampled token is a pure function of (seed, i): splitmix64
of ``splitmix64(seed) + i``, top 24 bits.  So a request's draws do not depend
on what else is in the batch, on preemption, or on the order of steps.
"""
from __future__ import annotations

import os

_M = (1 << 64) - 1


def splitmix64(x: int) -> int:
    z = (x + 0x9E3779B97F4A7C15) & _M
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M
    return z ^ (z >> 31)


def resolve_seed(seed: int) -> int:
    """Seed 0 means "random" (src/sampler.c:34-50)."""
    if seed == 0:
        seed = int.from_bytes(os.urandom(8), "little") or 0xDEADBEEFCAFEBABE
    return seed & _M


def uniform(seed: int, index: int) -> float:
    """A float in [0, 1) with 24 random bits."""
    z = splitmix64((splitmix64(seed & _M) + index) & _M)
    return (z >> 40) * (1.0 / (1 << 24))
