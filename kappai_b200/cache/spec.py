"""What a mixer may ask of the cache manager.

Two kinds of per-request memory exist, as in the reference's hybrid cache
(src/kvcache.h:8-21,33-56: a KV region that grows with the position, and a
recurrent/conv state of fixed size per layer):

* :class:`PagedKVSpec` — keys and values that grow with the tokens; kept in
  pages.  Mixers with the same (kv heads, head dim, window) form a *group*
  that shares block tables; groups with different needs have pages of their
  own.
* :class:`StateSpec` — a fixed-size tensor per request; kept in a slot.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class PagedKVSpec:
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None      # keys older than this many positions are never read again

    @property
    def group_key(self) -> Tuple:
        return ("kv", self.num_kv_heads, self.head_dim, self.window)


@dataclass(frozen=True)
class StateSpec:
    shape: Tuple[int, ...]            # per request
    dtype: str = "float32"
