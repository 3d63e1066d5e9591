"""Device memory of the cache: page pools and state slots.

For a page group with ``L`` caches (one per schedule entry that keeps keys and
values in it) the pool is one tensor ``[L, n_pages, 2, G, page_size, hd]`` in
the compute dtype: page ``p`` exists in all ``L`` layers at once, so one block
table serves the whole group (the reference keeps ``[layer][kv head][pos][hd]``
per session, src/backend/cpu/common.c:1494-1601).  State of fixed size is one
tensor ``[n_slots, *shape]`` per schedule entry that keeps one.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Tuple

import torch

from .spec import PagedKVSpec, StateSpec


@dataclass
class KVLayerView:
    """One schedule entry's keys and values: ``tensor`` is
    [n_pages, 2, G, page_size, hd]; ``writes`` is False for an entry that only
    reads another entry's cache."""

    group: Hashable
    tensor: torch.Tensor
    writes: bool = True


@dataclass
class StateView:
    tensor: torch.Tensor           # [n_slots, *shape]
    writes: bool = True


class CacheStorage:
    def __init__(self, specs: List[Optional[object]], cache_of: List[Optional[int]], n_pages: Dict[Hashable, int],
                 page_size: int, n_slots: int, dtype: torch.dtype, device: torch.device):
        """``specs[i]`` is what schedule entry ``i`` asks for (None for an entry
        without a cache, or for one that borrows: ``cache_of[i]`` then names the
        lender).  ``n_pages`` gives the pool size of each page group."""
        self.page_size, self.n_slots = page_size, n_slots
        self.groups: Dict[Hashable, PagedKVSpec] = {}
        members: Dict[Hashable, List[int]] = {}
        for i, s in enumerate(specs):
            if isinstance(s, PagedKVSpec) and cache_of[i] is None:
                self.groups.setdefault(s.group_key, s)
                members.setdefault(s.group_key, []).append(i)
        self.pools: Dict[Hashable, torch.Tensor] = {}
        for gk, idx in members.items():
            s = self.groups[gk]
            self.pools[gk] = torch.zeros((len(idx), n_pages[gk], 2, s.num_kv_heads, page_size, s.head_dim),
                                         dtype=dtype, device=device)
        self.views: List[Optional[object]] = [None] * len(specs)
        for gk, idx in members.items():
            for j, i in enumerate(idx):
                self.views[i] = KVLayerView(gk, self.pools[gk][j], True)
        for i, s in enumerate(specs):
            if isinstance(s, StateSpec) and cache_of[i] is None:
                dt = getattr(torch, s.dtype)
                self.views[i] = StateView(torch.zeros((n_slots,) + tuple(s.shape), dtype=dt, device=device), True)
        for i, src in enumerate(cache_of):
            if src is not None:
                v = self.views[src]
                if v is None:
                    raise ValueError(f"schedule entry {i} borrows the cache of entry {src}, which keeps none")
                self.views[i] = (KVLayerView(v.group, v.tensor, False) if isinstance(v, KVLayerView)
                                 else StateView(v.tensor, False))

    def bytes_per_token(self, group: Hashable) -> int:
        t = self.pools[group]
        return t[:, 0, :, :, 0, :].numel() * t.element_size()

    def total_bytes(self) -> int:
        n = sum(t.numel() * t.element_size() for t in self.pools.values())
        for v in self.views:
            if isinstance(v, StateView) and v.writes:
                n += v.tensor.numel() * v.tensor.element_size()
        return n
