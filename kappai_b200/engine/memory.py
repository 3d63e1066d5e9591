"""How large the cache pools are made, decided before anything is allocated.

The reference refuses to run when the KV cache for the asked context does not
fit in what the device has free after the weights, with a sentence that gives
the figures (src/context.c:395-429,479-491).  Here the pools are paged and
shared by the requests, so there are two cases: a pool size that the caller
asked for (``kv_tokens``) either fits or is refused; a pool size left open is
made as large as the requests could ever use (``max_batch * ctx_size``) or as
the free memory allows, whichever is less, and refused only if not even one
request of ``ctx_size`` tokens would fit.

Plain arithmetic with no device call: the free-memory figure comes in as an
argument, so the decision is tested on any machine.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional


class CacheMemoryError(RuntimeError):
    pass


@dataclass
class GroupNeed:
    """One page group: bytes a token takes in all its layers, and its window (None: all keys are kept)."""

    key: Hashable
    bytes_per_token: int
    window: Optional[int] = None


@dataclass
class CachePlan:
    tokens: int                          # tokens the unwindowed pools hold
    pages: Dict[Hashable, int]           # pages of every group
    cache_bytes: int                     # pools and state slots together


MIB = 1024.0 * 1024.0


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def pages_of_group(g: GroupNeed, n_pages: int, page_size: int, n_slots: int, max_step_tokens: Optional[int]) -> int:
    """A windowed group never holds more than the window, the portion being run and the page both ends
    straddle for each request: a full pool for it would lie unused."""
    if g.window is None or max_step_tokens is None:
        return n_pages
    per_request = _ceil_div(g.window + max_step_tokens, page_size) + 1
    return max(1, min(n_pages, n_slots * per_request))


def plan_cache(groups: List[GroupNeed], state_bytes_per_slot: int, n_slots: int, page_size: int, ctx_size: int,
               asked_tokens: int, free_bytes: Optional[int], max_step_tokens: Optional[int] = None,
               reserve_fraction: float = 0.08, what: str = "") -> CachePlan:
    """``asked_tokens`` > 0: exactly that many tokens (rounded up to pages) or an error.  0: as many as
    ``n_slots`` requests of ``ctx_size`` tokens need, or as fit.  ``free_bytes``: what the device has free
    now, the weights already loaded (None: do not look; the asked or the full size is taken).
    ``reserve_fraction`` of the free memory is left for activations, scratch and captured graphs."""

    def cost(tokens: int):
        n_pages = max(1, _ceil_div(tokens, page_size))
        pages = {g.key: pages_of_group(g, n_pages, page_size, n_slots, max_step_tokens) for g in groups}
        kv = sum(pages[g.key] * page_size * g.bytes_per_token for g in groups)
        return pages, kv + n_slots * state_bytes_per_slot

    state = n_slots * state_bytes_per_slot
    usable = None if free_bytes is None else int(free_bytes * (1.0 - reserve_fraction))
    want = asked_tokens if asked_tokens > 0 else n_slots * ctx_size
    pages, need = cost(want)
    if usable is None or need <= usable:
        return CachePlan(max(1, _ceil_div(want, page_size)) * page_size, pages, need)
    figures = (f"{need / MIB:.1f} MB (keys and values of {want} tokens in {len(groups)} page group(s) at "
               f"{sum(g.bytes_per_token for g in groups)} B a token, and {state / MIB:.1f} MB of state for "
               f"{n_slots} slots) but only {usable / MIB:.1f} MB can be used of the {free_bytes / MIB:.1f} MB "
               f"that are free on the device after loading the weights")
    if asked_tokens > 0:
        raise CacheMemoryError(f"{what}the cache asked for needs {figures} -- refusing to run "
                               "(lower kv_tokens, ctx_size or max_batch)")
    # the size was left open: take what fits, if at least one request of ctx_size does
    lo, hi = 0, want                                   # largest token count whose cost fits (cost is monotone)
    while lo < hi:
        mid = (lo + hi + 1) // 2
        if cost(mid)[1] <= usable:
            lo = mid
        else:
            hi = mid - 1
    tokens = lo // page_size * page_size
    if tokens < min(ctx_size, want):
        raise CacheMemoryError(f"{what}a cache for {n_slots} requests of {ctx_size} tokens needs {figures}, and "
                               f"not even one request of {ctx_size} tokens fits -- refusing to run "
                               "(lower ctx_size or max_batch)")
    pages, need = cost(tokens)
    return CachePlan(tokens, pages, need)
