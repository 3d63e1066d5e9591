"""Host side of the cache: who holds which page and which state slot.

The reference keeps one contiguous KV region per session and a per-session
conv-state array (src/kvcache.c:166-314, hybrid part :208-237) and gives
nothing back before the session ends.  Here keys and values live in pages:
each group of layers with the same needs has a pool of pages and, for every
request, a block table (logical block -> page).  Pages return to the pool
when the request ends or, in a windowed group, when the window has passed
them; returned pages are handed out again.  Fixed-size per-request state lives
in slots of a slot pool.

This module is plain Python with no device code, so its bookkeeping can be
tested anywhere.  ``cache.storage`` holds the device tensors that the page and
slot numbers index.
"""
from __future__ import annotations

import numpy as np
from typing import Dict, Hashable, List, Optional

RELEASED = -1     # block-table entry of a page that the window has passed


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    pass


class OutOfSlots(CacheError):
    pass


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


class PagePool:
    """Pages of one layer group."""

    def __init__(self, n_pages: int, page_size: int, window: Optional[int] = None):
        if n_pages < 1 or page_size < 1:
            raise CacheError("a page pool needs at least one page and a positive page size")
        if window is not None and window < 1:
            raise CacheError("window must be positive")
        self.n_pages, self.page_size, self.window = n_pages, page_size, window
        self._free: List[int] = list(range(n_pages - 1, -1, -1))      # stack: lowest page first
        self._tables: Dict[Hashable, List[int]] = {}
        self._held: Dict[Hashable, int] = {}                          # pages currently held per request
        self._version: Dict[Hashable, int] = {}                       # stamp of the last change of a request's table
        self._tick = 0                                                # source of the stamps: never repeats
        self._used_before = [False] * n_pages
        self.n_handed_out = 0                                         # pages given to requests so far
        self.n_reused = 0                                             # of those, pages that another table held before

    # -- queries
    @property
    def n_free(self) -> int:
        return len(self._free)

    def table(self, req: Hashable) -> List[int]:
        return self._tables[req]

    def version(self, req: Hashable) -> int:
        """A stamp that changes whenever the request's block table does (a page added or
        released) and is never used twice in this pool, not even by a later request of
        the same name: a copy of the table elsewhere knows by it when it is stale."""
        return self._version[req]

    def pages_needed(self, req: Hashable, new_len: int) -> int:
        have = len(self._tables.get(req, ()))
        return max(0, _ceil_div(new_len, self.page_size) - have)

    # -- changes
    def _stamp(self) -> int:
        self._tick += 1
        return self._tick

    def open(self, req: Hashable) -> None:
        if req in self._tables:
            raise CacheError(f"request {req!r} already has a block table")
        self._tables[req] = []
        self._held[req] = 0
        self._version[req] = self._stamp()

    def extend(self, req: Hashable, new_len: int) -> None:
        """Make the table cover tokens [0, new_len)."""
        need = self.pages_needed(req, new_len)
        if need > len(self._free):
            raise OutOfPages(f"need {need} pages, {len(self._free)} free")
        if need == 0:
            return
        t = self._tables[req]
        for _ in range(need):
            page = self._free.pop()
            self.n_handed_out += 1
            self.n_reused += self._used_before[page]
            self._used_before[page] = True
            t.append(page)
        self._held[req] += need
        self._version[req] = self._stamp()

    def release_behind(self, req: Hashable, next_pos: int) -> int:
        """Windowed groups: give back pages whose every key lies before the
        window of position ``next_pos`` (the next token to run) and hence of
        all later ones.  Returns the number of pages released."""
        if self.window is None:
            return 0
        first_needed = next_pos - self.window + 1
        if first_needed <= 0:
            return 0
        t = self._tables[req]
        n = 0
        for b in range(min(first_needed // self.page_size, len(t))):
            if t[b] != RELEASED:
                self._free.append(t[b])
                t[b] = RELEASED
                n += 1
        if n:
            self._held[req] -= n
            self._version[req] = self._stamp()
        return n

    def close(self, req: Hashable) -> None:
        t = self._tables.pop(req, None)
        if t is None:
            raise CacheError(f"request {req!r} has no block table (freed twice?)")
        for p in t:
            if p != RELEASED:
                self._free.append(p)
        del self._held[req]
        del self._version[req]

    def check(self) -> None:
        """Every page is either free or held by exactly one block table."""
        seen = {}
        for p in self._free:
            if p in seen:
                raise CacheError(f"page {p} is in the free list twice")
            seen[p] = "free"
        for r, t in self._tables.items():
            held = 0
            for p in t:
                if p == RELEASED:
                    continue
                held += 1
                if p in seen:
                    raise CacheError(f"page {p} held by {r!r} is also {seen[p]!r}")
                seen[p] = r
            if held != self._held[r]:
                raise CacheError(f"request {r!r}: held count {self._held[r]} != {held}")
        if len(seen) != self.n_pages or any(not (0 <= p < self.n_pages) for p in seen):
            raise CacheError(f"{self.n_pages - len(seen)} pages lost")


class SlotPool:
    """Slots of fixed-size per-request state."""

    def __init__(self, n_slots: int):
        if n_slots < 1:
            raise CacheError("a slot pool needs at least one slot")
        self.n_slots = n_slots
        self._free: List[int] = list(range(n_slots - 1, -1, -1))
        self._owner: Dict[int, Hashable] = {}

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self, req: Hashable) -> int:
        if not self._free:
            raise OutOfSlots("no state slot free")
        s = self._free.pop()
        self._owner[s] = req
        return s

    def give_back(self, slot: int) -> None:
        if slot not in self._owner:
            raise CacheError(f"slot {slot} is not held (freed twice?)")
        del self._owner[slot]
        self._free.append(slot)

    def check(self) -> None:
        if len(set(self._free)) != len(self._free) or set(self._free) & set(self._owner):
            raise CacheError("a slot is free twice or free and held")
        if len(self._free) + len(self._owner) != self.n_slots:
            raise CacheError("a slot is lost")


class RequestCache:
    """What one live request holds."""

    __slots__ = ("req", "slot", "length")

    def __init__(self, req: Hashable, slot: int):
        self.req, self.slot, self.length = req, slot, 0


class CacheManager:
    """All page groups and the slot pool of one engine.

    ``groups`` maps a group key to ``(n_pages, page_size, window)``.  Each
    request gets one slot (used by every state-holding layer) and one block
    table per group.
    """

    def __init__(self, groups: Dict[Hashable, tuple], n_slots: int):
        self.pools: Dict[Hashable, PagePool] = {k: PagePool(*v) for k, v in groups.items()}
        self.slots = SlotPool(n_slots)
        self.requests: Dict[Hashable, RequestCache] = {}

    # -- admission
    def can_admit(self) -> bool:
        return self.slots.n_free > 0

    def admit(self, req: Hashable) -> RequestCache:
        if req in self.requests:
            raise CacheError(f"request {req!r} is already live")
        rc = RequestCache(req, self.slots.take(req))
        for p in self.pools.values():
            p.open(req)
        self.requests[req] = rc
        return rc

    # -- growth
    def can_extend(self, req: Hashable, new_len: int) -> bool:
        return all(p.pages_needed(req, new_len) <= p.n_free for p in self.pools.values())

    def extend(self, req: Hashable, new_len: int) -> None:
        """Pages for tokens [0, new_len) in every group, or none at all."""
        if req not in self.requests:
            raise CacheError(f"request {req!r} is not live")
        if not self.try_extend(req, new_len):
            raise OutOfPages(f"request {req!r}: no pages for {new_len} tokens")

    def try_extend(self, req: Hashable, new_len: int) -> bool:
        """:meth:`extend` that answers False (and takes nothing) where it would raise OutOfPages."""
        pools = self.pools.values()
        needs = [p.pages_needed(req, new_len) for p in pools]
        if not any(needs):
            return True
        if any(n > p.n_free for n, p in zip(needs, pools)):
            return False
        for p in pools:
            p.extend(req, new_len)
        return True

    def advance(self, req: Hashable, new_len: int) -> None:
        """The request now holds ``new_len`` tokens; release what windows have passed."""
        rc = self.requests[req]
        if new_len < rc.length:
            raise CacheError("a request's length cannot shrink")
        rc.length = new_len
        for p in self.pools.values():
            p.release_behind(req, new_len)

    # -- end
    def free(self, req: Hashable) -> None:
        rc = self.requests.pop(req, None)
        if rc is None:
            raise CacheError(f"request {req!r} is not live (freed twice?)")
        for p in self.pools.values():
            p.close(req)
        self.slots.give_back(rc.slot)

    # -- views for the step function
    def block_table(self, req: Hashable, group: Hashable) -> List[int]:
        return self.pools[group].table(req)

    def token_slots(self, req: Hashable, group: Hashable, start: int, n: int) -> List[int]:
        """Physical token slot (page * page_size + offset) of positions start..start+n-1."""
        pool = self.pools[group]
        t, ps = pool.table(req), pool.page_size
        if n > 32:
            # a prompt portion: by arrays (a Python loop over 2048 positions costs 0.3 ms a step and page group)
            pos = np.arange(start, start + n)
            pages = np.asarray(t[start // ps:(start + n - 1) // ps + 1], dtype=np.int64)[pos // ps - start // ps]
            if (pages == RELEASED).any():
                bad = int(pos[pages == RELEASED][0])
                raise CacheError(f"position {bad} of {req!r} lies in a released page")
            return (pages * ps + pos % ps).tolist()
        out = []
        for pos in range(start, start + n):
            page = t[pos // ps]
            if page == RELEASED:
                raise CacheError(f"position {pos} of {req!r} lies in a released page")
            out.append(page * ps + pos % ps)
        return out

    def check(self) -> None:
        for p in self.pools.values():
            p.check()
        self.slots.check()
        for p in self.pools.values():
            if set(p._tables) != set(self.requests):
                raise CacheError("block tables and live requests disagree")
