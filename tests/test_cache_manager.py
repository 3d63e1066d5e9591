"""The cache manager's bookkeeping (no GPU): no page lost, held twice or freed twice."""
import random

import pytest

from kappai_b200.cache import CacheManager, CacheError, OutOfPages, OutOfSlots, PagePool, SlotPool, RELEASED


def test_pool_extend_and_close():
    p = PagePool(8, 16)
    p.open("a")
    p.extend("a", 1)
    assert len(p.table("a")) == 1 and p.n_free == 7
    p.extend("a", 16)
    assert len(p.table("a")) == 1
    p.extend("a", 17)
    assert len(p.table("a")) == 2
    p.open("b")
    p.extend("b", 6 * 16)
    assert p.n_free == 0
    with pytest.raises(OutOfPages):
        p.extend("a", 33)
    p.check()
    p.close("a")
    assert p.n_free == 2
    with pytest.raises(CacheError, match="twice"):
        p.close("a")
    p.check()


def test_pages_are_used_again():
    p = PagePool(4, 8)
    p.open("a"); p.extend("a", 32)
    used = set(p.table("a"))
    p.close("a")
    p.open("b"); p.extend("b", 32)
    assert set(p.table("b")) == used
    p.check()


def test_window_gives_pages_back():
    p = PagePool(16, 4, window=6)
    p.open("a")
    p.extend("a", 20)
    assert p.release_behind("a", 20) == 3          # next position 20 reads keys 15..20: blocks 0,1,2 are behind
    t = p.table("a")
    assert t[:3] == [RELEASED] * 3 and all(x != RELEASED for x in t[3:])
    assert p.n_free == 16 - 2
    p.check()
    assert p.release_behind("a", 20) == 0
    p.extend("a", 24)
    p.release_behind("a", 24)
    p.check()
    p.close("a")
    assert p.n_free == 16
    p.check()
    q = PagePool(4, 4)                              # no window: nothing is released early
    q.open("a"); q.extend("a", 16)
    assert q.release_behind("a", 16) == 0


def test_slots():
    s = SlotPool(2)
    a, b = s.take("a"), s.take("b")
    assert a != b
    with pytest.raises(OutOfSlots):
        s.take("c")
    s.give_back(a)
    with pytest.raises(CacheError, match="twice"):
        s.give_back(a)
    assert s.take("c") == a
    s.check()


def test_manager_is_atomic_over_groups():
    m = CacheManager({"full": (4, 8, None), "win": (2, 8, 8)}, n_slots=2)
    m.admit("a")
    assert m.can_extend("a", 16)
    m.extend("a", 16)
    assert not m.can_extend("a", 17)               # the windowed group has no third page
    with pytest.raises(OutOfPages):
        m.extend("a", 17)
    assert len(m.block_table("a", "full")) == 2    # nothing was taken in the other group either
    m.advance("a", 16)                             # window 8 at next position 16: block 0 is behind
    assert m.block_table("a", "win")[0] == RELEASED
    m.extend("a", 17)
    m.check()
    assert m.token_slots("a", "full", 15, 2) == [m.block_table("a", "full")[1] * 8 + 7,
                                                  m.block_table("a", "full")[2] * 8 + 0]
    with pytest.raises(CacheError, match="released"):
        m.token_slots("a", "win", 0, 1)
    m.free("a")
    with pytest.raises(CacheError, match="twice"):
        m.free("a")
    m.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted(seed):
    rng = random.Random(seed)
    window = [None, 24, 40][seed % 3]
    m = CacheManager({"kv": (24, 8, window), "kv2": (40, 8, None)}, n_slots=5)
    live, held_slots, next_id = {}, {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.can_admit():
            rc = m.admit(next_id)
            assert rc.slot not in held_slots.values()
            held_slots[next_id] = rc.slot
            live[next_id] = 0
            next_id += 1
        elif op < 0.8 and live:
            r = rng.choice(list(live))
            new_len = live[r] + rng.choice([1, 1, 1, 2, 7, 16, 33])
            if m.can_extend(r, new_len):
                m.extend(r, new_len)
                m.advance(r, new_len)
                live[r] = new_len
                # every position the next token may read has a page
                lo = 0 if window is None else max(0, new_len - window + 1)
                t = m.block_table(r, "kv")
                assert all(t[pos // 8] != RELEASED for pos in range(lo, new_len))
            else:
                with pytest.raises(OutOfPages):
                    m.extend(r, new_len)
        elif live:
            r = rng.choice(list(live))
            m.free(r)
            del live[r], held_slots[r]
        m.check()
        # no page in two tables
        for g in ("kv", "kv2"):
            pages = [p for r in live for p in m.block_table(r, g) if p != RELEASED]
            assert len(pages) == len(set(pages))
    for r in list(live):
        m.free(r)
    m.check()
    assert all(p.n_free == p.n_pages for p in m.pools.values()) and m.slots.n_free == 5


def test_token_slots_of_a_long_portion_are_those_of_its_positions_one_by_one():
    """Portions of more than 32 tokens take their slots by arrays: the same slots as asked one by one, from any
    start, across page edges; a released page in the range is refused by its first position."""
    m = CacheManager({"full": (64, 8, None), "win": (64, 8, 40)}, n_slots=2)
    m.admit("a")
    m.extend("a", 300)
    rnd = random.Random(3)
    for _ in range(50):
        start = rnd.randrange(0, 250)
        n = rnd.randrange(33, 300 - start + 1) if 300 - start > 33 else 33
        n = min(n, 300 - start)
        one_by_one = [m.token_slots("a", "full", p, 1)[0] for p in range(start, start + n)]
        assert m.token_slots("a", "full", start, n) == one_by_one
    m.advance("a", 300)                            # window 40 at next position 300: blocks before 261 // 8 are behind
    first_kept = next(i for i, p in enumerate(m.block_table("a", "win")) if p != RELEASED) * 8
    assert m.token_slots("a", "win", first_kept, 300 - first_kept) == \
        [m.token_slots("a", "win", p, 1)[0] for p in range(first_kept, 300)]
    with pytest.raises(CacheError, match=f"position {first_kept - 8} "):
        m.token_slots("a", "win", first_kept - 8, 40)
