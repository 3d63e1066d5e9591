"""The scheduler's decisions, driven with a fake "model" that returns a fixed
next token (no GPU): admission, portions under a token budget, decode first,
finishing and freeing, and what happens when pages run out."""
import pytest

from kappai_b200.cache import CacheManager
from kappai_b200.engine.scheduler import (Request, Scheduler, FINISH_CONTEXT, FINISH_EOS, FINISH_LENGTH,
                                          FINISH_OOM, RUNNING, WAITING)
from kappai_b200.sampling import SamplingParams


def make(n_pages=16, page=4, slots=4, budget=8, max_running=4, max_len=64, eos=None):
    cache = CacheManager({"kv": (n_pages, page, None)}, slots)
    return cache, Scheduler(cache, budget, max_running, max_len, eos)


def req(i, n_prompt, n_predict=4):
    return Request(i, list(range(1, n_prompt + 1)), SamplingParams(temperature=0.0, n_predict=n_predict))


def run_step(s, token=7):
    plan = s.schedule()
    s.update(plan, {e.request.id: token for e in plan if e.sample})
    s.cache.check()
    return plan


def test_prompt_is_cut_under_the_budget_and_decodes_come_first():
    cache, s = make(budget=8)
    s.add(req("a", 13)); s.add(req("b", 3))
    p = run_step(s)
    assert [(e.request.id, e.start, e.n, e.sample) for e in p] == [("a", 0, 8, False)]
    p = run_step(s)       # a's rest (5) then b's whole prompt (3) fill the budget
    assert [(e.request.id, e.start, e.n, e.sample) for e in p] == [("a", 8, 5, True), ("b", 0, 3, True)]
    s.add(req("c", 20))
    p = run_step(s)       # two decode tokens first, then 6 tokens of c
    assert [(e.request.id, e.n) for e in p] == [("a", 1), ("b", 1), ("c", 6)]
    assert p[2].sample is False
    p = run_step(s)
    assert [(e.request.id, e.start, e.n) for e in p] == [("a", 14, 1), ("b", 4, 1), ("c", 6, 6)]


def test_portion_may_be_one_token():
    cache, s = make(budget=3)
    s.add(req("a", 2, n_predict=10)); s.add(req("b", 2, n_predict=10)); s.add(req("c", 5))
    run_step(s)           # a whole (2) + b first token (1)
    p = run_step(s)       # a decodes (1), b's last prompt token (1), c gets 1 token
    assert [(e.request.id, e.n, e.sample) for e in p] == [("a", 1, True), ("b", 1, True), ("c", 1, False)]


def test_finish_reasons_and_freeing():
    cache, s = make(max_len=8, eos=99)
    s.add(req("a", 3, n_predict=2)); s.add(req("b", 3, n_predict=-1)); s.add(req("c", 2, n_predict=-1))
    run_step(s)
    plan = s.schedule()
    s.update(plan, {"a": 7, "b": 7, "c": 99})
    done = {r.id: r.finish_reason for r in s.finished}
    assert done == {"a": FINISH_LENGTH, "c": FINISH_EOS}
    assert "a" not in cache.requests and "c" not in cache.requests and "b" in cache.requests
    while s.has_work():
        run_step(s)
    b = [r for r in s.finished if r.id == "b"][0]
    assert b.finish_reason == FINISH_CONTEXT and b.n_tokens == 8
    assert cache.pools["kv"].n_free == 16 and cache.slots.n_free == 4
    cache.check()


def test_admission_waits_for_slots_and_running_limit():
    cache, s = make(slots=2, max_running=2, budget=32)
    for i in range(4):
        s.add(req(i, 2, n_predict=2))
    p = run_step(s)
    assert [e.request.id for e in p] == [0, 1] and len(s.waiting) == 2
    run_step(s)           # 0 and 1 finish (2 tokens each) ...
    assert [r.id for r in s.finished] == [0, 1]
    p = run_step(s)       # ... and only now are 2 and 3 admitted, FIFO
    assert [e.request.id for e in p] == [2, 3]


def test_admission_needs_pages_for_the_first_portion():
    cache, s = make(n_pages=4, page=4, budget=32)
    s.add(req("a", 12, n_predict=8)); s.add(req("b", 8))
    p = run_step(s)
    assert [e.request.id for e in p] == ["a"]          # b's 8 tokens need 2 pages, 1 is free
    assert s.waiting[0].id == "b"


def test_out_of_pages_preempts_the_newest_and_recomputes():
    cache, s = make(n_pages=4, page=4, budget=32, slots=4)
    s.add(req("a", 7, n_predict=20)); s.add(req("b", 7, n_predict=20))
    run_step(s)                                        # both prefilled: 2 pages each, pool full
    assert cache.pools["kv"].n_free == 0
    p = run_step(s)                                    # token 8 of each still fits its second page
    assert [e.request.id for e in p] == ["a", "b"]
    p = run_step(s)                                    # a needs a third page: b (newest) is preempted
    assert [e.request.id for e in p] == ["a"] and s.n_preemptions == 1
    b = s.waiting[0]
    assert b.id == "b" and b.state == WAITING and b.n_computed == 0 and len(b.output) == 2
    assert "b" not in cache.requests
    b_entries = []
    while [r for r in s.finished if r.id == "a"] == []:
        p = run_step(s)
        b_entries += [(e.start, e.n, e.sample) for e in p if e.request.id == "b"]
    # a alone grows to 4 pages = 16 tokens, needs a 5th page and cannot have it
    a = [r for r in s.finished if r.id == "a"][0]
    assert a.finish_reason == FINISH_OOM and a.n_tokens == 17
    # in the step that ended a, b came back with prompt + its two tokens, from position 0
    assert b_entries == [(0, 9, True)]
    while s.has_work():
        run_step(s)
    assert cache.pools["kv"].n_free == 4 and cache.slots.n_free == 4


def test_request_that_can_never_fit_fails_cleanly():
    cache, s = make(n_pages=2, page=4, budget=32)
    s.add(req("big", 9)); s.add(req("ok", 3, n_predict=1))
    run_step(s)
    assert [(r.id, r.finish_reason) for r in s.finished][0] == ("big", FINISH_OOM)
    while s.has_work():
        run_step(s)
    assert [r.id for r in s.finished] == ["big", "ok"]
    with pytest.raises(ValueError, match="limit"):
        s.add(req("long", 64))


def test_every_token_is_computed_exactly_once_between_preemptions():
    """Replay the plans: positions of a request come in order, without gaps or repeats."""
    cache, s = make(n_pages=6, page=4, budget=5, slots=3, max_running=3)
    for i, n in enumerate([9, 4, 11, 2]):
        s.add(req(i, n, n_predict=6))
    seen = {}
    steps = 0
    while s.has_work():
        plan = s.schedule()
        assert sum(e.n for e in plan) <= 5
        for e in plan:
            if e.start == 0:
                seen[e.request.id] = 0                 # (re)started from scratch
            assert e.start == seen[e.request.id]
            seen[e.request.id] += e.n
            assert e.sample == (e.start + e.n == e.request.n_tokens)
        s.update(plan, {e.request.id: 5 for e in plan if e.sample})
        cache.check()
        steps += 1
        assert steps < 500
    assert sorted(r.id for r in s.finished) == [0, 1, 2, 3]
    assert all(len(r.output) == 6 for r in s.finished)
