"""Trace replay through bin/trace_run, in every way of cutting the work, in
32-bit and in bfloat16, against the plain implementation."""
import numpy as np
import pytest

import replay_util as R
from tolerances import tol_for

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [21, 33, 49, 127, 2, 70], "B": [25, 33, 88, 154, 250, 3], "C": [40, 130, 77, 300],
           "D": [300, 700, 130, 520]}
PROMPTS = {"A": [5, 17, 33, 100, 1, 40], "B": [1, 9, 64, 130, 200, 2], "C": [8, 100, 70, 260],
           "D": [260, 600, 100, 500]}


def requests_of(name, vocab, seed):
    rng = np.random.default_rng(seed)
    reqs = {f"{name.lower()}{i}": rng.integers(0, vocab, n).tolist() for i, n in enumerate(LENGTHS[name])}
    prompt_len = {rid: p for rid, p in zip(reqs, PROMPTS[name])}
    return reqs, prompt_len


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page_size", [("A", None), ("B", None), ("B", 16), ("C", 32), ("D", None), ("D", 16)])
def test_all_cuts_agree_with_plain(name, page_size, dtype, model_dirs, plain_models, tmp_path):
    plain = plain_models[name]
    reqs, prompt_len = requests_of(name, plain.cfg["vocab_size"], seed=11)
    expected = {rid: plain.logits(t) for rid, t in reqs.items()}
    tol = max(tol_for(dtype, e) for e in expected.values()) if dtype == "float32" else \
        min(tol_for(dtype, e) for e in expected.values())
    page = page_size or 64
    longest = max(-(-len(t) // page) * page for t in reqs.values())
    # room for the longest request plus two more pages: the mixed family must reuse pages
    max_tokens = longest + 2 * page
    tr = R.Trace()
    bounds = {}
    for fam, fn in (("whole", R.whole), ("last32", R.last_decoded), ("portions", R.portions)):
        b = len(tr.steps)
        fn(tr, reqs)
        bounds[fam] = (b, len(tr.steps))
    b = len(tr.steps)
    R.mixed(tr, reqs, prompt_len, seed=3, max_live=4, page=page, max_tokens=max_tokens)
    bounds["mixed"] = (b, len(tr.steps))
    assert max(len(s["entries"]) for s in tr.steps[b:]) >= 2, "the mixed family never had two requests in a step"
    out = R.run_trace(model_dirs[name], dtype, tr, str(tmp_path / "out"), max_tokens, page_size)
    worst = R.compare(tr, out, expected, tol, f"{name}/{dtype}/page{page}")
    # the pool was small enough that pages went from one request to another
    stats = R.cache_stats(str(tmp_path / "out"))
    assert stats and all(g["reused"] > 0 and g["handed_out"] > g["pages"] for g in stats.values()), stats
    if dtype == "float32":
        # the 32-bit path sums in an order that does not depend on the cut: every way of cutting gives the
        # same bits for a (request, position)
        for place, rows in R.rows_by_place(tr, out).items():
            assert len(rows) >= 2, place
            for r in rows[1:]:
                assert np.array_equal(rows[0], r), f"{name}: float32 logits of {place} differ between cuts"
    print(f"{name} {dtype} page {page}: worst |error| {worst:.3e} (tolerance {tol:.3e}), {len(tr.steps)} steps")


def test_replay_rejects_what_cannot_fit(model_dirs, tmp_path):
    tr = R.Trace()
    tr.add([("x", list(range(100)), [99])])
    with pytest.raises(AssertionError, match="exceed the limit|pages"):
        R.run_trace(model_dirs["A"], "float32", tr, str(tmp_path / "o"), max_tokens=64)
