"""The device sampler against the plain restatement of the reference's sampler,
with the reference's own cases (src/test/test_sampler.c:65-257): greedy is the
argmax with the lowest index on ties, t=0 and k=1 are greedy, seeds reproduce,
top-k keeps exactly k, top-p keeps the crossing token, min-p keeps its boundary."""
import numpy as np
import pytest
import torch

import plain_sampler as PS

pytestmark = pytest.mark.gpu


def run(logits, params, seeds=None, idx=None, recent=None):
    from kappai_b200.sampling.sampler import sample
    n = logits.shape[0]
    t = torch.as_tensor(np.asarray(logits, dtype=np.float32)).cuda().clone()
    return sample(t, params, seeds or [1] * n, idx or list(range(n)), recent).cpu().tolist()


def SP(**kw):
    from kappai_b200.sampling import SamplingParams
    return SamplingParams(**kw)


@pytest.mark.parametrize("V", [7, 331, 1000, 65536, 70001])
def test_greedy_is_argmax_lowest_index_on_ties(V):
    rng = np.random.default_rng(0)
    l = rng.standard_normal((6, V)).astype(np.float32)
    l[1, [V // 3, V - 1]] = 9.0
    l[2, :] = 0.5                                     # all tied: index 0
    l[3, [V - 1]] = 11.0
    l[4, 0] = 12.0
    want = [PS.argmax(r) for r in l]
    assert want[1] == V // 3 and want[2] == 0
    assert run(l, [SP(temperature=0.0)] * 6) == want
    assert run(l, [SP(temperature=0.7, top_k=1)] * 6) == want


@pytest.mark.parametrize("V", [50, 331, 5000, 65536])
@pytest.mark.parametrize("cfg", [dict(temperature=0.8, top_k=40, top_p=0.9, min_p=0.1),
                                 dict(temperature=1.3, top_k=0, top_p=1.0, min_p=0.0),
                                 dict(temperature=0.5, top_k=0, top_p=0.7, min_p=0.0),
                                 dict(temperature=1.0, top_k=0, top_p=1.0, min_p=0.05),
                                 dict(temperature=2.0, top_k=1000, top_p=0.95, min_p=0.0),
                                 dict(temperature=0.8, top_k=5, top_p=1.0, min_p=0.0)])
def test_sampling_matches_plain(V, cfg):
    from kappai_b200.sampling import uniform
    rng = np.random.default_rng(1)
    n = 24
    l = (rng.standard_normal((n, V)) * 3).astype(np.float32)
    seeds = [int(s) for s in rng.integers(1, 2**62, n)]
    idx = [int(i) for i in rng.integers(0, 1000, n)]
    got = run(l, [SP(**cfg)] * n, seeds, idx)
    bad = 0
    for r in range(n):
        want, slack = PS.sample(l[r], uniform(seeds[r], idx[r]), **cfg)
        if got[r] != want:
            assert slack < 1e-5, f"row {r}: device {got[r]}, plain {want}, slack {slack}"
            bad += 1
    assert bad <= 1


def test_distribution_of_draws():
    """Many draws from a 4-token distribution follow its probabilities."""
    probs = np.array([0.5, 0.25, 0.15, 0.10])
    l = np.tile(np.log(probs).astype(np.float32), (4000, 1))
    got = np.array(run(l, [SP(temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, seed=5)] * 4000, [5] * 4000))
    freq = np.bincount(got, minlength=4) / 4000
    assert np.abs(freq - probs).max() < 0.03


def test_top_k_top_p_min_p_boundaries():
    V = 100
    l = np.full((1, V), -20.0, np.float32)
    l[0, [10, 20, 30, 40]] = np.log([0.4, 0.3, 0.2, 0.1]).astype(np.float32)
    n = 300
    L = np.repeat(l, n, 0)
    idx = list(range(n))
    draws = lambda **kw: set(run(L, [SP(temperature=1.0, **kw)] * n, [9] * n, idx))
    assert draws(top_k=2, top_p=1.0, min_p=0.0) == {10, 20}                  # exactly k
    assert draws(top_k=0, top_p=0.65, min_p=0.0) == {10, 20}                 # 0.4, then 0.7 > 0.65: crossing token kept
    assert draws(top_k=0, top_p=0.75, min_p=0.0) == {10, 20, 30}
    assert draws(top_k=0, top_p=1.0, min_p=0.5) == {10, 20, 30}              # p >= 0.5 * 0.4 keeps 0.2, drops 0.1
    assert draws(top_k=0, top_p=1.0, min_p=0.99) == {10}                     # at least one


def test_seed_reproducibility_and_batch_independence():
    rng = np.random.default_rng(2)
    l = (rng.standard_normal((5, 777)) * 2).astype(np.float32)
    p = [SP(temperature=0.9, top_k=50, top_p=0.95, min_p=0.02)] * 5
    a = run(l, p, [11, 12, 13, 14, 15], [0, 1, 2, 3, 4])
    b = run(l, p, [11, 12, 13, 14, 15], [0, 1, 2, 3, 4])
    assert a == b
    # a row's draw does not depend on the rows beside it
    alone = run(l[2:3], p[:1], [13], [2])
    assert alone == a[2:3]
    c = run(l, p, [21, 22, 23, 24, 25], [0, 1, 2, 3, 4])
    assert c != a


def test_repeat_penalty():
    V = 64
    rng = np.random.default_rng(3)
    l = rng.standard_normal((3, V)).astype(np.float32)
    l[0, 5], l[0, 6] = 10.0, 9.0
    l[1, 7], l[1, 8] = -0.5, -0.6
    l[1, :7] = -5; l[1, 9:] = -5
    recent = [[1, 5, 5, 2], [7, 3], [4]]
    pens = [4.0, 1.5, 1.0]
    from kappai_b200.sampling.sampler import sample
    t = torch.as_tensor(l).cuda().clone()
    params = [SP(temperature=0.0, repeat_penalty=p, repeat_last_n=3) for p in pens]
    got = sample(t, params, [1] * 3, [0] * 3, recent).cpu().tolist()
    want = []
    for r in range(3):
        want.append(PS.argmax(PS.apply_repeat_penalty(l[r], recent[r], 3, pens[r])))
    assert got == want and got[0] == 6 and got[1] == 8      # 10/16 < 9 ; -0.5*1.5 < -0.6
    np.testing.assert_allclose(t.cpu().numpy()[0], PS.apply_repeat_penalty(l[0], recent[0], 3, 4.0), rtol=1e-6)


def test_top_k_beyond_the_cap_is_refused():
    with pytest.raises(ValueError, match="1024"):
        run(np.zeros((1, 5000), np.float32), [SP(temperature=1.0, top_k=2000)])
