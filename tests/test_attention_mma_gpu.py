"""The tensor-core prefill attention kernels alone (the tcgen05 kernel where it
takes the sizes, and the mma.sync kernel), against whole-sequence attention:
segments that start anywhere in a sequence, tiles that end inside a page,
windows, one far key, and a batch that mixes long and short segments."""
import math

import numpy as np
import pytest
import torch

import plain_lfm2 as P
from test_kernels_gpu import dev, i32, paged_setup, rt

pytestmark = pytest.mark.gpu
DT = torch.bfloat16
TOL = 1.5e-2


@pytest.fixture(autouse=True, params=["tcgen05 two heads a CTA", "tcgen05 one head a CTA", "mma.sync"])
def _both_kernels(request):
    """Every test runs three times: with the tcgen05 kernels allowed (two heads a CTA where the head counts
    allow it; one head a CTA always), and with the mma.sync kernel only."""
    from kappai_b200.ops import kernels as Kn
    from kappai_b200.ops.build import load_library
    old = Kn.USE_TC_ATTENTION
    Kn.USE_TC_ATTENTION = request.param != "mma.sync"
    load_library("attention_tc").kp_attention_tc_set_pair(1 if "two heads" in request.param else 0)
    yield
    Kn.USE_TC_ATTENTION = old
    load_library("attention_tc").kp_attention_tc_set_pair(1)
    assert Kn.attention_tc_status() == 0, "a bounded wait of the tcgen05 attention kernel gave up"


def run_prefill(qs, q_from, seq_lens, cache, bt, scale, window, page, H, G, hd):
    from kappai_b200.ops import kernels as Kn
    rows, cu, seg_pos, tile_seg, tile_row0, big = [], [0], [], [], [], []
    for i, (L, a) in enumerate(zip(seq_lens, q_from)):
        rows.append(qs[i][a:])
        for r0 in range(cu[-1], cu[-1] + L - a, Kn.PREFILL_TILE):
            tile_seg.append(i)
            tile_row0.append(r0)
        for r0 in range(cu[-1], cu[-1] + L - a, 128):
            big.append((-(a + min(r0 + 128, cu[-1] + L - a) - cu[-1] - 1), i, r0))     # most keys first
        cu.append(cu[-1] + L - a)
        seg_pos.append(a)
    big.sort()
    q_rows = np.concatenate(rows, 0).reshape(cu[-1], H * hd)
    out = torch.empty((cu[-1], H * hd), dtype=DT, device="cuda")
    assert Kn.attention_prefill_ok(dev(q_rows, DT), hd)
    Kn.attention_prefill(dev(q_rows, DT), dev(cache, DT), i32(bt), i32(cu), i32(seg_pos), i32(tile_seg), i32(tile_row0),
                         out, scale, window, page, H, G, hd, i32([x[1] for x in big]), i32([x[2] for x in big]))
    return out.cpu().double().numpy().reshape(cu[-1], H, hd), cu


@pytest.mark.parametrize("H,G,hd,page,window", [
    (4, 2, 64, 64, None), (32, 8, 64, 64, None), (6, 3, 64, 16, None), (5, 1, 128, 32, None), (8, 2, 64, 16, 100),
    (2, 2, 128, 8, 33), (3, 1, 64, 128, None)])
def test_prefill_mma_mixed_segments(H, G, hd, page, window):
    rng = np.random.default_rng(50)
    seq_lens = [70, 300, 129, 1, 64, 200]
    q_from = [0, 130, 128, 0, 63, 0]                  # whole prompts, late portions, single rows
    cache, bt, ks, vs = paged_setup(rng, seq_lens, page, G, hd, DT)
    scale = 1.0 / math.sqrt(hd)
    qs = [rt(rng.standard_normal((L, H, hd)), DT) for L in seq_lens]
    got, cu = run_prefill(qs, q_from, seq_lens, cache, bt, scale, window, page, H, G, hd)
    for i, (L, a) in enumerate(zip(seq_lens, q_from)):
        ref = P.attention(qs[i], ks[i], vs[i], scale, window)[a:]
        err = np.abs(got[cu[i]:cu[i + 1]] - ref).max()
        assert err <= TOL, f"segment {i}: {err}"


@pytest.mark.parametrize("far", [0, 63, 64, 500, 1023])
def test_prefill_mma_finds_one_far_key(far):
    """Every row of a late portion points at one far key; the output must be that key's value."""
    rng = np.random.default_rng(51)
    H, G, hd, page, L, a = 4, 2, 64, 64, 1100, 1024
    cache, bt, ks, vs = paged_setup(rng, [L], page, G, hd, DT)
    q = rt(rng.standard_normal((L, H, hd)) * 0.01, DT)
    for h in range(H):
        q[a:, h] = ks[0][far, h // (H // G)] * 8.0
    got, _ = run_prefill([q], [a], [L], cache, bt, 1.0 / math.sqrt(hd), None, page, H, G, hd)
    for h in range(H):
        np.testing.assert_allclose(got[:, h], np.broadcast_to(vs[0][far, h // (H // G)], (L - a, hd)), atol=3e-2)


def test_prefill_mma_window_edge_and_released_pages():
    rng = np.random.default_rng(52)
    H, G, hd, page, L, window, a = 2, 1, 64, 16, 400, 70, 300
    cache, bt, ks, vs = paged_setup(rng, [L], page, G, hd, DT)
    # keys that no row of the portion may read carry a huge value; their pages count as released
    first_needed = a - window + 1
    for key in range(first_needed):
        cache[bt[0][key // page], 1, :, key % page, :] = 3e4
        vs[0][key] = 3e4
    bt2 = bt.copy()
    bt2[0, :first_needed // page] = -1
    q = rt(rng.standard_normal((L, H, hd)), DT)
    got, _ = run_prefill([q], [a], [L], cache, bt2, 1.0 / math.sqrt(hd), window, page, H, G, hd)
    ref = P.attention(q, ks[0], vs[0], 1.0 / math.sqrt(hd), window)[a:]
    assert np.abs(got).max() < 50
    assert np.abs(got - ref).max() <= TOL


def test_prefill_mma_agrees_with_the_general_kernel_and_the_split_kernel():
    """The same rows through the three attention kernels."""
    from kappai_b200.ops import kernels as Kn
    rng = np.random.default_rng(53)
    H, G, hd, page = 8, 2, 64, 32
    seq_lens, q_from = [257, 90], [250, 88]
    cache, bt, ks, vs = paged_setup(rng, seq_lens, page, G, hd, DT)
    qs = [rt(rng.standard_normal((L, H, hd)), DT) for L in seq_lens]
    got, cu = run_prefill(qs, q_from, seq_lens, cache, bt, 0.125, None, page, H, G, hd)
    pos = list(range(250, 257)) + [88, 89]
    row_seg = [0] * 7 + [1] * 2
    q_rows = np.concatenate([qs[0][250:], qs[1][88:]]).reshape(9, H * hd)
    gen = torch.empty((9, H * hd), dtype=DT, device="cuda")
    Kn.attention_rows(dev(q_rows, DT), dev(cache, DT), i32(bt), i32(row_seg), i32(pos), gen, 0.125, None, page, H, G, hd)
    ws = torch.empty(Kn.attention_split_scratch(9, H, hd, 2), device="cuda")
    spl = torch.empty_like(gen)
    Kn.attention_split(dev(q_rows, DT), dev(cache, DT), i32(bt), i32(row_seg), i32(pos), spl, ws, 2, 0.125, None, page,
                       H, G, hd)
    g = got.reshape(9, H * hd)
    assert np.abs(g - gen.cpu().double().numpy()).max() <= TOL
    assert np.abs(g - spl.cpu().double().numpy()).max() <= TOL
