"""The split-KV attention kernel alone: against whole-sequence attention and
against the general kernel, over head sizes, group ratios, page sizes, windows
and chunk edges (positions around multiples of 256)."""
import math

import numpy as np
import pytest
import torch

import plain_lfm2 as P
from test_kernels_gpu import dev, i32, paged_setup, rt, tol

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def run_split(q_rows, cache, bt, row_seg, pos, scale, window, page, H, G, hd, dtype, n_chunks=None):
    from kappai_b200.ops import kernels as Kn
    n = len(pos)
    n_chunks = n_chunks or -(-(max(pos) + 1) // Kn.SPLIT_CHUNK)
    ws = torch.full((Kn.attention_split_scratch(n, H, hd, n_chunks),), float("nan"), device="cuda")
    out = torch.empty((n, H * hd), dtype=dtype, device="cuda")
    Kn.attention_split(dev(q_rows, dtype), dev(cache, dtype), i32(bt), i32(row_seg), i32(pos), out, ws, n_chunks,
                       scale, window, page, H, G, hd)
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,hd,page,window", [
    (4, 2, 16, 16, None), (5, 1, 48, 32, None), (32, 8, 64, 64, None), (8, 2, 128, 16, 300), (2, 2, 256, 8, None),
    (8, 1, 32, 64, None), (6, 3, 80, 128, 17),
    # head size 64 in bfloat16 takes the persistent kernel: pages of 8 keys (32 boxes a chunk) to 128 (half a box a
    # tile), one to eight heads a kv head, windows that cut chunks and tiles
    (8, 8, 64, 16, None), (16, 2, 64, 32, 100), (4, 2, 64, 128, None), (6, 2, 64, 8, 37), (8, 4, 64, 64, 300)])
def test_split_matches_whole_sequence_attention(dtype, H, G, hd, page, window):
    rng = np.random.default_rng(40)
    seq_lens = [1, 255, 256, 257, 700, 513]
    cache, bt, ks, vs = paged_setup(rng, seq_lens, page, G, hd, dtype)
    scale = 1.0 / math.sqrt(hd)
    qs = [rt(rng.standard_normal((L, H, hd)), dtype) for L in seq_lens]
    # the last row of every request (a decode step), plus two rows of the longest (a short portion)
    pos = [L - 1 for L in seq_lens] + [697, 698]
    row_seg = list(range(len(seq_lens))) + [4, 4]
    q_rows = np.stack([qs[s][p] for s, p in zip(row_seg, pos)]).reshape(len(pos), H * hd)
    out = run_split(q_rows, cache, bt, row_seg, pos, scale, window, page, H, G, hd, dtype)
    got = out.cpu().double().numpy().reshape(len(pos), H, hd)
    for j, (s, p) in enumerate(zip(row_seg, pos)):
        ref = P.attention(qs[s][:p + 1], ks[s][:p + 1], vs[s][:p + 1], scale, window)[-1]
        np.testing.assert_allclose(got[j], ref, rtol=tol(dtype), atol=tol(dtype), err_msg=f"row {j} (pos {p})")
    # a wider grid than needed (as under a captured graph) changes nothing
    out2 = run_split(q_rows, cache, bt, row_seg, pos, scale, window, page, H, G, hd, dtype, n_chunks=7)
    assert torch.equal(out, out2)
    # and the general kernel agrees closely
    from kappai_b200.ops import kernels as Kn
    gen = torch.empty_like(out)
    Kn.attention_rows(dev(q_rows, dtype), dev(cache, dtype), i32(bt), i32(row_seg), i32(pos), gen, scale, window, page,
                      H, G, hd)
    assert (gen.float() - out.float()).abs().max().item() <= tol(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far", [0, 255, 256, 511, 512, 1000])
def test_split_finds_one_far_key(dtype, far):
    rng = np.random.default_rng(41)
    H, G, hd, page, L = 8, 2, 64, 64, 1001
    cache, bt, ks, vs = paged_setup(rng, [L], page, G, hd, dtype)
    q = rt(rng.standard_normal((1, H, hd)) * 0.01, dtype)
    for h in range(H):
        q[0, h] = ks[0][far, h // (H // G)] * 8.0
    out = run_split(q.reshape(1, -1), cache, bt, [0], [L - 1], 1.0 / math.sqrt(hd), None, page, H, G, hd, dtype)
    got = out.cpu().double().numpy().reshape(H, hd)
    for h in range(H):
        np.testing.assert_allclose(got[h], vs[0][far, h // (H // G)], atol=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd,window", [(64, None), (128, None), (64, 7000), (48, None)])
def test_split_over_many_chunks(dtype, hd, window):
    """20,000 keys: 79 chunks, more than the merge holds in shared memory at a time (it adds them batch by
    batch, in chunk order); with a window the first chunks are left out.  One far key stands out."""
    rng = np.random.default_rng(43)
    H, G, page, L = 4, 2, 64, 20000
    cache, bt, ks, vs = paged_setup(rng, [L, 300], page, G, hd, dtype)
    q = rt(rng.standard_normal((2, H, hd)), dtype)
    q[0, 1] = ks[0][L - 6500, 0] * 4.0                       # head 1 looks at one key far back (inside the window)
    scale = 1.0 / math.sqrt(hd)
    out = run_split(q.reshape(2, -1), cache, bt, [0, 1], [L - 1, 299], scale, window, page, H, G, hd, dtype)
    got = out.cpu().double().numpy().reshape(2, H, hd)
    for j, (s_, p) in enumerate([(0, L - 1), (1, 299)]):
        # the last row only: scores of one query against all keys
        kk, vv = ks[s_][:p + 1], vs[s_][:p + 1]
        lo = max(0, p - window + 1) if window else 0
        for h in range(H):
            sc = (kk[lo:, h // (H // G)] @ q[j, h]) * scale
            w = np.exp(sc - sc.max()); w /= w.sum()
            np.testing.assert_allclose(got[j, h], w @ vv[lo:, h // (H // G)], rtol=tol(dtype), atol=tol(dtype),
                                       err_msg=f"row {j} head {h}")


def test_split_row_does_not_depend_on_the_batch():
    rng = np.random.default_rng(42)
    H, G, hd, page = 32, 8, 64, 64
    seq_lens = [900, 300, 2048]
    cache, bt, ks, vs = paged_setup(rng, seq_lens, page, G, hd, torch.bfloat16)
    q = rt(rng.standard_normal((3, H * hd)), torch.bfloat16)
    pos = [L - 1 for L in seq_lens]
    both = run_split(q, cache, bt, [0, 1, 2], pos, 0.125, None, page, H, G, hd, torch.bfloat16)
    for r in range(3):
        alone = run_split(q[r:r + 1], cache, bt, [r], pos[r:r + 1], 0.125, None, page, H, G, hd, torch.bfloat16)
        assert torch.equal(alone[0], both[r])


def test_split_refuses_large_group_ratio():
    from kappai_b200.ops import kernels as Kn
    q = torch.zeros((1, 16 * 16), device="cuda")
    with pytest.raises(Kn.KernelError, match="not supported"):
        Kn.attention_split(q, torch.zeros((1, 2, 1, 16, 16), device="cuda"), i32([[0]]), i32([0]), i32([0]),
                           torch.empty_like(q), torch.zeros(100000, device="cuda"), 1, 1.0, None, 16, 16, 1, 16)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,hd,page", [(32, 8, 64, 64), (5, 1, 48, 32), (8, 2, 128, 16)])
def test_both_merge_kernels_give_the_same_bits(dtype, H, G, hd, page):
    """Rows of at most 64 chunks are merged by a warp each, longer ones by a CTA each; which of the two runs is
    decided by the width of the grid (the largest position of the batch), so a row must get the same bits from
    both: the same rows once with the chunks they need and once in a grid of 70 chunks."""
    rng = np.random.default_rng(44)
    seq_lens = [1, 300, 2000, 513]
    cache, bt, ks, vs = paged_setup(rng, seq_lens, page, G, hd, dtype)
    scale = 1.0 / math.sqrt(hd)
    q_rows = rt(rng.standard_normal((len(seq_lens), H * hd)), dtype)
    pos = [L - 1 for L in seq_lens]
    row_seg = list(range(len(seq_lens)))
    by_warp = run_split(q_rows, cache, bt, row_seg, pos, scale, None, page, H, G, hd, dtype)
    by_cta = run_split(q_rows, cache, bt, row_seg, pos, scale, None, page, H, G, hd, dtype, n_chunks=70)
    assert torch.equal(by_warp, by_cta)
    assert torch.isfinite(by_warp.float()).all()
