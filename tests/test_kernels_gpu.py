"""Each CUDA kernel alone against a plain float64 reference of the same op,
at sizes other than the engine's tiny models (odd widths, head sizes in steps
of 16, vocabularies that are no power of two), in float32 and bfloat16."""
import math

import numpy as np
import pytest
import torch

import plain_lfm2 as P

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def dev(a, dtype=None):
    t = torch.as_tensor(np.asarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def rt(a, dtype):
    """The values a tensor of ``dtype`` actually holds, as float64 numpy."""
    return torch.as_tensor(np.asarray(a, dtype=np.float32)).to(dtype).double().numpy()


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 1.2e-2) * scale


def i32(a):
    return torch.as_tensor(np.asarray(a, dtype=np.int32)).cuda()


# ---------------------------------------------------------------- rowwise

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("V,d,n", [(331, 120, 7), (1000, 2048, 3), (50, 17, 1)])
def test_embed_rows(dtype, V, d, n):
    from kappai_b200.ops import kernels as K
    rng = np.random.default_rng(0)
    table = rt(rng.standard_normal((V, d)), dtype)
    ids = rng.integers(0, V, n)
    ids[0], ids[-1] = V - 1, 0
    out = torch.empty((n, d), dtype=torch.float32, device="cuda")
    K.embed_rows(dev(table, dtype), i32(ids), out, 1.0)
    assert np.array_equal(out.cpu().double().numpy(), P.embedding(table, ids))
    K.embed_rows(dev(table, dtype), i32(ids), out, 0.5)
    np.testing.assert_allclose(out.cpu().double().numpy(), 0.5 * P.embedding(table, ids), rtol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,d,eps", [(5, 120, 1e-5), (3, 2048, 1e-6), (2, 5000, 1e-5), (1, 7, 0.1)])
def test_rmsnorm_rows(dtype, n, d, eps):
    from kappai_b200.ops import kernels as K
    rng = np.random.default_rng(1)
    x = (rng.standard_normal((n, d)) * rng.uniform(0.01, 30, (n, 1))).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    ref = P.rmsnorm(x.astype(np.float64), w.astype(np.float64), eps)
    out = torch.empty((n, d), dtype=dtype, device="cuda")
    K.rmsnorm_rows(dev(x), dev(w), eps, out)
    np.testing.assert_allclose(out.cpu().double().numpy(), ref, rtol=tol(dtype), atol=tol(dtype))
    rows = [n - 1, 0, n - 1]
    out2 = torch.empty((3, d), dtype=dtype, device="cuda")
    K.rmsnorm_rows(dev(x), dev(w), eps, out2, i32(rows))
    assert torch.equal(out2, out[torch.tensor(rows, device="cuda")])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [2048, 1000, 64])
def test_rmsnorm_rows_same_bits_for_few_and_many_rows(dtype, d):
    """Few rows and many rows run different kernels (a block or a warp a row) with the
    same arithmetic: a row's result must not depend on how many rows there are."""
    from kappai_b200.ops import kernels as K
    rng = np.random.default_rng(11)
    n = 600
    x = (rng.standard_normal((n, d)) * rng.uniform(0.01, 30, (n, 1))).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    many = K.rmsnorm_rows(dev(x), dev(w), 1e-5, torch.empty((n, d), dtype=dtype, device="cuda"))
    ref = P.rmsnorm(x.astype(np.float64), w.astype(np.float64), 1e-5)
    np.testing.assert_allclose(many.cpu().double().numpy(), ref, rtol=tol(dtype), atol=tol(dtype))
    for lo, hi in ((0, 1), (7, 15), (100, 356), (599, 600)):
        few = K.rmsnorm_rows(dev(x[lo:hi]), dev(w), 1e-5, torch.empty((hi - lo, d), dtype=dtype, device="cuda"))
        assert torch.equal(few, many[lo:hi]), (lo, hi)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    from kappai_b200.ops import kernels as K
    rng = np.random.default_rng(2)
    n, ff = 5, 333
    gu = rt(rng.standard_normal((n, 2 * ff)) * 4, dtype)
    out = torch.empty((n, ff), dtype=dtype, device="cuda")
    K.swiglu(dev(gu, dtype), out)
    ref = P.swiglu(gu[:, :ff], gu[:, ff:])
    np.testing.assert_allclose(out.cpu().double().numpy(), ref, rtol=tol(dtype), atol=tol(dtype))


# ------------------------------------------------------------------- gemm

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 65, 33), (70, 130, 100), (8, 2048, 2048), (64, 331, 120),
                                   (200, 96, 5632), (129, 64, 16), (2, 1000, 17)])
def test_linear_against_plain(dtype, M, N, K):
    from kappai_b200.ops.linear import linear
    rng = np.random.default_rng(3)
    a = rt(rng.standard_normal((M, K)), dtype)
    w = rt(rng.standard_normal((N, K)) / math.sqrt(K), dtype)
    b = rng.standard_normal(N).astype(np.float32)
    ref = P.linear(a, w, b.astype(np.float64))
    A, W, B = dev(a, dtype), dev(w, dtype), dev(b)
    out = linear(A, W, B)
    assert out.dtype == dtype
    np.testing.assert_allclose(out.cpu().double().numpy(), ref, rtol=tol(dtype), atol=tol(dtype, 2))
    out32 = linear(A, W, B, out_dtype=torch.float32)
    np.testing.assert_allclose(out32.cpu().double().numpy(), ref, rtol=2e-5, atol=2e-5 * math.sqrt(K))
    res = rng.standard_normal((M, N)).astype(np.float32)
    acc = dev(res).clone()
    linear(A, W, None, out=acc, accumulate=True)
    np.testing.assert_allclose(acc.cpu().double().numpy(), res + P.linear(a, w), rtol=2e-5, atol=2e-5 * math.sqrt(K))


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_rows_do_not_depend_on_the_batch(dtype):
    """The same row gives the same bits alone, in a small batch and in a large one."""
    from kappai_b200.ops.linear import linear
    rng = np.random.default_rng(4)
    K_, N = 520, 300
    a = dev(rt(rng.standard_normal((150, K_)), dtype), dtype)
    w = dev(rt(rng.standard_normal((N, K_)) / 20, dtype), dtype)
    full = linear(a, w, out_dtype=torch.float32)
    for rows in ([0], [149], [3, 77], list(range(64)), list(range(5, 14))):
        part = linear(a[rows].contiguous(), w, out_dtype=torch.float32)
        err = (part - full[rows]).abs().max().item()
        assert err <= (1e-5 if dtype == torch.float32 else 2e-3), (rows[:3], err)


def test_linear_with_a_weight_stored_in_32_bit():
    from kappai_b200.ops.linear import linear
    rng = np.random.default_rng(5)
    a = rt(rng.standard_normal((4, 40)), torch.bfloat16)
    w = rng.standard_normal((9, 40)).astype(np.float32)          # not representable in bfloat16
    out = linear(dev(a, torch.bfloat16), dev(w), out_dtype=torch.float32)
    np.testing.assert_allclose(out.cpu().double().numpy(), P.linear(a, w.astype(np.float64)), rtol=1e-5, atol=1e-5)


# -------------------------------------------------------------- shortconv

def conv_stream_reference(p, w, bias, state, fresh):
    """The reference's loop (src/backend/cpu/common.c:2393-2431) in float64:
    one row at a time with an explicit history."""
    n, d3 = p.shape
    d = d3 // 3
    K = w.shape[1]
    hist = np.zeros((K - 1, d)) if fresh else state.copy()
    out = np.zeros((n, d))
    for t in range(n):
        bx = p[t, :d] * p[t, 2 * d:]
        s = bx * w[:, K - 1]
        for k in range(K - 1):
            s = s + hist[k] * w[:, k]
        if bias is not None:
            s = s + bias
        out[t] = p[t, d:2 * d] * s
        hist = np.concatenate([hist[1:], bx[None]], 0)
    return out, hist


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,K,with_bias", [(33, 2, False), (64, 3, False), (96, 4, True), (130, 7, True), (16, 16, False)])
def test_shortconv_segments_and_state(dtype, d, K, with_bias):
    """Segments of 1, 2, K-2, K-1, K and many rows; some fresh (position 0),
    some continuing from a slot; slots in scrambled order; untouched slots stay."""
    from kappai_b200.ops import kernels as Kn
    rng = np.random.default_rng(6)
    lens = [1, 2, max(1, K - 2), K - 1, K, 37, 1]
    fresh = [False, True, False, False, True, False, True]
    n_slots = len(lens) + 3
    slots = rng.permutation(n_slots)[:len(lens)]
    n = sum(lens)
    p = rt(rng.standard_normal((n, 3 * d)), dtype)
    w = rng.uniform(-0.6, 0.6, (d, K)).astype(np.float32)
    bias = rng.standard_normal(d).astype(np.float32) * 0.1 if with_bias else None
    state0 = rng.standard_normal((n_slots, K - 1, d)).astype(np.float32)
    cu = np.concatenate([[0], np.cumsum(lens)])
    row_seg = np.repeat(np.arange(len(lens)), lens)
    seg_pos = [0 if f else 5 + i for i, f in enumerate(fresh)]

    state = dev(state0).clone()
    out = torch.empty((n, d), dtype=dtype, device="cuda")
    args = (i32(cu), i32(seg_pos), i32(slots))
    Kn.shortconv_forward(dev(p, dtype), dev(w), None if bias is None else dev(bias), state, i32(row_seg), *args, out)
    Kn.shortconv_update_state(dev(p, dtype), state, *args, len(lens))
    got, new_state = out.cpu().double().numpy(), state.cpu().double().numpy()
    for i, L in enumerate(lens):
        ref, hist = conv_stream_reference(p[cu[i]:cu[i + 1]], w.astype(np.float64),
                                          None if bias is None else bias.astype(np.float64),
                                          state0[slots[i]].astype(np.float64), fresh[i])
        np.testing.assert_allclose(got[cu[i]:cu[i + 1]], ref, rtol=tol(dtype), atol=tol(dtype), err_msg=f"segment {i}")
        np.testing.assert_allclose(new_state[slots[i]], hist, rtol=1e-6, atol=1e-6, err_msg=f"state of segment {i}")
    untouched = [s for s in range(n_slots) if s not in slots]
    assert np.array_equal(new_state[untouched], state0[untouched].astype(np.float64))


@pytest.mark.parametrize("M,d,K,Kc,with_bias", [(1, 64, 512, 3, False), (8, 96, 1024, 4, True), (11, 200, 512, 2, True),
                                                (16, 2048, 2048, 3, False)])
def test_conv_step_in_the_in_proj_epilogue(M, d, K, Kc, with_bias):
    """The weight-streaming product with the conv step of a decode step in its epilogue: [B | C | X] = a W^T is
    never written out.  Against the plain product followed by the plain conv step; and the same bits, output and
    state, as the separate product and decode kernels."""
    from kappai_b200.ops import kernels as Kn
    dtype = torch.bfloat16
    rng = np.random.default_rng(8)
    a = rt(rng.standard_normal((M, K)), dtype)
    w_in = rt(rng.standard_normal((3 * d, K)) / np.sqrt(K), dtype)
    b_in = rng.standard_normal(3 * d).astype(np.float32) * 0.1 if with_bias else None
    cw = rng.uniform(-0.6, 0.6, (d, Kc)).astype(np.float32)
    cb = rng.standard_normal(d).astype(np.float32) * 0.1 if with_bias else None
    n_slots = M + 3
    slots = rng.permutation(n_slots)[:M]
    pos = [0 if i % 3 == 1 else 4 + i for i in range(M)]                    # some rows start their sequence
    state0 = rng.standard_normal((n_slots, Kc - 1, d)).astype(np.float32)
    A, W = dev(a, dtype), dev(w_in, dtype)
    assert Kn.conv_step_fusable(A, W, Kc)
    opt = lambda t: None if t is None else dev(t)
    st_fused = dev(state0).clone()
    y_fused = torch.full((M, d), float("nan"), dtype=dtype, device="cuda")
    Kn.gemm_stream_conv_step(A, W, opt(b_in), dev(cw), opt(cb), st_fused, i32(pos), i32(slots), y_fused)
    # the separate kernels
    p = Kn.gemm_skinny(A, W, torch.empty((M, 3 * d), dtype=dtype, device="cuda"), opt(b_in))
    st_sep = dev(state0).clone()
    y_sep = torch.empty((M, d), dtype=dtype, device="cuda")
    Kn.shortconv_decode(p, dev(cw), opt(cb), st_sep, i32(pos), i32(slots), y_sep)
    assert torch.equal(y_fused, y_sep) and torch.equal(st_fused, st_sep)
    # the plain implementation, row by row (the product rounded to the storage type, as both paths do)
    pq = rt(P.linear(a, w_in, None if b_in is None else b_in.astype(np.float64)), dtype)
    got, new_state = y_fused.cpu().double().numpy(), st_fused.cpu().double().numpy()
    for i in range(M):
        ref, hist = conv_stream_reference(pq[i:i + 1], cw.astype(np.float64), None if cb is None else cb.astype(np.float64),
                                          state0[slots[i]].astype(np.float64), pos[i] == 0)
        np.testing.assert_allclose(got[i:i + 1], ref, rtol=tol(dtype), atol=tol(dtype), err_msg=f"row {i}")
        np.testing.assert_allclose(new_state[slots[i]], hist, rtol=1e-2, atol=1e-2, err_msg=f"state of row {i}")
    untouched = [s for s in range(n_slots) if s not in slots]
    assert np.array_equal(new_state[untouched], state0[untouched].astype(np.float64))
    assert Kn.stream_status() == 0


def test_shortconv_closed_form():
    """All-ones inputs: y_t = sum of the taps that see data, as in the reference's
    own unit test (src/test/test_hybrid.c:113-142)."""
    from kappai_b200.ops import kernels as Kn
    d, K, n = 5, 4, 9
    p = np.ones((n, 3 * d), np.float32)
    p[:, d:2 * d] = 2.0                                   # C gate
    w = np.tile(np.array([1.0, 10.0, 100.0, 1000.0], np.float32), (d, 1))
    state = torch.full((1, K - 1, d), 7.0, device="cuda")
    out = torch.empty((n, d), device="cuda")
    Kn.shortconv_forward(dev(p), dev(w), None, state, i32([0] * n), i32([0, n]), i32([0]), i32([0]), out)
    want = [2 * 1000.0, 2 * 1100.0, 2 * 1110.0] + [2 * 1111.0] * (n - 3)     # position 0: the 7s are not read
    assert np.allclose(out.cpu().numpy(), np.array(want)[:, None])


# ----------------------------------------------------- qk norm, rope, cache

def rope_ref(v, pos, rot, theta, interleaved):
    """v [n, heads, hd] float64."""
    cos, sin = P.rope_tables(int(max(pos)) + 1, rot, theta)
    out = v.copy()
    half = rot // 2
    for r, p_ in enumerate(pos):
        c, s = cos[p_], sin[p_]
        if interleaved:
            a, b = v[r, :, 0:rot:2], v[r, :, 1:rot:2]
            out[r, :, 0:rot:2], out[r, :, 1:rot:2] = a * c - b * s, a * s + b * c
        else:
            a, b = v[r, :, :half], v[r, :, half:rot]
            out[r, :, :half], out[r, :, half:rot] = a * c - b * s, a * s + b * c
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,hd,rot,inter,norm", [
    (4, 2, 16, 16, False, True), (5, 1, 48, 48, False, True), (6, 3, 128, 64, False, True),
    (3, 3, 256, 256, True, True), (8, 2, 64, 32, True, False), (7, 7, 80, 80, False, False)])
def test_qk_norm_rope_kv(dtype, H, G, hd, rot, inter, norm):
    from kappai_b200.ops import kernels as Kn
    rng = np.random.default_rng(7)
    n, page, n_pages, theta, eps = 11, 8, 6, 12345.0, 1e-5
    pos = rng.integers(0, 500, n)
    qkv = rt(rng.standard_normal((n, (H + 2 * G) * hd)) * 2, dtype)
    qw = (1 + 0.2 * rng.standard_normal(hd)).astype(np.float32)
    kw = (1 + 0.2 * rng.standard_normal(hd)).astype(np.float32)
    cos, sin = P.rope_tables(512, rot, theta)
    slots = rng.permutation(page * n_pages)[:n]
    cache0 = rng.standard_normal((n_pages, 2, G, page, hd)).astype(np.float32)
    cache = dev(cache0, dtype).clone()
    q_out = torch.empty((n, H * hd), dtype=dtype, device="cuda")
    Kn.qk_norm_rope_kv(dev(qkv, dtype), dev(qw) if norm else None, dev(kw) if norm else None, eps,
                       dev(cos.astype(np.float32)), dev(sin.astype(np.float32)), rot, inter, i32(pos), i32(slots),
                       q_out, cache, page, H, G, hd)
    q = qkv[:, :H * hd].reshape(n, H, hd)
    k = qkv[:, H * hd:(H + G) * hd].reshape(n, G, hd)
    v = qkv[:, (H + G) * hd:].reshape(n, G, hd)
    if norm:
        q, k = P.rmsnorm(q, qw.astype(np.float64), eps), P.rmsnorm(k, kw.astype(np.float64), eps)
    q, k = rope_ref(q, pos, rot, theta, inter), rope_ref(k, pos, rot, theta, inter)
    t = tol(dtype, 4)
    np.testing.assert_allclose(q_out.cpu().double().numpy().reshape(n, H, hd), q, rtol=t, atol=t)
    got = cache.cpu().double().numpy()
    want = rt(cache0, dtype)
    for r, s in enumerate(slots):
        want[s // page, 0, :, s % page, :] = k[r]
        want[s // page, 1, :, s % page, :] = v[r]
    np.testing.assert_allclose(got, want, rtol=t, atol=t)       # other slots of the cache are untouched
    # the in-place form norms and rotates q and k where they are and leaves v and the cache alone
    buf = dev(qkv, dtype).clone()
    cache2 = cache.clone()
    Kn.qk_norm_rope_kv(buf, dev(qw) if norm else None, dev(kw) if norm else None, eps, dev(cos.astype(np.float32)),
                       dev(sin.astype(np.float32)), rot, inter, i32(pos), None, None, None, page, H, G, hd)
    b = buf.cpu().double().numpy()
    np.testing.assert_allclose(b[:, :H * hd].reshape(n, H, hd), q, rtol=t, atol=t)
    np.testing.assert_allclose(b[:, H * hd:(H + G) * hd].reshape(n, G, hd), k, rtol=t, atol=t)
    assert np.array_equal(b[:, (H + G) * hd:], qkv[:, (H + G) * hd:]) and torch.equal(cache2, cache)


# -------------------------------------------------------------- attention

def paged_setup(rng, seq_lens, page, G, hd, dtype, n_pages_extra=3):
    """Random keys/values of several requests scattered over scrambled pages."""
    blocks = [-(-L // page) for L in seq_lens]
    n_pages = sum(blocks) + n_pages_extra
    perm = rng.permutation(n_pages)
    cache = rt(rng.standard_normal((n_pages, 2, G, page, hd)) * 5, dtype)      # garbage where nothing is written
    tables, ks, vs, o = [], [], [], 0
    for L, nb in zip(seq_lens, blocks):
        t = perm[o:o + nb]
        o += nb
        k = rt(rng.standard_normal((L, G, hd)), dtype)
        v = rt(rng.standard_normal((L, G, hd)), dtype)
        for pos in range(L):
            cache[t[pos // page], 0, :, pos % page, :] = k[pos]
            cache[t[pos // page], 1, :, pos % page, :] = v[pos]
        tables.append(t)
        ks.append(k)
        vs.append(v)
    bt = np.full((len(seq_lens), max(blocks)), -1, np.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = t
    return cache, bt, ks, vs


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,hd,page,window", [
    (4, 2, 16, 16, None), (5, 1, 48, 32, None), (6, 3, 64, 64, None), (8, 2, 128, 16, 40), (2, 2, 256, 8, None),
    (32, 8, 64, 64, None), (3, 1, 80, 16, 7)])
def test_attention_rows_mixed_batch(dtype, H, G, hd, page, window):
    """A batch with a whole prompt, a late portion of a long request and single
    decode rows, each checked against whole-sequence attention."""
    from kappai_b200.ops import kernels as Kn
    rng = np.random.default_rng(8)
    seq_lens = [70, 300, 129, 1, 64]
    q_from = [0, 283, 128, 0, 63]                          # rows of each segment: positions q_from..len-1
    cache, bt, ks, vs = paged_setup(rng, seq_lens, page, G, hd, dtype)
    scale = 1.0 / math.sqrt(hd)
    qs, pos, row_seg = [], [], []
    for i, (L, a) in enumerate(zip(seq_lens, q_from)):
        qs.append(rt(rng.standard_normal((L, H, hd)), dtype))
        pos += list(range(a, L))
        row_seg += [i] * (L - a)
    q_rows = np.concatenate([q[a:] for q, a in zip(qs, q_from)], 0).reshape(len(pos), H * hd)
    out = torch.empty((len(pos), H * hd), dtype=dtype, device="cuda")
    Kn.attention_rows(dev(q_rows, dtype), dev(cache, dtype), i32(bt), i32(row_seg), i32(pos), out, scale, window,
                      page, H, G, hd)
    got = out.cpu().double().numpy().reshape(len(pos), H, hd)
    r = 0
    for i, (L, a) in enumerate(zip(seq_lens, q_from)):
        ref = P.attention(qs[i], ks[i], vs[i], scale, window)[a:]
        np.testing.assert_allclose(got[r:r + L - a], ref, rtol=tol(dtype), atol=tol(dtype), err_msg=f"segment {i}")
        r += L - a


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far", [0, 63, 64, 127, 128, 511, 700])
def test_attention_finds_one_far_key(dtype, far):
    """One key among hundreds matches the query (its score stands out); the
    output must be that key's value, wherever in the pages it lies."""
    from kappai_b200.ops import kernels as Kn
    rng = np.random.default_rng(9)
    H, G, hd, page, L = 4, 2, 64, 64, 701
    cache, bt, ks, vs = paged_setup(rng, [L], page, G, hd, dtype)
    q = rt(rng.standard_normal((1, H, hd)) * 0.01, dtype)
    for h in range(H):
        q[0, h] = ks[0][far, h // (H // G)] * 8.0           # score of the far key is about 8*hd/sqrt(hd) = 64
    out = torch.empty((1, H * hd), dtype=dtype, device="cuda")
    Kn.attention_rows(dev(q.reshape(1, -1), dtype), dev(cache, dtype), i32(bt), i32([0]), i32([L - 1]), out,
                      1.0 / math.sqrt(hd), None, page, H, G, hd)
    got = out.cpu().double().numpy().reshape(H, hd)
    for h in range(H):
        np.testing.assert_allclose(got[h], vs[0][far, h // (H // G)], atol=2e-2)
    ref = P.attention(np.repeat(q, L, 0), ks[0], vs[0], 1.0 / math.sqrt(hd))[-1]
    np.testing.assert_allclose(got, ref, rtol=tol(dtype), atol=tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_window_edge(dtype):
    """The key just outside the window carries a huge value: it must not leak in;
    the key just inside must count."""
    from kappai_b200.ops import kernels as Kn
    rng = np.random.default_rng(10)
    H, G, hd, page, L, window = 2, 1, 32, 16, 100, 33
    cache, bt, ks, vs = paged_setup(rng, [L], page, G, hd, dtype)
    p = L - 1
    outside, inside = p - window, p - window + 1
    t = bt[0]
    cache[t[outside // page], 1, :, outside % page, :] = 1e4
    vs[0][outside] = 1e4
    q = rt(rng.standard_normal((1, H, hd)), dtype)
    out = torch.empty((1, H * hd), dtype=dtype, device="cuda")
    Kn.attention_rows(dev(q.reshape(1, -1), dtype), dev(cache, dtype), i32(bt), i32([0]), i32([p]), out,
                      1.0 / math.sqrt(hd), window, page, H, G, hd)
    ref = P.attention(np.repeat(q, L, 0), ks[0], vs[0], 1.0 / math.sqrt(hd), window)[-1]
    got = out.cpu().double().numpy().reshape(H, hd)
    assert np.abs(got).max() < 50
    np.testing.assert_allclose(got, ref, rtol=tol(dtype), atol=tol(dtype))
    # released pages before the window are never touched: poison their table entries
    bt2 = bt.copy()
    bt2[0, :inside // page] = -1
    out2 = torch.empty_like(out)
    Kn.attention_rows(dev(q.reshape(1, -1), dtype), dev(cache, dtype), i32(bt2), i32([0]), i32([p]), out2,
                      1.0 / math.sqrt(hd), window, page, H, G, hd)
    assert torch.equal(out, out2)


def test_kernels_refuse_what_they_cannot_do():
    from kappai_b200.ops import kernels as Kn
    x = torch.zeros((2, 8))
    with pytest.raises(Kn.KernelError, match="CUDA"):
        Kn.rmsnorm_rows(x, torch.ones(8), 1e-5, torch.empty((2, 8)))
    with pytest.raises(Kn.KernelError):
        Kn.swiglu(torch.zeros((2, 7), device="cuda"), torch.zeros((2, 4), device="cuda"))
    q = torch.zeros((1, 2 * 512), device="cuda")
    with pytest.raises(Kn.KernelError, match="not supported"):
        Kn.attention_rows(q, torch.zeros((1, 2, 1, 4, 512), device="cuda"), i32([[0]]), i32([0]), i32([0]),
                          torch.empty_like(q), 1.0, None, 4, 2, 1, 512)


# ------------------------------------------------- weight-streaming (decode) gemm

@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 17, 33, 48, 49, 64])
@pytest.mark.parametrize("N,K", [(331, 64), (2050, 2048), (96, 5632), (7, 32)])
def test_gemm_skinny(M, N, K):
    from kappai_b200.ops import kernels as Kn
    rng = np.random.default_rng(30)
    dt = torch.bfloat16
    a = rt(rng.standard_normal((M, K)), dt)
    w = rt(rng.standard_normal((N, K)) / math.sqrt(K), dt)
    b = rng.standard_normal(N).astype(np.float32)
    A, W = dev(a, dt), dev(w, dt)
    assert Kn.skinny_ok(A, W)
    ref = P.linear(a, w, b.astype(np.float64))
    out = Kn.gemm_skinny(A, W, torch.empty((M, N), dtype=torch.float32, device="cuda"), dev(b))
    np.testing.assert_allclose(out.cpu().double().numpy(), ref, rtol=2e-5, atol=2e-5 * math.sqrt(K))
    out16 = Kn.gemm_skinny(A, W, torch.empty((M, N), dtype=dt, device="cuda"), dev(b))
    np.testing.assert_allclose(out16.cpu().double().numpy(), ref, rtol=1e-2, atol=2e-2)
    res = rng.standard_normal((M, N)).astype(np.float32)
    acc = dev(res).clone()
    Kn.gemm_skinny(A, W, acc, None, accumulate=True)
    np.testing.assert_allclose(acc.cpu().double().numpy(), res + P.linear(a, w), rtol=2e-5, atol=2e-5 * math.sqrt(K))
    # the same row alone gives the same bits
    r = M // 2
    alone = Kn.gemm_skinny(A[r:r + 1], W, torch.empty((1, N), dtype=torch.float32, device="cuda"), dev(b))
    assert torch.equal(alone[0], out[r])


@pytest.mark.parametrize("M", [1, 8, 20, 64])
@pytest.mark.parametrize("ff,K", [(100, 64), (5632, 2048), (333, 96)])
def test_gemm_skinny_swiglu(M, ff, K):
    from kappai_b200.ops import kernels as Kn
    from kappai_b200.ops.linear import linear_swiglu
    rng = np.random.default_rng(31)
    dt = torch.bfloat16
    a = rt(rng.standard_normal((M, K)), dt)
    w = rt(rng.standard_normal((2 * ff, K)) * (2.0 / math.sqrt(K)), dt)
    b = rng.standard_normal(2 * ff).astype(np.float32) * 0.1
    gu = rt(P.linear(a, w, b.astype(np.float64)), dt)              # gate and up are stored in bfloat16
    ref = P.swiglu(gu[:, :ff], gu[:, ff:])
    for bias in (dev(b), None):
        if bias is None:
            gu = rt(P.linear(a, w), dt)
            ref = P.swiglu(gu[:, :ff], gu[:, ff:])
        out = linear_swiglu(dev(a, dt), dev(w, dt), bias)
        assert out.shape == (M, ff) and out.dtype == dt
        np.testing.assert_allclose(out.cpu().double().numpy(), ref, rtol=2e-2, atol=2e-2)
        # fused and unfused agree to the last bfloat16 rounding
        unf = Kn.swiglu(Kn.gemm_nt_simt(dev(a, dt), dev(w, dt), torch.empty((M, 2 * ff), dtype=dt, device="cuda"), bias),
                        torch.empty((M, ff), dtype=dt, device="cuda"))
        assert ((out.float() - unf.float()).abs() <= 2e-2 * unf.float().abs() + 2e-2).all().item()
