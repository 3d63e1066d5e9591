"""Each part alone (norm, position encoding, attention, short convolution,
feed-forward, embedding/head, block) against the plain functions, with sizes
and options other than the tiny models' (windows, biases, partial rotary,
interleaved pairs, no qk norm), in a batch of several segments."""
import math

import numpy as np
import pytest
import torch

import plain_lfm2 as P

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def env_for(dtype, max_pos=512):
    from kappai_b200.parts import BuildEnv
    return BuildEnv(torch.device("cuda:0"), dtype, max_pos)


def bind_random(part, rng, dtype):
    """Random weights in the part's declared shapes; returns them as float64 numpy (the stored values)."""
    ws, vals = {}, {}
    for name, spec in part.weight_specs().items():
        if spec.role == "norm":
            a = 1 + 0.1 * rng.standard_normal(spec.shape)
        elif spec.role == "conv":
            a = rng.uniform(-0.5, 0.5, spec.shape)
        elif spec.role == "bias":
            a = 0.1 * rng.standard_normal(spec.shape)
        else:
            a = rng.standard_normal(spec.shape) / math.sqrt(spec.shape[-1])
        store = dtype if spec.role in ("matrix", "embedding") else torch.float32
        t = torch.as_tensor(a.astype(np.float32)).to(store)
        ws[name] = t.cuda()
        vals[name] = t.double().numpy()
    part.bind(ws)
    return vals


def rt(a, dtype):
    return torch.as_tensor(np.asarray(a, dtype=np.float32)).to(dtype).double().numpy()


class Batch:
    """Several requests, each cut in two steps; builds StepContexts through the real cache manager."""

    def __init__(self, specs, lens, cuts, page, dtype):
        from kappai_b200.cache import CacheManager, PagedKVSpec
        from kappai_b200.cache.storage import CacheStorage
        self.lens, self.cuts, self.page = lens, cuts, page
        gks = {s.group_key: s for s in specs if isinstance(s, PagedKVSpec)}
        n_pages = sum(-(-L // page) for L in lens) + 2
        self.storage = CacheStorage(specs, [None] * len(specs), {g: n_pages for g in gks}, page, len(lens) + 1,
                                    dtype, torch.device("cuda:0"))
        self.cache = CacheManager({g: (n_pages, page, s.window) for g, s in gks.items()}, len(lens) + 1)
        self.groups = {g: page for g in gks}
        for i in range(len(lens)):
            self.cache.admit(i)

    def context(self, step):
        from kappai_b200.engine.batch import Segment, build_step_context
        segs = []
        for i, (L, c) in enumerate(zip(self.lens, self.cuts)):
            a, b = (0, c) if step == 0 else (c, L)
            if b <= a:
                continue
            self.cache.extend(i, b)
            rc = self.cache.requests[i]
            segs.append(Segment(i, [0] * (b - a), a, [], rc.slot,
                                {g: self.cache.block_table(i, g) for g in self.groups},
                                {g: self.cache.token_slots(i, g, a, b - a) for g in self.groups}))
        ctx = build_step_context(segs, self.groups, torch.device("cuda:0"), 10, 4096)
        rows = [(s.req, s.pos_start, len(s.tokens)) for s in segs]
        for s in segs:
            self.cache.advance(s.req, s.pos_start + len(s.tokens))
        return ctx, rows


def run_mixer_two_steps(mixer, h_all, lens, cuts, page, dtype):
    """Run each request's rows 0..cut in step 0 and cut..len in step 1 (all requests in one batch);
    returns the mixer's output (what it adds to a zero residual) per request."""
    d = h_all[0].shape[1]
    b = Batch([mixer.cache_spec()], lens, cuts, page, dtype)
    outs = [np.zeros((L, d)) for L in lens]
    for step in (0, 1):
        ctx, rows = b.context(step)
        h = np.concatenate([h_all[i][a:a + n] for i, a, n in rows], 0)
        res = torch.zeros((h.shape[0], d), dtype=torch.float32, device="cuda")
        mixer.forward(torch.as_tensor(h.astype(np.float32)).to(dtype).cuda(), res, ctx, b.storage.views[0])
        r = 0
        got = res.cpu().double().numpy()
        for i, a, n in rows:
            outs[i][a:a + n] = got[r:r + n]
            r += n
    return outs


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("opts", [
    dict(H=4, G=2, hd=16, window=None, qk=1e-5, rot=16, pairing="neox", bias=False, page=16),
    dict(H=5, G=1, hd=48, window=None, qk=None, rot=24, pairing="interleaved", bias=True, page=32),
    dict(H=6, G=3, hd=32, window=21, qk=1e-6, rot=32, pairing="neox", bias=False, page=8),
    dict(H=2, G=2, hd=128, window=None, qk=1e-5, rot=0, pairing="neox", bias=False, page=64),
])
def test_attention_part(dtype, opts):
    from kappai_b200.config import PartSpec
    from kappai_b200.parts import make_part
    rng = np.random.default_rng(0)
    H, G, hd, d = opts["H"], opts["G"], opts["hd"], 72
    scale, theta = 0.9 / math.sqrt(hd), 5000.0
    pos = PartSpec("rope", {"rotary_dim": opts["rot"], "theta": theta, "pairing": opts["pairing"]}) \
        if opts["rot"] else PartSpec("none")
    mixer = make_part("mixer", PartSpec("attention", dict(
        hidden_size=d, num_heads=H, num_kv_heads=G, head_dim=hd, scale=scale, qk_norm_eps=opts["qk"],
        window=opts["window"], position=pos, bias=opts["bias"])), env_for(dtype))
    w = bind_random(mixer, rng, dtype)
    lens, cuts = [50, 9, 131, 1], [33, 0, 129, 1]
    h_all = [rt(rng.standard_normal((L, d)), dtype) for L in lens]
    outs = run_mixer_two_steps(mixer, h_all, lens, cuts, opts["page"], dtype)
    for i, L in enumerate(lens):
        h = h_all[i]
        b = (lambda n: w[n + ".bias"]) if opts["bias"] else (lambda n: None)
        q = P.linear(h, w["q_proj.weight"], b("q_proj")).reshape(L, H, hd)
        k = P.linear(h, w["k_proj.weight"], b("k_proj")).reshape(L, G, hd)
        v = P.linear(h, w["v_proj.weight"], b("v_proj")).reshape(L, G, hd)
        if opts["qk"] is not None:
            q, k = P.rmsnorm(q, w["q_norm.weight"], opts["qk"]), P.rmsnorm(k, w["k_norm.weight"], opts["qk"])
        if opts["rot"]:
            from test_kernels_gpu import rope_ref
            q = rope_ref(q, list(range(L)), opts["rot"], theta, opts["pairing"] == "interleaved")
            k = rope_ref(k, list(range(L)), opts["rot"], theta, opts["pairing"] == "interleaved")
        o = P.attention(q, k, v, scale, opts["window"]).reshape(L, H * hd)
        ref = P.linear(o, w["out_proj.weight"], b("out_proj"))
        t = 3e-5 if dtype == torch.float32 else 0.05 * ref.std()
        err = np.abs(outs[i] - ref).max()
        assert err <= t, f"request {i}: {err} > {t}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,K,bias", [(40, 2, False), (64, 3, True), (100, 5, False)])
def test_shortconv_part(dtype, d, K, bias):
    from kappai_b200.config import PartSpec
    from kappai_b200.parts import make_part
    rng = np.random.default_rng(1)
    mixer = make_part("mixer", PartSpec("shortconv", dict(hidden_size=d, kernel_size=K, bias=bias)), env_for(dtype))
    w = bind_random(mixer, rng, dtype)
    lens, cuts = [40, 3, 2, 17], [39, 1, 0, 2]
    h_all = [rt(rng.standard_normal((L, d)), dtype) for L in lens]
    outs = run_mixer_two_steps(mixer, h_all, lens, cuts, 16, dtype)
    for i, L in enumerate(lens):
        b = (lambda n: w[n + ".bias"]) if bias else (lambda n: None)
        y = P.shortconv(P.linear(h_all[i], w["in_proj.weight"], b("in_proj")), w["conv.weight"], b("conv"))
        ref = P.linear(y, w["out_proj.weight"], b("out_proj"))
        t = 3e-5 if dtype == torch.float32 else 0.05 * ref.std()
        err = np.abs(outs[i] - ref).max()
        assert err <= t, f"request {i}: {err} > {t}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,ff,bias", [(40, 100, False), (96, 333, True)])
def test_swiglu_part(dtype, d, ff, bias):
    from kappai_b200.config import PartSpec
    from kappai_b200.parts import make_part
    rng = np.random.default_rng(2)
    ffn = make_part("feed_forward", PartSpec("swiglu", dict(hidden_size=d, intermediate_size=ff, bias=bias)),
                    env_for(dtype))
    w = bind_random(ffn, rng, dtype)
    h = rt(rng.standard_normal((13, d)), dtype)
    res0 = rng.standard_normal((13, d)).astype(np.float32)
    res = torch.as_tensor(res0).cuda()
    ffn.forward(torch.as_tensor(h.astype(np.float32)).to(dtype).cuda(), res, None)
    b = (lambda n: w[n + ".bias"]) if bias else (lambda n: None)
    ref = res0 + P.linear(P.swiglu(P.linear(h, w["gate_proj.weight"], b("gate_proj")),
                                   P.linear(h, w["up_proj.weight"], b("up_proj"))), w["down_proj.weight"], b("down_proj"))
    t = 3e-5 if dtype == torch.float32 else 0.05
    assert np.abs(res.cpu().double().numpy() - ref).max() <= t


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_embedding_head_parts(dtype):
    from kappai_b200.config import PartSpec
    from kappai_b200.parts import make_part
    rng = np.random.default_rng(3)
    V, d = 331, 56
    env = env_for(dtype)
    emb = make_part("embedding", PartSpec("embedding", dict(vocab_size=V, hidden_size=d, scale=None)), env)
    we = bind_random(emb, rng, dtype)
    norm = make_part("norm", PartSpec("rmsnorm", dict(size=d, eps=1e-6)), env)
    wn = bind_random(norm, rng, dtype)
    tied = make_part("head", PartSpec("lm_head", dict(vocab_size=V, hidden_size=d, tied=True)), env)
    tied.tie(emb)
    free = make_part("head", PartSpec("lm_head", dict(vocab_size=V, hidden_size=d, tied=False)), env)
    wh = bind_random(free, rng, dtype)
    ids = rng.integers(0, V, 9)
    x = emb.forward(torch.as_tensor(ids.astype(np.int32)).cuda())
    assert np.array_equal(x.cpu().double().numpy(), we["weight"][ids])
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device="cuda")
    h = norm.forward(x, rows=rows)
    href = P.rmsnorm(we["weight"][ids][[8, 0, 3]], wn["weight"], 1e-6)
    t = 2e-5 if dtype == torch.float32 else 1.5e-2
    np.testing.assert_allclose(h.cpu().double().numpy(), href, rtol=t, atol=t)
    hh = h.cpu().double().numpy()
    for head, W in ((tied, we["weight"]), (free, wh["weight"])):
        lg = head.forward(h)
        assert lg.dtype == torch.float32 and lg.shape == (3, V)
        np.testing.assert_allclose(lg.cpu().double().numpy(), hh @ W.T, rtol=2e-5, atol=2e-4)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prenorm_block(dtype):
    """The block arrangement: x += mixer(norm1(x)); x += ffn(norm2(x))."""
    from kappai_b200.config import PartSpec
    from kappai_b200.parts import make_part
    rng = np.random.default_rng(4)
    d, K, ff, L = 48, 3, 80, 21
    env = env_for(dtype)
    mixer = make_part("mixer", PartSpec("shortconv", dict(hidden_size=d, kernel_size=K, bias=False)), env)
    ffn = make_part("feed_forward", PartSpec("swiglu", dict(hidden_size=d, intermediate_size=ff)), env)
    n1 = make_part("norm", PartSpec("rmsnorm", dict(size=d, eps=1e-5)), env)
    n2 = make_part("norm", PartSpec("rmsnorm", dict(size=d, eps=1e-5)), env)
    wm, wf, w1, w2 = (bind_random(p, rng, dtype) for p in (mixer, ffn, n1, n2))
    block = make_part("block", PartSpec("prenorm_residual"), env).assemble(mixer, ffn, n1, n2)
    b = Batch([mixer.cache_spec()], [L], [L], 16, dtype)
    ctx, _ = b.context(0)
    x0 = rng.standard_normal((L, d)).astype(np.float32)
    x = torch.as_tensor(x0).cuda()
    block.forward(x, ctx, b.storage.views[0])
    xr = x0.astype(np.float64)
    h = P.rmsnorm(xr, w1["weight"], 1e-5)
    xr = xr + P.linear(P.shortconv(P.linear(h, wm["in_proj.weight"]), wm["conv.weight"]), wm["out_proj.weight"])
    h = P.rmsnorm(xr, w2["weight"], 1e-5)
    xr = xr + P.linear(P.swiglu(P.linear(h, wf["gate_proj.weight"]), P.linear(h, wf["up_proj.weight"])),
                       wf["down_proj.weight"])
    t = 3e-5 if dtype == torch.float32 else 0.06
    assert np.abs(x.cpu().double().numpy() - xr).max() <= t
