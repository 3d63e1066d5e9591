"""The plain implementation against outputs of the reference's own C kernels
(tests/golden/golden.npz, made by tests/golden/make_golden.py from the
reference's source tree), part by part.  No GPU."""
import os

import numpy as np
import pytest

import plain_lfm2 as P
import plain_sampler as PS

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden.npz"))
f64 = lambda k: G[k].astype(np.float64)


@pytest.mark.parametrize("i", range(3))
def test_rmsnorm(i):
    y = P.rmsnorm(f64(f"rmsnorm{i}_x"), f64(f"rmsnorm{i}_w"), float(G[f"rmsnorm{i}_eps"]))
    np.testing.assert_allclose(y, f64(f"rmsnorm{i}_y"), rtol=2e-6, atol=1e-6)


def test_rmsnorm_per_head():
    y = P.rmsnorm(f64("perhead_x").reshape(3, 16), f64("perhead_w"), 1e-5).reshape(-1)
    np.testing.assert_allclose(y, f64("perhead_y"), rtol=2e-6, atol=1e-6)


@pytest.mark.parametrize("i", range(2))
def test_rope_table_and_rotation(i):
    pos = G[f"rope{i}_positions"]
    hd = G[f"rope{i}_cos"].shape[1] * 2
    cos, sin = P.rope_tables(int(pos.max()) + 1, hd, float(G[f"rope{i}_theta"]))
    # the reference steps the angle by a recurrence in double and stores float32
    np.testing.assert_allclose(cos[pos], f64(f"rope{i}_cos"), atol=2e-7)
    np.testing.assert_allclose(sin[pos], f64(f"rope{i}_sin"), atol=2e-7)
    p = int(G[f"rope{i}_pos"])
    v = f64(f"rope{i}_v")[None]                      # [1, heads, hd]
    rot = P.rope_neox(v, cos[p:p + 1], sin[p:p + 1])[0]
    np.testing.assert_allclose(rot, f64(f"rope{i}_rot"), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("i", range(4))
def test_shortconv_whole_sequence_equals_reference_in_two_chunks(i):
    mixed, w = f64(f"conv{i}_mixed"), f64(f"conv{i}_w")
    y = P.shortconv(mixed, w)
    np.testing.assert_allclose(y, f64(f"conv{i}_out"), rtol=1e-5, atol=1e-6)
    # the reference's final state is the last K-1 values of B*X, oldest first, stored [dim][K-1]
    d, K = w.shape
    bx = mixed[:, :d] * mixed[:, 2 * d:]
    padded = np.concatenate([np.zeros((K - 1, d)), bx])
    np.testing.assert_allclose(padded[-(K - 1):].T, f64(f"conv{i}_state"), rtol=1e-6, atol=1e-7)
    r1 = int(G[f"conv{i}_r1"])
    np.testing.assert_allclose(padded[r1:r1 + K - 1].T, f64(f"conv{i}_mid"), rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("i", range(4))
def test_attention_over_the_cache(i):
    k, v, q = f64(f"attn{i}_k16"), f64(f"attn{i}_v16"), f64(f"attn{i}_q")
    n, hd = k.shape
    qq = np.zeros((n, 1, hd))
    qq[-1, 0] = q                                   # the query sits at the last position and sees every key
    o = P.attention(qq, k[:, None, :], v[:, None, :], 1.0 / np.sqrt(hd))[-1, 0]
    np.testing.assert_allclose(o, f64(f"attn{i}_out1"), rtol=2e-5, atol=2e-6)      # online softmax
    np.testing.assert_allclose(o, f64(f"attn{i}_out0"), rtol=2e-5, atol=2e-6)      # scores, softmax, sum


def test_swiglu():
    np.testing.assert_allclose(P.swiglu(f64("swiglu_g"), f64("swiglu_u")), f64("swiglu_o"), rtol=2e-6, atol=1e-7)


def test_argmax_and_sampler():
    assert PS.argmax(G["argmax_l"]) == int(G["argmax_i"]) == 7
    logits = G["sample_logits"].astype(np.float32)
    differ = 0
    for l, (t, k, p, m, u, tok) in zip(logits, G["sample_rows"]):
        got, slack = PS.sample(l, float(u), temperature=float(t), top_k=int(k), top_p=float(p), min_p=float(m))
        if got != int(tok):
            assert slack < 1e-6, (t, k, p, m, got, tok, slack)
            differ += 1
    assert differ <= 1


# ------------------------------------------------------------------ whole models through the reference's own code
# The reference keeps keys and values in 16-bit floats (src/backend/backend.h:143-149) and sums in float32; the plain
# implementation is float64 throughout.  Logits of these models have a standard deviation of about 0.2; the two
# agree to about 1.5e-4, and 5e-4 is the bound (the reference's own bar between its backends is 4e-3,
# src/test/test_hybrid.c:205).
MODEL_ATOL = 5e-4


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_models_against_the_reference(name, tmp_path):
    """The reference's loader, recipe and CPU backend ran these models (tests/golden/make_golden.py wrote them as
    GGUF files from the same random weights) whole, token by token and in portions; the plain implementation
    gives the same logits.  Model B is Tiny B without its biases, which the reference's LFM2 does not have; model
    C is Tiny C with hidden 240, so that head_dim = hidden / heads as in every real LFM2 (tests/golden/make_golden.py
    says what the reference does otherwise)."""
    from kappai_b200.weights import write_random_model
    from plain_lfm2 import PlainLfm2
    from tiny_configs import CONFIGS
    override = {"B": {"conv_bias": False}, "C": {"hidden_size": 240}}.get(name, {})
    cfg, seed = CONFIGS[name]
    d = str(tmp_path / "m")
    write_random_model(dict(cfg, **override), d, seed)
    toks = G[f"model{name}_tokens"].tolist()
    logits = PlainLfm2(d).logits(toks)
    n_rows = 0
    for cut in ("whole", "each", "portions"):
        pos, want = G[f"model{name}_{cut}_positions"], G[f"model{name}_{cut}_logits"]
        assert len(pos) == len(want) and len(pos) >= 1
        err = np.abs(logits[pos] - want).max()
        assert err <= MODEL_ATOL, f"model {name}, cut '{cut}': plain and reference differ by {err:.3e}"
        n_rows += len(pos)
    assert n_rows >= 15 and float(np.std(want)) > 0.05
