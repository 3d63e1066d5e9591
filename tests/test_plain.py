"""The plain implementation against itself: properties that hold whatever the weights (no GPU)."""
import numpy as np

import plain_lfm2 as P


def test_causality_and_prefix_consistency(plain_models):
    """Logits at a position depend only on the tokens up to it."""
    for name, m in plain_models.items():
        rng = np.random.default_rng(0)
        t = rng.integers(0, m.cfg["vocab_size"], 40).tolist()
        full = m.logits(t)
        np.testing.assert_allclose(m.logits(t[:17]), full[:17], rtol=1e-9, atol=1e-11)
        t2 = list(t)
        t2[30] = (t2[30] + 1) % m.cfg["vocab_size"]
        np.testing.assert_allclose(m.logits(t2)[:30], full[:30], rtol=1e-9, atol=1e-11)
        assert np.abs(m.logits(t2)[30:] - full[30:]).max() > 1e-6


def test_intermediate_size():
    assert P.intermediate_size(dict(block_ff_dim=8192, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0,
                                    block_multiple_of=256)) == 5632
    assert P.intermediate_size(dict(block_ff_dim=192)) == 192


def test_window_attention_equals_full_inside_the_window():
    rng = np.random.default_rng(1)
    q, k, v = rng.standard_normal((20, 2, 8)), rng.standard_normal((20, 1, 8)), rng.standard_normal((20, 1, 8))
    full = P.attention(q, k, v, 0.3)
    win = P.attention(q, k, v, 0.3, window=6)
    np.testing.assert_allclose(win[:6], full[:6])
    assert np.abs(win[10] - full[10]).max() > 1e-6
    np.testing.assert_allclose(win[10], P.attention(q[5:11], k[5:11], v[5:11], 0.3)[-1])


def test_float32_mode_is_close_to_float64(model_dirs):
    m64, m32 = P.PlainLfm2(model_dirs["A"]), P.PlainLfm2(model_dirs["A"], dtype=np.float32)
    t = list(range(30))
    assert np.abs(m64.logits(t) - m32.logits(t)).max() < 1e-5
