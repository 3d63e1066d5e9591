"""A few thousand tokens at head size 64, where the tensor-core attention kernels run (tcgen05 for the
prompt portions, the TMA-fed split kernel for the decoded tokens): a prompt cut into portions of odd sizes
that start anywhere, then tokens one by one, in 32-bit and in bfloat16, against the plain implementation."""
import numpy as np
import pytest

from tolerances import tol_for

pytestmark = pytest.mark.gpu

CONFIG = {'architectures': ['Lfm2ForCausalLM'], 'vocab_size': 384, 'hidden_size': 256, 'num_hidden_layers': 3,
          'num_attention_heads': 4, 'num_key_value_heads': 2, 'layer_types': ['conv', 'full_attention', 'full_attention'],
          'max_position_embeddings': 8192, 'norm_eps': 1e-05, 'conv_L_cache': 3, 'conv_bias': False,
          'block_ff_dim': 320, 'block_auto_adjust_ff_dim': False, 'rope_theta': 1000000.0, 'tie_embedding': True}


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    from kappai_b200 import write_random_model
    from plain_lfm2 import PlainLfm2
    d = str(tmp_path_factory.mktemp("long") / "m")
    write_random_model(CONFIG, d, 11)
    return d, PlainLfm2(d)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompt_in_odd_portions_then_decoding(dtype, model):
    from kappai_b200 import ModelRunner, StepEntry
    from kappai_b200.ops import kernels as K
    d, plain = model
    rng = np.random.default_rng(3)
    T, n_dec = 3000, 6
    toks = rng.integers(0, CONFIG["vocab_size"], T + n_dec).tolist()
    ref = plain.logits(toks)
    r = ModelRunner(d, dtype=dtype, max_tokens=4096, max_requests=2, page_size=64, max_model_len=4096)
    cuts = [0, 129, 700, 701, 1500, 2047, 2048, 2900, T]                 # portions of 129, 571, 1, 799, ... tokens
    tol = tol_for(dtype, ref)
    for a, b in zip(cuts[:-1], cuts[1:]):
        want = sorted({0, (b - a) // 2, b - a - 1})
        lg = r.step([StepEntry("a", toks[a:b], want)]).float().cpu().numpy()
        for j, w in enumerate(want):
            assert np.abs(lg[j] - ref[a + w]).max() <= tol, (dtype, a, b, w)
    for i in range(n_dec):
        lg = r.step([StepEntry("a", [toks[T + i]], [0])]).float().cpu().numpy()
        assert np.abs(lg[0] - ref[T + i]).max() <= tol, (dtype, "decode", i)
    assert K.tc_status() == 0 and K.stream_status() == 0 and K.attention_tc_status() == 0
