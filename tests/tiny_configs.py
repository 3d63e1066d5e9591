"""Tiny LFM2 configurations that differ in every size and option, and
helpers that write them as model folders with random weights."""
import os
import tempfile

TINY_A = dict(
    architectures=["Lfm2ForCausalLM"], vocab_size=256, hidden_size=64, num_hidden_layers=4,
    num_attention_heads=4, num_key_value_heads=2,
    layer_types=["conv", "full_attention", "conv", "full_attention"],
    max_position_embeddings=128, norm_eps=1e-5, conv_L_cache=3, conv_bias=False,
    block_ff_dim=192, block_auto_adjust_ff_dim=False, rope_theta=10000.0, tie_embedding=True)
TINY_A_SEED = 0

TINY_B = dict(
    architectures=["Lfm2ForCausalLM"], vocab_size=512, hidden_size=96, num_hidden_layers=6,
    num_attention_heads=6, num_key_value_heads=3,
    layer_types=["full_attention", "conv", "conv", "full_attention", "conv", "conv"],
    max_position_embeddings=256, norm_eps=1e-6, conv_L_cache=4, conv_bias=True,
    block_ff_dim=384, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0, block_multiple_of=32,
    rope_theta=1000000.0, tie_embedding=False)
TINY_B_SEED = 1

# a third shape: sizes that are no power of two, head_dim 48 given explicitly (not hidden/heads),
# one kv head, an odd vocabulary, K = 2
TINY_C = dict(
    architectures=["Lfm2ForCausalLM"], vocab_size=331, hidden_size=120, num_hidden_layers=3,
    num_attention_heads=5, num_key_value_heads=1, head_dim=48,
    layer_types=["conv", "full_attention", "full_attention"],
    max_position_embeddings=512, norm_eps=1e-5, conv_L_cache=2, conv_bias=False,
    block_ff_dim=200, block_auto_adjust_ff_dim=False, rope_theta=50000.0, tie_embedding=True)
TINY_C_SEED = 7

# a fourth shape with head size 64, where the tensor-core attention kernels run (tcgen05 for prompt portions,
# the TMA-fed split kernel for decoded tokens); two query heads share the one kv head
TINY_D = dict(
    architectures=["Lfm2ForCausalLM"], vocab_size=300, hidden_size=128, num_hidden_layers=3,
    num_attention_heads=2, num_key_value_heads=1,
    layer_types=["full_attention", "conv", "full_attention"],
    max_position_embeddings=1024, norm_eps=1e-5, conv_L_cache=3, conv_bias=True,
    block_ff_dim=256, block_auto_adjust_ff_dim=False, rope_theta=10000.0, tie_embedding=True)
TINY_D_SEED = 9

# the LFM2-1.2B shape (for the tests that run the sizes the benchmark times)
LFM2_1P2B = dict(
    architectures=["Lfm2ForCausalLM"], vocab_size=65536, hidden_size=2048, num_hidden_layers=16,
    num_attention_heads=32, num_key_value_heads=8,
    layer_types=["conv", "conv", "full_attention", "conv", "conv", "full_attention", "conv", "conv",
                 "full_attention", "conv", "full_attention", "conv", "full_attention", "conv",
                 "full_attention", "conv"],
    max_position_embeddings=128000, norm_eps=1e-5, conv_L_cache=3, conv_bias=False,
    block_ff_dim=8192, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0, block_multiple_of=256,
    rope_theta=1000000.0, tie_embedding=True)
LFM2_1P2B_SEED = 2

CONFIGS = {"A": (TINY_A, TINY_A_SEED), "B": (TINY_B, TINY_B_SEED), "C": (TINY_C, TINY_C_SEED),
           "D": (TINY_D, TINY_D_SEED)}


def make_model_dir(name, root=None):
    from kappai_b200.weights import write_random_model

    cfg, seed = CONFIGS[name]
    d = tempfile.mkdtemp(prefix=f"tiny_{name}_", dir=root)
    write_random_model(cfg, d, seed)
    return d
