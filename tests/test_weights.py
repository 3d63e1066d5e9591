"""Weights: the safetensors container, the loader's one error, random weights (no GPU)."""
import json
import os

import numpy as np
import pytest
import torch

from kappai_b200.config import config_from_dict
from kappai_b200.engine.model import Model
from kappai_b200.parts.base import BuildEnv
from kappai_b200.weights import (SafetensorsFile, SafetensorsError, WeightError, load_weights, random_weights,
                                 save_safetensors, write_random_model)
from kappai_b200.weights.loader import _convert
from tiny_configs import TINY_A, TINY_B


def _model(cfg, dtype=torch.float32):
    arch, c = config_from_dict(cfg)
    return Model(arch.build_spec(c), BuildEnv(torch.device("cpu"), dtype, max_positions=8))


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
         "h": torch.randn(4).to(torch.float16)}
    p = str(tmp_path / "x.safetensors")
    save_safetensors(p, t, {"k": "v"})
    with SafetensorsFile(p) as f:
        assert set(f.keys()) == set(t) and f.metadata == {"k": "v"}
        for k, v in t.items():
            assert f.info(k) == (v.dtype, tuple(v.shape))
            assert torch.equal(f.tensor(k), v)


def test_safetensors_bad_files(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 8)       # data shorter than claimed
    with pytest.raises(SafetensorsError, match="'w'"):
        SafetensorsFile(str(p))


def test_random_weights_are_seeded_and_order_free(tmp_path):
    a = random_weights(TINY_A, 0)
    b = random_weights(TINY_A, 0)
    c = random_weights(TINY_A, 1)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    # a tensor's values depend on (seed, name) only: the same name in another model has the same head
    big = random_weights(TINY_B, 0)
    n = "model.embedding_norm.weight"
    assert torch.equal(a[n][:8], big[n][:8]) or a[n].numel() != big[n].numel()
    # storage dtypes and distributions by role
    assert a["model.layers.0.conv.in_proj.weight"].dtype == torch.bfloat16
    assert a["model.layers.0.conv.conv.weight"].dtype == torch.float32
    assert a["model.layers.0.operator_norm.weight"].dtype == torch.float32
    assert abs(a["model.embed_tokens.weight"].float().std().item() - 0.02) < 2e-3
    assert abs(a["model.layers.0.operator_norm.weight"].mean().item() - 1.0) < 0.05
    assert a["model.layers.0.conv.conv.weight"].abs().max().item() <= 1 / np.sqrt(3) + 1e-6
    bb = random_weights(TINY_B, 1)
    assert "model.layers.1.conv.conv.bias" in bb and "lm_head.weight" in bb
    assert "lm_head.weight" not in a


def test_tensor_names_of_lfm2():
    names = set(_model(TINY_B).weight_table())
    for n in ["model.embed_tokens.weight", "model.embedding_norm.weight", "lm_head.weight",
              "model.layers.0.operator_norm.weight", "model.layers.0.ffn_norm.weight",
              "model.layers.0.self_attn.q_proj.weight", "model.layers.0.self_attn.k_proj.weight",
              "model.layers.0.self_attn.v_proj.weight", "model.layers.0.self_attn.out_proj.weight",
              "model.layers.0.self_attn.q_layernorm.weight", "model.layers.0.self_attn.k_layernorm.weight",
              "model.layers.1.conv.in_proj.weight", "model.layers.1.conv.conv.weight",
              "model.layers.1.conv.out_proj.weight", "model.layers.1.conv.in_proj.bias",
              "model.layers.1.conv.conv.bias", "model.layers.1.conv.out_proj.bias",
              "model.layers.5.feed_forward.w1.weight", "model.layers.5.feed_forward.w2.weight",
              "model.layers.5.feed_forward.w3.weight"]:
        assert n in names, n
    assert "model.layers.0.conv.in_proj.weight" not in names      # layer 0 of B is attention


def test_loader_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = str(tmp_path / "m")
    write_random_model(TINY_A, d, 0)
    with SafetensorsFile(os.path.join(d, "model.safetensors")) as f:
        t = {k: f.tensor(k) for k in f.keys()}
    del t["model.layers.1.self_attn.q_layernorm.weight"]
    del t["model.layers.0.conv.conv.weight"]
    t["model.layers.0.conv.extra.weight"] = torch.zeros(2)
    t["model.layers.3.feed_forward.w2.weight"] = torch.zeros(5, 5).to(torch.bfloat16)
    save_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightError) as e:
        load_weights(_model(TINY_A), d)
    msg = str(e.value)
    assert "model.layers.1.self_attn.q_layernorm.weight" in msg and "model.layers.0.conv.conv.weight" in msg
    assert "model.layers.0.conv.extra.weight" in msg
    assert "model.layers.3.feed_forward.w2.weight" in msg and "[5, 5]" in msg and "[64, 192]" in msg
    assert e.value.missing == sorted(["model.layers.1.self_attn.q_layernorm.weight", "model.layers.0.conv.conv.weight"])
    assert e.value.unexpected == ["model.layers.0.conv.extra.weight"]
    assert len(e.value.wrong_shape) == 1


def test_loader_no_file(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    with pytest.raises(WeightError, match="safetensors"):
        load_weights(_model(TINY_A), str(tmp_path))


def test_dtype_rules():
    bf = torch.randn(4).to(torch.bfloat16)
    assert _convert(bf, torch.bfloat16).dtype == torch.bfloat16
    assert _convert(bf, torch.float32).dtype == torch.float32
    assert torch.equal(_convert(bf, torch.float32), bf.float())            # the bfloat16 values, widened
    f32 = torch.randn(4)
    assert _convert(f32, torch.bfloat16).dtype == torch.float32            # stored in 32-bit stays so
    assert _convert(torch.randn(4).half(), torch.bfloat16).dtype == torch.float32
    assert _convert(torch.arange(4), torch.bfloat16).dtype == torch.int32


def test_load_binds_and_ties(tmp_path):
    d = str(tmp_path / "m")
    write_random_model(TINY_A, d, 0)
    m = _model(TINY_A, torch.bfloat16)
    load_weights(m, d)
    assert m.head.weight is m.embedding.weight and m.embedding.weight.dtype == torch.bfloat16
    assert m.blocks[0].mixer.w_conv.shape == (64, 3) and m.blocks[0].mixer.w_conv.dtype == torch.float32
    assert m.blocks[1].mixer.w_qkv.shape == ((4 + 2 + 2) * 16, 64)
    assert m.blocks[0].ffn.w_gu.shape == (2 * 192, 64)
    m32 = _model(TINY_A, torch.float32)
    load_weights(m32, d)
    assert m32.embedding.weight.dtype == torch.float32
    assert torch.equal(m32.embedding.weight, m.embedding.weight.float())
