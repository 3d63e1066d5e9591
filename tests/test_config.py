"""Configuration and registry (no GPU)."""
import copy
import json
import os

import pytest

from kappai_b200.config import (ConfigError, config_from_dict, load_config, lookup_architecture,
                                architecture_names, register_architecture, unregister_architecture,
                                TypedConfig, cfg, ModelSpec, PartSpec, LayerSpec, ScheduleEntry)
from tiny_configs import TINY_A, TINY_B, TINY_C


def test_registry_knows_lfm2_and_names_unknown():
    assert "Lfm2ForCausalLM" in architecture_names()
    with pytest.raises(ConfigError, match="NopeForCausalLM"):
        lookup_architecture("NopeForCausalLM")
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({"hidden_size": 8})


@pytest.mark.parametrize("block_ff,mult,multiple,want", [
    (8192, 1.0, 256, 5632), (10752, 1.0, 256, 7168), (6656, 1.0, 256, 4608), (384, 1.0, 32, 256),
    (384, None, 32, 256), (1000, 1.3, 64, 896)])
def test_ff_auto_adjust(block_ff, mult, multiple, want):
    d = dict(TINY_B, block_ff_dim=block_ff, block_ffn_dim_multiplier=mult, block_multiple_of=multiple)
    _, c = config_from_dict(d)
    assert c.intermediate_size == want


def test_ff_auto_adjust_off_keeps_width():
    _, c = config_from_dict(TINY_A)
    assert c.intermediate_size == 192


def test_typed_fields_and_defaults():
    _, a = config_from_dict(TINY_A)
    assert (a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 4, 2, 16)
    assert a.conv_L_cache == 3 and a.conv_bias is False and a.tie_embedding is True
    assert a.rope_theta == 10000.0 and a.norm_eps == 1e-5
    _, c = config_from_dict(TINY_C)
    assert c.head_dim == 48                      # given, not hidden/heads
    d = dict(TINY_A)
    del d["rope_theta"]
    assert config_from_dict(d)[1].rope_theta == 1e6
    d["some_key_nobody_reads"] = [1, 2, 3]        # unknown keys are ignored
    config_from_dict(d)


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                                 "num_key_value_heads", "layer_types", "max_position_embeddings", "norm_eps",
                                 "conv_L_cache", "block_ff_dim"])
def test_missing_required_key_is_named(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


@pytest.mark.parametrize("patch,word", [
    ({"layer_types": ["conv"]}, "layer_types"),
    ({"layer_types": ["conv", "attn", "conv", "conv"]}, "attn"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"conv_L_cache": 1}, "conv_L_cache"),
    ({"hidden_size": "64"}, "hidden_size"),
    ({"norm_eps": 0.0}, "norm_eps"),
    ({"head_dim": 15}, "head_dim"),
    ({"conv_bias": "yes"}, "conv_bias"),
    ({"vocab_size": 12.5}, "vocab_size"),
])
def test_bad_values_are_refused(patch, word):
    with pytest.raises(ConfigError, match=word):
        config_from_dict(dict(TINY_A, **patch))


def test_spec_is_layer_by_layer_data():
    arch, c = config_from_dict(TINY_B)
    spec = arch.build_spec(c)
    kinds = [l.mixer.kind for l in spec.layers]
    assert kinds == ["attention", "shortconv", "shortconv", "attention", "shortconv", "shortconv"]
    assert [e.layer for e in spec.schedule] == list(range(6))
    att = spec.layers[0].mixer.params
    assert att["num_heads"] == 6 and att["num_kv_heads"] == 3 and att["head_dim"] == 16
    assert att["position"].params["theta"] == 1e6 and att["qk_norm_eps"] == 1e-6
    conv = spec.layers[1].mixer.params
    assert conv["kernel_size"] == 4 and conv["bias"] is True
    assert spec.layers[0].ffn.params["intermediate_size"] == 256
    assert spec.head.params["tied"] is False


def test_schedule_validation():
    arch, c = config_from_dict(TINY_A)
    spec = arch.build_spec(c)
    spec.schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1, cache_of=1), ScheduleEntry(0)]
    spec.validate()
    spec.schedule = [ScheduleEntry(0), ScheduleEntry(9)]
    with pytest.raises(ConfigError, match="layer 9"):
        spec.validate()
    spec.schedule = [ScheduleEntry(0, cache_of=0)]
    with pytest.raises(ConfigError, match="earlier"):
        spec.validate()


def test_load_config_from_folder(tmp_path):
    with pytest.raises(ConfigError, match="config.json"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    arch, c = load_config(str(tmp_path))
    assert arch.name == "Lfm2ForCausalLM" and c.vocab_size == 256


def test_register_another_architecture():
    from dataclasses import dataclass

    @dataclass
    class ToyConfig(TypedConfig):
        width: int = cfg()

    def build(c):
        raise NotImplementedError

    register_architecture("ToyArch", ToyConfig, build)
    try:
        arch, c = config_from_dict({"architectures": ["ToyArch"], "width": 3})
        assert c.width == 3 and arch.build_spec is build
        with pytest.raises(ConfigError, match="already"):
            register_architecture("ToyArch", ToyConfig, build)
    finally:
        unregister_architecture("ToyArch")
