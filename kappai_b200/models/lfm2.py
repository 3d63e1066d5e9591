"""The LFM2 hybrid: gated short-convolution layers and GQA attention layers
(per-head QK RMSNorm, NeoX RoPE), each followed by a SwiGLU feed-forward.

This file is the only place that knows LFM2's ``config.json`` keys and tensor
names.  It turns them into a :class:`ModelSpec`; the parts it names live in
``kappai_b200.parts`` and know nothing of LFM2.

Reference: layer op lists src/models/lfm.c:7-62; registry entry
src/arch.c:73-82 (qk norm, NeoX rope, theta default 1e6, short conv);
metadata keys src/model.c:2309-2521; tensor names src/model.c:2539-3190
(GGUF names; the safetensors names below are their config.json-side twins).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

from ..config.schema import (ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry,
                             TypedConfig, cfg)
from ..config.registry import register_architecture

ARCHITECTURE = "Lfm2ForCausalLM"
LAYER_CONV = "conv"
LAYER_ATTENTION = "full_attention"


@dataclass
class Lfm2Config(TypedConfig):
    vocab_size: int = cfg()
    hidden_size: int = cfg()
    num_hidden_layers: int = cfg()
    num_attention_heads: int = cfg()
    num_key_value_heads: int = cfg()
    layer_types: List[str] = cfg()
    max_position_embeddings: int = cfg()
    norm_eps: float = cfg()
    conv_L_cache: int = cfg()
    block_ff_dim: int = cfg()
    head_dim: Optional[int] = cfg(None)
    block_auto_adjust_ff_dim: bool = cfg(False)
    block_ffn_dim_multiplier: Optional[float] = cfg(None)
    block_multiple_of: int = cfg(256)
    conv_bias: bool = cfg(False)
    rope_theta: float = cfg(1000000.0)          # src/arch.c:77
    tie_embedding: bool = cfg(True)
    eos_token_id: Optional[int] = cfg(None)

    def validate(self) -> None:
        L = self.num_hidden_layers
        if L < 1:
            raise ConfigError("num_hidden_layers must be at least 1")
        if len(self.layer_types) != L:
            # src/model.c:2368-2374: the per-layer array must have one entry a layer
            raise ConfigError(f"layer_types has {len(self.layer_types)} entries, num_hidden_layers is {L}")
        for i, t in enumerate(self.layer_types):
            if t not in (LAYER_CONV, LAYER_ATTENTION):
                raise ConfigError(f"layer_types[{i}]='{t}': expected '{LAYER_CONV}' or '{LAYER_ATTENTION}'")
        H, G = self.num_attention_heads, self.num_key_value_heads
        if H < 1 or G < 1 or H % G != 0:
            raise ConfigError(f"num_attention_heads={H} must be a positive multiple of num_key_value_heads={G}")
        if self.head_dim is None:
            if self.hidden_size % H != 0:
                raise ConfigError(f"hidden_size={self.hidden_size} is not divisible by num_attention_heads={H} "
                                  "and no head_dim is given")
            self.head_dim = self.hidden_size // H      # src/model.c:2437-2441
        if self.head_dim % 2 != 0 or self.head_dim < 2:
            raise ConfigError(f"head_dim={self.head_dim} must be even (rotary pairs)")
        if self.conv_L_cache < 2:
            raise ConfigError(f"conv_L_cache={self.conv_L_cache} must be at least 2")  # src/model.c:2491-2499
        if self.norm_eps <= 0:
            raise ConfigError("norm_eps must be positive")
        if self.block_multiple_of < 1:
            raise ConfigError("block_multiple_of must be positive")
        if self.max_position_embeddings < 1:
            raise ConfigError("max_position_embeddings must be positive")

    @property
    def intermediate_size(self) -> int:
        """Width of the SwiGLU feed-forward.  With auto-adjust:
        ``t = floor(2*block_ff_dim/3)``; times the multiplier if one is given;
        rounded up to a multiple of ``block_multiple_of``."""
        ff = self.block_ff_dim
        if self.block_auto_adjust_ff_dim:
            ff = (2 * ff) // 3
            if self.block_ffn_dim_multiplier is not None:
                ff = int(self.block_ffn_dim_multiplier * ff)
            m = self.block_multiple_of
            ff = m * ((ff + m - 1) // m)
        return ff


def build_spec(c: Lfm2Config) -> ModelSpec:
    d, hd = c.hidden_size, c.head_dim
    norm = lambda prefix: PartSpec("rmsnorm", {"size": d, "eps": c.norm_eps}, prefix)
    layers = []
    for i, kind in enumerate(c.layer_types):
        p = f"model.layers.{i}."
        if kind == LAYER_CONV:
            mixer = PartSpec(
                "shortconv",
                {"hidden_size": d, "kernel_size": c.conv_L_cache, "bias": c.conv_bias},
                p + "conv.")
        else:
            mixer = PartSpec(
                "attention",
                {"hidden_size": d, "num_heads": c.num_attention_heads,
                 "num_kv_heads": c.num_key_value_heads, "head_dim": hd,
                 "qk_norm_eps": c.norm_eps,                      # src/models/lfm.c:36-37
                 "scale": 1.0 / math.sqrt(hd),                   # src/recipe/builders.c:244-248
                 "window": None,
                 "position": PartSpec("rope", {"rotary_dim": hd, "theta": c.rope_theta,
                                               "pairing": "neox"}),   # src/arch.c:79
                 "bias": False},
                p + "self_attn.",
                rename={"q_norm.weight": "q_layernorm.weight", "k_norm.weight": "k_layernorm.weight"})
        ffn = PartSpec("swiglu", {"hidden_size": d, "intermediate_size": c.intermediate_size, "bias": False},
                       p + "feed_forward.",
                       rename={"gate_proj.weight": "w1.weight", "up_proj.weight": "w3.weight",
                               "down_proj.weight": "w2.weight"})
        layers.append(LayerSpec(mixer=mixer, ffn=ffn,
                                mixer_norm=norm(p + "operator_norm."), ffn_norm=norm(p + "ffn_norm."),
                                block="prenorm_residual"))
    spec = ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=d,
        vocab_size=c.vocab_size,
        max_positions=c.max_position_embeddings,
        embedding=PartSpec("embedding", {"vocab_size": c.vocab_size, "hidden_size": d, "scale": None},
                           "model.embed_tokens."),
        layers=layers,
        schedule=[ScheduleEntry(i) for i in range(len(layers))],
        final_norm=norm("model.embedding_norm."),                # src/model.c:2552-2560
        head=PartSpec("lm_head", {"vocab_size": c.vocab_size, "hidden_size": d,
                                  "tied": c.tie_embedding}, "lm_head."),
        eos_token_id=c.eos_token_id,
    )
    spec.validate()
    return spec


register_architecture(ARCHITECTURE, Lfm2Config, build_spec)
