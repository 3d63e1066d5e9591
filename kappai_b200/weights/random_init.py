"""Random-weights mode: write a model folder from a configuration and a seed.

The folder holds ``config.json`` and ``model.safetensors`` and loads like any
other.  Each tensor is drawn from a counter-based generator keyed by the seed
and the tensor's name, so a tensor's values do not depend on which other
tensors exist or in what order they are made.  Distributions by role:
matrices and embeddings N(0, 0.02), stored in bfloat16; norm weights
1 + N(0, 0.1); convolution weights U(-1/sqrt(3), 1/sqrt(3)); biases N(0, 0.02);
these three stored in float32.  (The reference has random weights only in its
tests: src/test/test_synth_gguf.c:50-68,349-460.)
"""
from __future__ import annotations

import json
import math
import os
import zlib
from typing import Any, Dict

import numpy as np
import torch

from ..config.registry import config_from_dict
from ..parts.base import BuildEnv
from .safetensors_io import save_safetensors


def _generator(seed: int, name: str) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[int(seed) & (2**64 - 1), zlib.crc32(name.encode("utf-8"))]))


def random_tensor(seed: int, name: str, shape, role: str) -> torch.Tensor:
    g = _generator(seed, name)
    if role in ("matrix", "embedding"):
        a = g.standard_normal(shape, dtype=np.float32) * np.float32(0.02)
        return torch.from_numpy(a).to(torch.bfloat16)
    if role == "norm":
        return torch.from_numpy(1.0 + g.standard_normal(shape, dtype=np.float32) * np.float32(0.1)).float()
    if role == "conv":
        b = 1.0 / math.sqrt(3.0)
        return torch.from_numpy(g.uniform(-b, b, shape).astype(np.float32))
    if role == "bias":
        return torch.from_numpy(g.standard_normal(shape, dtype=np.float32) * np.float32(0.02))
    raise ValueError(f"no random distribution for tensor role '{role}'")


def random_weights(config_dict: Dict[str, Any], seed: int) -> Dict[str, torch.Tensor]:
    from ..engine.model import Model

    arch, cfg = config_from_dict(config_dict)
    spec = arch.build_spec(cfg)
    model = Model(spec, BuildEnv(torch.device("cpu"), torch.float32, max_positions=1))
    return {name: random_tensor(seed, name, ws.shape, ws.role) for name, ws in model.weight_table().items()}


def write_random_model(config_dict: Dict[str, Any], out_dir: str, seed: int) -> str:
    os.makedirs(out_dir, exist_ok=True)
    tensors = random_weights(config_dict, seed)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config_dict, f, indent=1)
    save_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                     {"format": "pt", "seed": str(seed), "generator": "kappai_b200.random_init"})
    return out_dir
