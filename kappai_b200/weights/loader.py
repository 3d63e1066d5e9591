"""Weights from safetensors, by tensor name.

Every tensor the model's parts declare is looked up by its name in the files
of the model folder.  Storage rules: tensors stored in bfloat16 are kept in
bfloat16 (float32 when the whole model runs in 32-bit; the values are then the
bfloat16 values, widened); a tensor stored in 32-bit stays so; float16 is
widened to float32; integer tables become int32.  All problems are gathered
into one error that lists missing tensors, unexpected tensors and wrong
shapes (the reference aborts the load on the first of these,
src/model.c:124-127,152-166,3337-3341).
"""
from __future__ import annotations

import glob
import os
from typing import Dict, List

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightError(ValueError):
    """The weight files do not fit the model."""

    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)


def weight_files(model_dir: str) -> List[str]:
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    files = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if not files:
        raise WeightError(f"{model_dir}: no model.safetensors (or any *.safetensors) found")
    return files


def _convert(t: torch.Tensor, compute_dtype: torch.dtype) -> torch.Tensor:
    if t.dtype == torch.bfloat16:
        return t if compute_dtype == torch.bfloat16 else t.to(torch.float32)
    if t.dtype == torch.float16:
        return t.to(torch.float32)
    if t.dtype in (torch.int64, torch.int32):
        return t.to(torch.int32)
    return t


def load_weights(model, model_dir: str) -> None:
    """Read, check and bind the weights of ``model`` from ``model_dir``."""
    table = model.weight_table()
    files = [SafetensorsFile(p) for p in weight_files(model_dir)]
    try:
        where: Dict[str, SafetensorsFile] = {}
        for f in files:
            for name in f.keys():
                if name in where:
                    raise WeightError(f"tensor '{name}' appears in two files")
                where[name] = f
        missing = sorted(n for n, ws in table.items() if n not in where and not ws.optional)
        unexpected = sorted(n for n in where if n not in table)
        wrong = []
        for n, ws in table.items():
            if n in where:
                _, shape = where[n].info(n)
                if tuple(shape) != tuple(ws.shape):
                    wrong.append(f"{n}: file has {list(shape)}, model wants {list(ws.shape)}")
        if missing or unexpected or wrong:
            lines = [f"{model_dir}: the weight files do not fit the model"]
            if missing:
                lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
            if unexpected:
                lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
            if wrong:
                lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
            raise WeightError("\n".join(lines), missing, unexpected, wrong)
        dev, dt = model.env.device, model.env.dtype
        tensors = {}
        for n in table:
            if n in where:
                tensors[n] = _convert(where[n].tensor(n), dt).to(dev)
        model.bind_weights(tensors)
    except SafetensorsError as e:
        raise WeightError(str(e)) from None
    finally:
        for f in files:
            f.close()
