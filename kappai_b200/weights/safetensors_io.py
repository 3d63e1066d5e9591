"""A small safetensors reader and writer.

File layout: 8 bytes little-endian header length N, N bytes of JSON
(``name -> {dtype, shape, data_offsets}`` plus an optional ``__metadata__``),
then the tensor bytes.  The reference reads the same container
(src/safetensors.c:75-144; dtypes F32/F16/BF16, src/safetensors.c:18-30).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Tuple

import numpy as np
import torch

_DTYPES = {
    "F32": (torch.float32, 4, np.float32),
    "F16": (torch.float16, 2, np.float16),
    "BF16": (torch.bfloat16, 2, np.uint16),
    "I32": (torch.int32, 4, np.int32),
    "I64": (torch.int64, 8, np.int64),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """Memory-mapped read access by tensor name."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8 or n > (1 << 30):
            raise SafetensorsError(f"{path}: header length {n} exceeds the file size {size}")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self._base = 8 + n
        self._entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        data_size = size - self._base
        for name, e in header.items():
            dt, shape, (b, en) = e["dtype"], tuple(int(s) for s in e["shape"]), e["data_offsets"]
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dt}")
            want = int(np.prod(shape, dtype=np.int64)) * _DTYPES[dt][1]
            if en - b != want or b < 0 or en > data_size:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' claims bytes [{b},{en}) for shape {list(shape)} {dt} "
                    f"(needs {want} bytes; data section has {data_size})")
            self._entries[name] = (dt, shape, b, en)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def keys(self) -> Iterable[str]:
        return self._entries.keys()

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dt, shape, _, _ = self._entries[name]
        return _DTYPES[dt][0], shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that owns its memory (copied out of the mapping)."""
        dt, shape, b, e = self._entries[name]
        tdt, _, ndt = _DTYPES[dt]
        arr = np.frombuffer(self._mm, dtype=ndt, count=(e - b) // np.dtype(ndt).itemsize,
                            offset=self._base + b).reshape(shape)
        t = torch.from_numpy(arr.copy())
        if dt == "BF16":
            t = t.view(torch.bfloat16)
        return t

    def close(self) -> None:
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def save_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.dtype == torch.bfloat16:
                t = t.view(torch.int16)
            f.write(t.numpy().tobytes())
