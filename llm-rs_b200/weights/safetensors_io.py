"""Reading and writing the safetensors container: 8 bytes little-endian header length,
a JSON header (name -> dtype, shape, data_offsets), then the raw data.

The reference maps the file and parses the same header
(llm-core/src/loader/safetensors.rs:21-101). This reader maps the file too and hands out
tensors that view the mapping; nothing is copied until a tensor goes to the device.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch


class WeightFileError(RuntimeError):
    pass


# name in the header -> (torch dtype, bytes per element)
_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One mapped ``.safetensors`` file."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
            self._f = open(path, "rb")
        except OSError as e:
            raise WeightFileError(f"cannot open {path}: {e}") from None
        if size < 8:
            raise WeightFileError(f"{path}: truncated (no header length)")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8:
            raise WeightFileError(f"{path}: truncated (header of {n} bytes does not fit in {size})")
        try:
            self.header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightFileError(f"{path}: bad header: {e}") from None
        self.header.pop("__metadata__", None)
        self._base = 8 + n
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        for name, info in self.header.items():
            if info.get("dtype") not in _DTYPES:
                raise WeightFileError(f"{path}: tensor {name} has unsupported dtype {info.get('dtype')!r}")
            lo, hi = info["data_offsets"]
            count = int(np.prod(info["shape"], dtype=np.int64)) if info["shape"] else 1
            if hi - lo != count * _DTYPES[info["dtype"]][1]:
                raise WeightFileError(f"{path}: tensor {name}: {hi - lo} bytes for shape {info['shape']}")
            if self._base + hi > size:
                raise WeightFileError(f"{path}: truncated (tensor {name} ends at {self._base + hi}, file has {size})")

    def names(self) -> List[str]:
        return list(self.header)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.header[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.header[name]["dtype"]][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped file (read-only data: copy before writing)."""
        info = self.header[name]
        dtype, width = _DTYPES[info["dtype"]]
        lo, hi = info["data_offsets"]
        count = (hi - lo) // width
        if count == 0:
            return torch.empty(info["shape"], dtype=dtype)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the buffer is not writable
            flat = torch.frombuffer(self._mm, dtype=dtype, count=count, offset=self._base + lo)
        return flat.reshape(info["shape"])


def save_file(tensors: Dict[str, torch.Tensor], path: str) -> None:
    """Write CPU tensors as one safetensors file (names in sorted order, data 8-byte aligned)."""
    header, offset, order = {}, 0, sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise WeightFileError(f"cannot store {name} of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-(8 + len(blob)) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)


def open_model_files(model_dir: str) -> List[SafetensorsFile]:
    """Every ``*.safetensors`` of a model folder (the reference reads them all,
    llm-core/src/backends/candle.rs:724-745)."""
    try:
        files = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    except OSError as e:
        raise WeightFileError(f"cannot list {model_dir}: {e}") from None
    if not files:
        raise WeightFileError(f"no safetensors files found in {model_dir}")
    return [SafetensorsFile(os.path.join(model_dir, f)) for f in files]
