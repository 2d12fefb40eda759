"""Loading a model folder's tensors by name, with one error for everything that is wrong.

Storage rule: floating tensors stay in the type the file stores them in when that is
bfloat16 or float32 (float16 is widened to the engine's type); in the float32 path
everything floating is widened to float32; integer tables become int32. The reference
casts every tensor to its compute type at load and checks neither shapes nor
unexpected names (llm-core/src/backends/candle.rs:738-745; a missing weight only shows
at first use, llm-core/src/backends/weights.rs:159); here all three are load-time errors.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from ..parts.spec import WeightSpec
from .safetensors_io import SafetensorsFile, WeightFileError, open_model_files


class WeightError(RuntimeError):
    """Lists every missing tensor, every unexpected tensor and every wrong shape or type."""

    def __init__(self, model_dir, missing, unexpected, wrong_shape, wrong_dtype, duplicates):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype, self.duplicates = list(wrong_shape), list(wrong_dtype), list(duplicates)
        lines = [f"the tensors in {model_dir} do not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        for name, got in self.wrong_dtype:
            lines.append(f"  wrong type: {name} is {got}")
        for name, files in self.duplicates:
            lines.append(f"  stored twice: {name} in {', '.join(files)}")
        super().__init__("\n".join(lines))


def _target_dtype(spec: WeightSpec, stored: torch.dtype, act_dtype: torch.dtype):
    if spec.role == "int_table":
        return torch.int32 if not stored.is_floating_point and stored != torch.bool else None
    if not stored.is_floating_point:
        return None
    if spec.role == "norm" or act_dtype == torch.float32 or stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def load_weights(model_dir: str, specs: Sequence[WeightSpec], act_dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    files = open_model_files(model_dir)
    where: Dict[str, SafetensorsFile] = {}
    duplicates = []
    for f in files:
        for name in f.names():
            if name in where:
                duplicates.append((name, [where[name].path, f.path]))
            where[name] = f
    by_name = {s.name: s for s in specs}
    missing = [s.name for s in specs if s.name not in where and not s.optional]
    unexpected = sorted(n for n in where if n not in by_name)
    wrong_shape, wrong_dtype = [], []
    for s in specs:
        if s.name in where:
            f = where[s.name]
            if f.shape(s.name) != tuple(s.shape):
                wrong_shape.append((s.name, s.shape, f.shape(s.name)))
            elif _target_dtype(s, f.dtype(s.name), act_dtype) is None:
                wrong_dtype.append((s.name, str(f.dtype(s.name)).replace("torch.", "")))
    if missing or unexpected or wrong_shape or wrong_dtype or duplicates:
        raise WeightError(model_dir, missing, unexpected, wrong_shape, wrong_dtype, duplicates)
    out = {}
    for s in specs:
        if s.name not in where or not s.load:
            continue
        f = where[s.name]
        t = f.tensor(s.name)
        out[s.name] = t.to(device=device, dtype=_target_dtype(s, t.dtype, act_dtype)).contiguous()
    return out
