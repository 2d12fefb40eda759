"""Random weights from a configuration and a seed: a model folder on disk, or tensors
made directly on the device (for sizes at which a file would take minutes).

Matrices, embeddings and biases are ~N(0, sigma); norm weights are 1 + N(0, norm_jitter).
Each tensor has its own generator seeded by (seed, index of the tensor in name order),
so one tensor's values do not depend on which others exist. The reference has no such
mode (its tests write 2x2 files by hand, llm-tests/tests/mlc_test.rs:186-195).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional, Sequence

import torch

from ..parts.spec import WeightSpec
from .safetensors_io import save_file


def _make(spec: WeightSpec, seed: int, index: int, sigma: float, norm_jitter: float, dtype: torch.dtype, device):
    gen = torch.Generator(device=device)
    gen.manual_seed((seed * 1_000_003 + index) & 0x7FFFFFFFFFFFFFFF)
    if spec.role == "int_table":
        return torch.randint(0, 2**15, spec.shape, generator=gen, dtype=torch.int32, device=device)
    # Drawn in float32 then rounded, so the bfloat16 and float32 forms of a seed agree.
    if spec.role == "norm":
        t = 1.0 + norm_jitter * torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)
    else:
        t = torch.empty(spec.shape, dtype=dtype, device=device)
        rows = spec.shape[0] if len(spec.shape) > 1 else 1
        # In slabs: a vocabulary-sized matrix in float32 would double the peak memory.
        step = max(1, (1 << 26) // max(1, t.numel() // max(rows, 1)))
        if len(spec.shape) > 1:
            for r in range(0, rows, step):
                n = min(step, rows - r)
                t[r:r + n] = (sigma * torch.randn((n, *spec.shape[1:]), generator=gen, dtype=torch.float32,
                                                   device=device)).to(dtype)
        else:
            t.copy_((sigma * torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)).to(dtype))
        return t
    return t.to(dtype)


def random_tensors(specs: Sequence[WeightSpec], seed: int, sigma: float = 0.02, norm_jitter: float = 0.0,
                   dtype: torch.dtype = torch.bfloat16, device="cpu", norm_dtype: Optional[torch.dtype] = None
                   ) -> Dict[str, torch.Tensor]:
    out = {}
    for index, spec in enumerate(sorted((s for s in specs if s.load), key=lambda s: s.name)):
        dt = (norm_dtype or dtype) if spec.role == "norm" else dtype
        out[spec.name] = _make(spec, seed, index, sigma, norm_jitter, dt, device)
    return out


def write_random_model(model_dir: str, config, seed: int, sigma: float = 0.02, norm_jitter: float = 0.1,
                       dtype: torch.dtype = torch.bfloat16, norm_dtype: Optional[torch.dtype] = None) -> str:
    """Write ``config.json`` and ``model.safetensors`` for a typed configuration.

    ``config`` is a registered architecture's configuration object (``to_dict()`` gives
    its config.json). Returns ``model_dir``.
    """
    from ..config import resolve_architecture
    from ..parts import DecoderModel
    raw = config.to_dict()
    entry = resolve_architecture(raw)
    model = DecoderModel(entry.build_spec(config))
    tensors = random_tensors(model.weight_specs(), seed, sigma, norm_jitter, dtype, "cpu", norm_dtype)
    os.makedirs(model_dir, exist_ok=True)
    raw["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(raw, f, indent=2)
    save_file(tensors, os.path.join(model_dir, "model.safetensors"))
    return model_dir
