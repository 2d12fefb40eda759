"""RMSNorm, fused with the residual sum that precedes it."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import Norm, Runtime
from .registry import register
from .spec import WeightSpec


@register("norm", "rmsnorm")
class RMSNorm(Norm):
    """``y = x / sqrt(mean(x^2) + eps) * w`` with float32 statistics and a plain weight
    (llm-core/src/backends/attention.rs:55-68,98-104). ``dim`` and ``eps`` are parameters;
    ``name`` is the weight's name after the prefix."""

    def __init__(self, dim: int, eps: float, name: str = "weight", prefix: str = ""):
        self.dim, self.eps, self.prefix, self.name = dim, float(eps), prefix, name
        self.weight: Optional[torch.Tensor] = None
        self.act_dtype = None

    def weight_specs(self):
        return [WeightSpec(self.prefix + self.name, (self.dim,), role="norm")]

    def bind(self, tensors, runtime: Runtime):
        self.weight = tensors[self.prefix + self.name].to(torch.float32).contiguous()
        self.act_dtype = runtime.act_dtype

    def forward(self, h, delta, rows=None):
        return ops.add_rmsnorm(h, delta, self.weight, self.eps, self.act_dtype, rows=rows)

    def link(self):
        return (self.weight, self.eps) if self.act_dtype == torch.bfloat16 else None
