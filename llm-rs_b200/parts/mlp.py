"""Feed-forward parts."""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, Runtime
from .linear import Linear
from .registry import register
from .spec import WeightSpec


@register("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """``down( silu(gate(x)) * up(x) )`` with silu(x) = x * sigmoid(x)
    (llm-core/src/graph/builder.rs:256-297, llm-core/src/backends/candle.rs:1645-1663).
    gate and up are concatenated at load: one product, then one fused kernel."""

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str = ""):
        self.hidden_size, self.intermediate_size, self.prefix = hidden_size, intermediate_size, prefix

    def weight_specs(self):
        p, H, I = self.prefix, self.hidden_size, self.intermediate_size
        return [WeightSpec(p + "gate_proj.weight", (I, H)), WeightSpec(p + "up_proj.weight", (I, H)),
                WeightSpec(p + "down_proj.weight", (H, I))]

    def bind(self, tensors, runtime: Runtime):
        p = self.prefix
        g, u = tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]
        dt = g.dtype if g.dtype == u.dtype else torch.float32
        self.gate_up = Linear(torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous(), None, runtime.act_dtype)
        self.down = Linear(tensors[p + "down_proj.weight"], None, runtime.act_dtype)

    def forward(self, x, ctx):
        return self.down.forward(ops.silu_mul(self.gate_up.forward(x)))
