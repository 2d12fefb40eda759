"""Feed-forward parts."""
from __future__ import annotations

import os

import torch

from .. import ops
from .base import FeedForward, PreNormed, Runtime
from .linear import Linear
from .registry import register
from .spec import WeightSpec


FUSE_GATE_UP = os.environ.get("LLMRS_FUSE_GATE_UP", "1") != "0"


@register("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """``down( silu(gate(x)) * up(x) )`` with silu(x) = x * sigmoid(x)
    (llm-core/src/graph/builder.rs:256-297, llm-core/src/backends/candle.rs:1645-1663).
    gate and up are concatenated at load into one weight: one product, then SiLU*up,
    inside the product's epilogue when the tcgen05 kernel runs, else as one kernel. For
    that epilogue the rows alternate 64 of gate and the 64 matching of up (when the
    intermediate size is a multiple of 128); the output may be added straight into the
    residual stream. ``names`` maps the roles gate, up and down to the tensors' names after the prefix
    (without ".weight"); an architecture's spec builder gives the names its checkpoints use."""

    fuses_residual = True
    ROLES = ("gate", "up", "down")

    def __init__(self, hidden_size: int, intermediate_size: int, names=None, prefix: str = ""):
        self.hidden_size, self.intermediate_size, self.prefix = hidden_size, intermediate_size, prefix
        self.names = {role: role for role in self.ROLES}
        self.names.update(names or {})
        if set(self.names) != set(self.ROLES):
            raise ValueError(f"names may rename {self.ROLES}, got {sorted(set(self.names) - set(self.ROLES))}")

    def _name(self, role: str) -> str:
        return f"{self.prefix}{self.names[role]}.weight"

    def weight_specs(self):
        H, I = self.hidden_size, self.intermediate_size
        return [WeightSpec(self._name("gate"), (I, H)), WeightSpec(self._name("up"), (I, H)),
                WeightSpec(self._name("down"), (H, I))]

    def bind(self, tensors, runtime: Runtime):
        g, u = tensors[self._name("gate")], tensors[self._name("up")]
        dt = g.dtype if g.dtype == u.dtype else torch.float32
        self.block = 0      # columns of gate and up alternate in runs of this many (0: all gate, then all up)
        if dt == torch.bfloat16 and self.intermediate_size % 128 == 0 and self.hidden_size % 8 == 0:
            self.block = 64
            w = ops.interleave_gate_up(g.to(dt), u.to(dt))
        else:
            w = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()
        self.gate_up = Linear(w, None, runtime.act_dtype)
        self.down = Linear(tensors[self._name("down")], None, runtime.act_dtype)

    def chain(self):
        return [self.gate_up, self.down]

    def takes_prenormed(self, n_tokens: int) -> bool:
        if not (self.block and self.gate_up.tc_enabled() and FUSE_GATE_UP):
            return False
        return 0 < n_tokens <= 64 or self.gate_up.uses_tc(n_tokens)

    def emits_prenormed(self, n_tokens: int) -> bool:
        return self.down.emits_prenormed(n_tokens)

    def forward(self, x, ctx, residual=None, next_norm=None):
        if isinstance(x, PreNormed):     # only when takes_prenormed
            act = ops.gemm_bf16(x.xw, self.gate_up.weight, epilogue="silu_mul", scale=x.scale,
                                then=self.gate_up.next_weight)
            if next_norm is not None:
                return self.down.forward_into_residual_for_norm(act, residual, *next_norm)
            return self.down.forward_into_residual(act, residual) if residual is not None else self.down.forward(act)
        # With interleaved weights the product and SiLU(gate) * up are one kernel at every number of
        # tokens: for few tokens the cluster kernel (40 against 44 us for the library product and the SiLU kernel at
        # 64 tokens), for many the persistent tcgen05 kernel on pairs of SMs (2,048 tokens: 261 against 271 + 20 us).
        if self.block and x.dtype == torch.bfloat16 and self.gate_up.tc_enabled() and FUSE_GATE_UP:
            act = ops.gemm_bf16(x, self.gate_up.weight, epilogue="silu_mul", then=self.gate_up.next_weight)
        else:
            act = ops.silu_mul(self.gate_up.forward(x), block=self.block)
        if next_norm is not None:
            return self.down.forward_into_residual_for_norm(act, residual, *next_norm)
        if residual is not None:
            return self.down.forward_into_residual(act, residual)
        return self.down.forward(act)
