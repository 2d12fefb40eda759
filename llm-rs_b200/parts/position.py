"""Position encodings."""
from __future__ import annotations

from typing import Optional

import torch

from .base import PositionEncoding, Runtime
from .registry import register


@register("position", "none")
class NoPosition(PositionEncoding):
    """Queries and keys go unrotated (layers listed in ``no_rope_layers``,
    llm-core/src/graph/builder.rs:154-198)."""

    def __init__(self, head_dim: int = 0, prefix: str = ""):
        self.rotary_dim = 0


@register("position", "rope_half")
class RotaryHalf(PositionEncoding):
    """Rotary encoding in the rotate-half pairing.

    Angles ``pos * theta^(-2i/rotary_dim)`` as in llm-core/src/backends/attention.rs:178-214;
    the pairing is (x[i], x[i + rotary_dim/2]), which the published Qwen3 weights assume,
    where the reference rotates (x[2i], x[2i+1]) (attention.rs:216-233).

    The table of cosines and sines is computed once, in float64 from the exact product
    ``pos * inv_freq`` and rounded to float32, for positions 0 .. max_positions-1.
    """

    def __init__(self, head_dim: int, theta: float, rotary_dim: Optional[int] = None, prefix: str = ""):
        self.head_dim = head_dim
        self.theta = float(theta)
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {head_dim}")
        self._table = None

    def bind(self, tensors, runtime: Runtime):
        half = self.rotary_dim // 2
        i = torch.arange(half, dtype=torch.float64)
        inv_freq = self.theta ** (-2.0 * i / self.rotary_dim)
        pos = torch.arange(runtime.max_positions, dtype=torch.float64)
        ang = pos[:, None] * inv_freq[None, :]
        table = torch.stack([ang.cos(), ang.sin()], dim=-1).to(torch.float32)
        self._table = table.contiguous().to(runtime.device)

    def rotation_table(self):
        return self._table
