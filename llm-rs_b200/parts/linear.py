"""Matrix products of the parts.

bfloat16 weights go through the library product (cuBLAS via ``torch``), as the
reference's projections go through its tensor library
(llm-core/src/backends/candle.rs:1276-1340). float32 weights, the whole float32 path
and tensors that the model folder stores in 32-bit, go through this package's own FFMA
kernel: true 32-bit, no reduced-precision tensor-core mode.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops


class Linear:
    """``y = x @ weight.T (+ bias)`` for ``weight`` of shape [out, in]."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], act_dtype: torch.dtype):
        if weight.dtype not in (torch.float32, torch.bfloat16):
            raise TypeError(f"weight must be float32 or bfloat16, got {weight.dtype}")
        self.weight = weight
        self.bias = None if bias is None else bias.to(weight.dtype).contiguous()
        self.act_dtype = act_dtype

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        out_dtype = out_dtype or self.act_dtype
        if self.weight.dtype == torch.float32:
            xf = x if x.dtype == torch.float32 else x.to(torch.float32)
            y = ops.gemm_f32(xf, self.weight, self.bias)
            return y if out_dtype == torch.float32 else y.to(out_dtype)
        xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        if out_dtype == torch.float32:
            y = torch.mm(xb, self.weight.t(), out_dtype=torch.float32)
            if self.bias is not None:
                y += self.bias.to(torch.float32)
            return y
        return torch.nn.functional.linear(xb, self.weight, self.bias)
