"""Matrix products of the parts.

bfloat16 weights: steps of up to ``TC_MAX_TOKENS`` tokens (decoding, 64 at most) run this package's
tcgen05 kernel (``csrc/gemm_tcgen05.cu``: weights fill the 128 rows of the MMA, the k range
is shared by a thread-block cluster) with the residual sum or SiLU*up fused into its
epilogue; larger steps go through the library product (cuBLAS via ``torch``), as the
reference's projections go through its tensor library
(llm-core/src/backends/candle.rs:1276-1340), except the gate|up product with its SiLU*up
epilogue (``parts/mlp.py``), which runs this package's kernel for many tokens (tiles of
256 x 256 on pairs of SMs, tcgen05.mma.cta_group::2) at every size. ``LLMRS_TC_MANY_TOKENS=n``
sends every product of steps of n tokens or more to that kernel, with the residual sum and the
norms spread over its epilogues as in decode steps. float32 weights, the whole float32 path and
tensors that the model folder stores in 32-bit, go through this package's own FFMA
kernel: true 32-bit, no reduced-precision tensor-core mode.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import ops
from .base import PreNormed

# Steps with at most this many tokens take the tcgen05 kernel for few tokens; 0 switches the tcgen05 products off.
# (Measured inside decode steps at Qwen3-8B sizes: with its fused epilogues the kernel is ahead of the library product
# plus the separate kernels at every number of tokens it takes, 4.08 -> 3.58 ms a step at 32 tokens; a product may set
# a lower limit of its own, ``Linear.tc_max_tokens``.)
TC_MAX_TOKENS = int(os.environ.get("LLMRS_TC_MAX_TOKENS", "64"))
# Steps with at least this many tokens take the tcgen05 kernel for many tokens for every product; 0 (the default)
# keeps all but gate|up on the library product. (Prefill of 2,048 tokens at Qwen3-8B sizes, 36 layers, timed over
# seconds under the power cap: 24.9 ms with the library's q|k|v, o and down products and the norm kernels, 25.6 ms
# with this package's kernel and no norm kernels, 26.0 ms with it and the norm kernels; launched alone in a burst
# the kernel is level with the library for q|k|v (72 us), 4 us behind for o (53 against 49, residual sum and the
# next norm's input included, which cost the library path 14 us more) and 13 us behind for down (145 against 132);
# with o alone, o and down, or all three on it the step took 25.5-25.8, 25.8-26.1 and 25.5-25.9 ms against 25.1.)
TC_MANY_TOKENS = int(os.environ.get("LLMRS_TC_MANY_TOKENS", "0"))


_SM_COUNT = {}


def _sm_count(device) -> int:
    if device not in _SM_COUNT:
        _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNT[device]


class Linear:
    """``y = x @ weight.T (+ bias)`` for ``weight`` of shape [out, in]."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], act_dtype: torch.dtype):
        if weight.dtype not in (torch.float32, torch.bfloat16):
            raise TypeError(f"weight must be float32 or bfloat16, got {weight.dtype}")
        self.weight = weight
        self.bias = None if bias is None else bias.to(weight.dtype).contiguous()
        self.act_dtype = act_dtype
        n, k = weight.shape
        # The weights of the product that runs after this one in a step (set by ``DecoderModel.bind``): in
        # steps of few tokens this product's kernel asks their start into the L2 as its own stream ends.
        self.next_weight: Optional[torch.Tensor] = None
        self.warms_next = True      # False: something else runs between this product and the next one
        self.tc_max_tokens: Optional[int] = None    # a limit of this product's own below TC_MAX_TOKENS
        self.tc_ok = (weight.dtype == torch.bfloat16 and bias is None and weight.is_contiguous()
                      and k % 8 == 0 and n % 8 == 0 and weight.data_ptr() % 16 == 0)

    def tc_enabled(self) -> bool:
        """The tcgen05 kernel can take this weight and has not been switched off (LLMRS_TC_MAX_TOKENS=0)."""
        return self.tc_ok and TC_MAX_TOKENS > 0

    def uses_tc(self, n_tokens: int) -> bool:
        if not self.tc_enabled() or n_tokens <= 0:
            return False
        few = TC_MAX_TOKENS if self.tc_max_tokens is None else min(TC_MAX_TOKENS, self.tc_max_tokens)
        return n_tokens <= few or 0 < TC_MANY_TOKENS <= n_tokens

    def forward(self, x, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        out_dtype = out_dtype or self.act_dtype
        if isinstance(x, PreNormed):     # only when takes_prenormed
            return ops.gemm_bf16(x.xw, self.weight, out_dtype=out_dtype, scale=x.scale, then=self.next_weight)
        if self.weight.dtype == torch.float32:
            xf = x if x.dtype == torch.float32 else x.to(torch.float32)
            y = ops.gemm_f32(xf, self.weight, self.bias)
            return y if out_dtype == torch.float32 else y.to(out_dtype)
        xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        if self.uses_tc(xb.size(0)) and out_dtype in (torch.float32, torch.bfloat16):
            return ops.gemm_bf16(xb, self.weight, out_dtype=out_dtype, then=self.next_weight)
        return ops.library_gemm(xb, self.weight, self.bias, out_dtype)

    def _splits(self, n_tokens: int) -> int:
        n, k = self.weight.shape
        return ops.tc_splits(n_tokens, n, k, _sm_count(self.weight.device))

    def takes_prenormed(self, n_tokens: int) -> bool:
        """True when ``forward`` accepts a ``PreNormed`` (the tcgen05 kernels scale their rows)."""
        return self.uses_tc(n_tokens) and (n_tokens <= 64 or self.weight.size(0) >= 256)

    def emits_prenormed(self, n_tokens: int) -> bool:
        """True when ``forward_into_residual`` can also write the input of the norm that follows."""
        return self.uses_tc(n_tokens) and (n_tokens <= 64 or self.weight.size(0) >= 256)

    def forward_into_residual_for_norm(self, x: torch.Tensor, h: torch.Tensor, norm_weight: torch.Tensor,
                                       eps: float) -> PreNormed:
        """``h += x @ weight.T`` and, in the same epilogue, the input of the norm that follows
        (see ``PreNormed``). Only when ``emits_prenormed``."""
        n = self.weight.size(0)
        splits = self._splits(x.size(0))
        n_parts = ops.norm_parts(n, splits, x.size(0))
        xw = torch.empty((x.size(0), n), dtype=torch.bfloat16, device=x.device)
        parts = torch.empty((n_parts, max(64, x.size(0))), dtype=torch.float32, device=x.device)
        ops.gemm_bf16(x, self.weight, out=h, epilogue="residual", splits=splits, emit=(norm_weight, xw, parts),
                      then=self.next_weight)
        return PreNormed(xw, parts, n_parts, n, eps)

    def forward_into_residual(self, x: torch.Tensor, h: torch.Tensor) -> Optional[torch.Tensor]:
        """``h += x @ weight.T`` inside the product's epilogue when the tcgen05 kernel runs
        (returns None); otherwise the product is returned for the caller to add."""
        if x.dtype == torch.bfloat16 and self.uses_tc(x.size(0)) and h.is_contiguous():
            ops.gemm_bf16(x, self.weight, out=h, epilogue="residual", then=self.next_weight)
            return None
        return self.forward(x)
