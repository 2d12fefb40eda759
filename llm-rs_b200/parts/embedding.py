"""Token embedding and the output head."""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, Runtime
from .linear import Linear
from .registry import register
from .spec import WeightSpec


@register("embedding", "token_embedding")
class TokenEmbedding(Part):
    """``h0[t] = table[id_t]``, no scale (llm-core/src/graph/builder.rs:8-14,
    llm-core/src/backends/candle.rs:1238-1261). The result is the float32 residual stream."""

    def __init__(self, vocab_size: int, hidden_size: int, name: str = "embedding.weight", prefix: str = ""):
        self.vocab_size, self.hidden_size, self.name = vocab_size, hidden_size, prefix + name

    def weight_specs(self):
        return [WeightSpec(self.name, (self.vocab_size, self.hidden_size), role="embedding")]

    def bind(self, tensors, runtime: Runtime):
        self.table = tensors[self.name]

    def forward(self, token_ids):
        return ops.embedding(self.table, token_ids)


@register("lm_head", "linear_head")
class LinearHead(Part):
    """``logits = x @ W^T`` in float32, no bias, no soft cap
    (llm-core/src/graph/builder.rs:408-437). ``tied_to`` names the embedding table that
    serves as W when the model ties them (llm-core/src/backends/weights.rs:144-157): one
    buffer, used by both. A tied model's folder may still store the head's matrix (a copy of the
    table); it is accepted and not read."""

    def __init__(self, vocab_size: int, hidden_size: int, name: str = "head.weight", tied_to: str = "",
                 prefix: str = ""):
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.name, self.tied_to = prefix + name, tied_to

    def weight_specs(self):
        if self.tied_to:
            return [WeightSpec(self.name, (self.vocab_size, self.hidden_size), optional=True, load=False)]
        return [WeightSpec(self.name, (self.vocab_size, self.hidden_size))]

    def bind(self, tensors, runtime: Runtime):
        self.proj = Linear(tensors[self.tied_to or self.name], None, runtime.act_dtype)

    def chain(self):
        return [self.proj]

    def forward(self, x):
        return self.proj.forward(x, out_dtype=torch.float32)
