"""Arrangements of a mixer and a feed-forward around the residual stream."""
from __future__ import annotations

from .base import Block, Runtime
from .registry import build, register
from .spec import LayerSpec


@register("block", "prenorm")
class PreNormBlock(Block):
    """``h += mixer(norm1(h)); h += feed_forward(norm2(h))``
    (llm-core/src/graph/builder.rs:74-88,223-254,322-333: norm before each branch, no
    norm on a branch's output). Each sum into ``h`` is fused with the norm that follows
    it, so the feed-forward's output leaves the block not yet added. A part that sets
    ``fuses_residual`` is handed ``h`` and may add its output itself (it then returns None)."""

    def __init__(self, layer: LayerSpec, prefix: str = ""):
        p = layer.prefix
        self.mixer_norm = build("norm", layer.mixer_norm, prefix=p)
        self.mixer = build("mixer", layer.mixer, prefix=p + layer.mixer_scope)
        self.feed_forward_norm = build("norm", layer.feed_forward_norm, prefix=p)
        self.feed_forward = build("feed_forward", layer.feed_forward, prefix=p + layer.feed_forward_scope)

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def weight_specs(self):
        return [s for part in self.parts() for s in part.weight_specs()]

    def bind(self, tensors, runtime: Runtime):
        for part in self.parts():
            part.bind(tensors, runtime)

    def forward(self, h, pending, ctx, cache):
        x = self.mixer_norm.forward(h, pending)
        if getattr(self.mixer, "fuses_residual", False):
            a = self.mixer.forward(x, ctx, cache, residual=h)
        else:
            a = self.mixer.forward(x, ctx, cache)
        y = self.feed_forward_norm.forward(h, a)
        if getattr(self.feed_forward, "fuses_residual", False):
            return h, self.feed_forward.forward(y, ctx, residual=h)
        return h, self.feed_forward.forward(y, ctx)
