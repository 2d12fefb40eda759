"""Arrangements of a mixer and a feed-forward around the residual stream."""
from __future__ import annotations

import os

from .base import Block, PreNormed, Runtime
from .registry import build, register
from .spec import LayerSpec


# Steps of few tokens spread each norm over the products around it (see ``PreNormed``); LLMRS_LINK_NORMS=0
# keeps the norm kernels.
LINK_NORMS = os.environ.get("LLMRS_LINK_NORMS", "1") != "0"


@register("block", "prenorm")
class PreNormBlock(Block):
    """``h += mixer(norm1(h)); h += feed_forward(norm2(h))``
    (llm-core/src/graph/builder.rs:74-88,223-254,322-333: norm before each branch, no
    norm on a branch's output). Each sum into ``h`` is fused with the norm that follows
    it, so the feed-forward's output leaves the block not yet added. A part that sets
    ``fuses_residual`` is handed ``h`` and may add its output itself (it then returns None).
    In steps of few tokens a part that can do so also writes the input of the norm after it
    (``PreNormed``), and the part after that norm applies its factor: no norm kernel runs."""

    def __init__(self, layer: LayerSpec, prefix: str = ""):
        p = layer.prefix
        self.mixer_norm = build("norm", layer.mixer_norm, prefix=p)
        self.mixer = build("mixer", layer.mixer, prefix=p + layer.mixer_scope)
        self.feed_forward_norm = build("norm", layer.feed_forward_norm, prefix=p)
        self.feed_forward = build("feed_forward", layer.feed_forward, prefix=p + layer.feed_forward_scope)

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def chain(self):
        return [lin for part in self.parts() for lin in part.chain()]

    def weight_specs(self):
        return [s for part in self.parts() for s in part.weight_specs()]

    def bind(self, tensors, runtime: Runtime):
        for part in self.parts():
            part.bind(tensors, runtime)

    links_norms = True

    def accepts_prenormed(self, n_tokens: int) -> bool:
        return LINK_NORMS and self.mixer_norm.link() is not None and self.mixer.takes_prenormed(n_tokens)

    def forward(self, h, pending, ctx, cache, next_norm=None):
        n = ctx.n_tokens
        # A PreNormed ``pending`` was made for this block's first norm by the block before (h holds the sum).
        x = pending if isinstance(pending, PreNormed) else self.mixer_norm.forward(h, pending)
        fused = getattr(self.mixer, "fuses_residual", False)
        link = self.feed_forward_norm.link() if LINK_NORMS and fused else None
        if link and self.mixer.emits_prenormed(n) and self.feed_forward.takes_prenormed(n):
            y = self.mixer.forward(x, ctx, cache, residual=h, next_norm=link)
        else:
            a = self.mixer.forward(x, ctx, cache, residual=h) if fused else self.mixer.forward(x, ctx, cache)
            y = self.feed_forward_norm.forward(h, a)
        fused = getattr(self.feed_forward, "fuses_residual", False)
        if next_norm is not None and fused and self.feed_forward.emits_prenormed(n):
            return h, self.feed_forward.forward(y, ctx, residual=h, next_norm=next_norm)
        if fused:
            return h, self.feed_forward.forward(y, ctx, residual=h)
        return h, self.feed_forward.forward(y, ctx)
