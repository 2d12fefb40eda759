"""Interfaces of the parts a layer is put together from.

Every part gets its sizes and constants as constructor parameters (from
``PartSpec.params``) plus ``prefix``, the string put before its weight names. No part
knows which model it is in.

Life of a part:  construct -> ``weight_specs()`` tells the loader which tensors it wants
-> ``bind(tensors, runtime)`` receives them on the device -> ``forward(...)`` per step.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import TYPE_CHECKING, Dict, List, Optional

if TYPE_CHECKING:
    import numpy as np

import torch

from .spec import CacheNeed, StateNeed, WeightSpec


@dataclass
class Runtime:
    """What ``bind`` needs to know about the engine a part runs in."""
    device: torch.device
    act_dtype: torch.dtype          # bfloat16 or float32: type of activations and of the cache
    max_positions: int              # positions 0 .. max_positions-1 can occur


@dataclass
class StepInfo:
    """What a mixer's ``plan`` may read about a step, on the host, before anything is launched.
    The arrays are int32 numpy views that are only valid during the call."""
    n_tokens: int
    n_requests: int
    q_start: "np.ndarray"        # per request: index of its first token in the step
    n_new: "np.ndarray"          # per request: tokens it brings
    cached_len: "np.ndarray"     # per request: tokens it has cached before the step
    slot_ids: "np.ndarray"       # per request: its state slot
    block_tables: List["np.ndarray"]   # per cache group: [requests, width], -1 where a page was released
    group_keys: List[tuple]      # per cache group: the ``CacheNeed.group_key()`` its entries share
    page_size: int
    for_graph: bool              # the step will be captured in a CUDA graph and replayed (see ``Plan``)

    def table_of(self, need: CacheNeed) -> "np.ndarray":
        """The block table of the group that a mixer with this need writes to."""
        return self.block_tables[self.group_keys.index(need.group_key())]


@dataclass
class Plan:
    """What a mixer has planned for a step.

    ``arrays``  int32 numpy arrays; they travel to the device in the same copy as the step's other index
                arrays and reach ``forward`` as device tensors (``ctx.plan(key).arrays[name]``).
    ``values``  host integers that size launches (``ctx.plan(key).values[name]``).

    A step of single tokens may be captured in a CUDA graph and replayed for later steps. The graph is chosen by
    the batch's shape AND by every plan's array sizes and values, so a replayed launch always sees the sizes
    it was captured with; array CONTENTS are fresh at every replay. With ``StepInfo.for_graph`` a plan should
    therefore round its values up to what the batch's shape implies (say, a table's width instead of the longest
    request), or every step captures a graph of its own."""
    arrays: Dict[str, "np.ndarray"]
    values: Dict[str, int]

    def signature(self):
        return (tuple(sorted((k, int(v.size)) for k, v in self.arrays.items())), tuple(sorted(self.values.items())))


class Part:
    prefix: str = ""

    def weight_specs(self) -> List[WeightSpec]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        """Take the tensors named in ``weight_specs`` (already on ``runtime.device``)."""

    def chain(self) -> list:
        """The part's ``Linear`` products in the order a step runs them (after ``bind``). The model links each
        to the one that runs after it (``Linear.next_weight``), across parts and layers, so that a decode
        kernel can warm the L2 for its successor. A part without such products returns []."""
        return []


class PreNormed:
    """The input of a norm whose two halves are spread over the products around it (steps of few
    tokens): ``xw`` = h * weight in the activation type and ``parts`` [n_parts, stride], per token the
    sums of squares of h in pieces. The normed activations are ``xw / sqrt(sum(parts) / dim + eps)``;
    a part whose ``takes_prenormed(n_tokens)`` is true gets this object as its ``x`` and applies the
    factor to the rows of its first product. A part whose ``emits_prenormed(n_tokens)`` is true takes
    ``next_norm=(weight, eps)`` with ``residual=h`` and returns such an object for the norm after it."""

    def __init__(self, xw: torch.Tensor, parts: torch.Tensor, n_parts: int, dim: int, eps: float):
        self.xw, self.parts, self.n_parts, self.dim, self.eps = xw, parts, n_parts, dim, eps

    @property
    def scale(self):
        return (self.parts, self.n_parts, self.dim, self.eps)


class Norm(Part):
    """``forward(h, delta)``: ``h += delta`` (float32 residual stream, in place; ``delta``
    may be None) and return the normed rows in the activation type. With ``rows`` only
    those rows are normed and ``h`` stays untouched."""

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None):
        raise NotImplementedError

    def link(self):
        """(weight float32 [dim], eps) when this norm is ``x / sqrt(mean(x^2) + eps) * weight`` and may be
        spread over the products around it (see ``PreNormed``); None otherwise."""
        return None


class PositionEncoding(Part):
    """Turns token positions into something a mixer applies to queries and keys.

    ``rotation_table()``: a float32 [positions, rotary_dim/2, 2] table of (cos, sin) that
    the fused norm+rotation kernel applies in the rotate-half pairing, or None.
    ``apply_unfused(q, k, positions)``: for encodings that are no such rotation; changes
    q and k ([tokens, heads*head_dim] views) in place before the fused kernel runs
    without a table.
    """
    rotary_dim: int = 0

    def rotation_table(self) -> Optional[torch.Tensor]:
        return None

    def apply_unfused(self, q, k, positions) -> None:
        return None


class Mixer(Part):
    """Mixes information between the tokens of a request (attention here).

    ``cache_need()``  pages this mixer wants for a run-order entry (None: no pages)
    ``state_need()``  fixed-size per-request state it wants (None: none)
    ``forward(x, ctx, cache)``  x: [tokens, hidden] activations; ctx: the step's
        ``StepContext``; cache: the ``LayerCache`` of this run-order entry. Returns
        [tokens, hidden] in the activation type.
    A part with ``fuses_residual = True`` also takes ``residual=h`` (the float32 residual
    stream) and may add its output into it itself, returning None.
    """
    fuses_residual = False

    def takes_prenormed(self, n_tokens: int) -> bool:
        """True when ``forward`` accepts a ``PreNormed`` as ``x`` in a step of ``n_tokens`` tokens."""
        return False

    def emits_prenormed(self, n_tokens: int) -> bool:
        """True when ``forward(..., residual=h, next_norm=(weight, eps))`` returns a ``PreNormed``."""
        return False

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def plan_key(self):
        """A hashable name for the plan this mixer wants per step, or None for none. Mixers with equal keys
        share one plan (it is made once per step, by the first of them in the run order): put into the key
        whatever the plan depends on."""
        return None

    def plan(self, step: "StepInfo") -> "Plan":
        """Host work for one step, done once before anything is launched (see ``Plan``). ``forward`` finds the
        result under ``ctx.plan(self.plan_key())``. A mixer whose ``forward`` itself works on the host
        (loops over requests, reads ``ctx.host_*``) sets ``graph_safe = False`` instead."""
        raise NotImplementedError

    def forward(self, x, ctx, cache):
        raise NotImplementedError


class FeedForward(Part):
    """``forward(x, ctx)``: [tokens, hidden] -> [tokens, hidden], token by token. With
    ``fuses_residual = True`` it also takes ``residual=h`` as a mixer does."""
    fuses_residual = False

    def takes_prenormed(self, n_tokens: int) -> bool:
        return False

    def emits_prenormed(self, n_tokens: int) -> bool:
        return False

    def forward(self, x, ctx):
        raise NotImplementedError


class Block(Part):
    """Arranges a mixer and a feed-forward around the residual stream.

    ``forward(h, pending, ctx, cache) -> (h, pending)``: ``h`` is the float32 residual
    stream; ``pending`` is a branch output that has not been added to ``h`` yet (None at
    the first layer), so that the sum can be fused with the next norm.

    A block with ``links_norms = True`` also has ``accepts_prenormed(n_tokens)`` (its first norm and
    mixer can take a ``PreNormed`` as ``pending``: ``h`` then holds the sum already) and takes
    ``next_norm=(weight, eps)``, the first norm of the block that runs after it, for which its last
    part may return a ``PreNormed``.
    """
    links_norms = False

    def forward(self, h, pending, ctx, cache):
        raise NotImplementedError
