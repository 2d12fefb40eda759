"""Data that describes a model: which parts each layer is made of, and in what order layers run.

An architecture is a function from its typed configuration to a ``ModelSpec``. Nothing
below this point knows the architecture's name: parts are looked up by ``PartSpec.kind``
in the part registries (``parts.registry``) and get their sizes and constants from
``PartSpec.params``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by name with its sizes and constants."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a mixer and a feed-forward, each behind a norm, arranged by a block.

    ``prefix`` is put before every weight name of the layer's parts
    (``model.layers.3.``); the mixer's and the feed-forward's names get their scope
    after it (``model.layers.3.self_attn.q_proj.weight``). Scopes and the parts' own tensor names
    (their ``names`` parameter) come from the architecture's spec builder: the parts' defaults are
    neutral role names.
    """
    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: Optional[PartSpec] = None     # a block with one norm for both branches has none
    mixer_scope: str = ""
    feed_forward_scope: str = ""


@dataclass(frozen=True)
class RunStep:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may be named by several entries: its
    weights are shared, each entry has a cache of its own). ``cache_of`` names an
    EARLIER entry of the run order whose cache this entry reads instead of owning one;
    such an entry writes no keys or values.
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunStep, ...]
    embedding: PartSpec
    final_norm: PartSpec
    lm_head: PartSpec
    max_positions: int
    eos_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        for s, step in enumerate(self.run_order):
            if not 0 <= step.layer < len(self.layers):
                raise ValueError(f"run_order[{s}] names layer {step.layer}, model has {len(self.layers)}")
            if step.cache_of is not None:
                if not 0 <= step.cache_of < s:
                    raise ValueError(f"run_order[{s}].cache_of must name an earlier entry, got {step.cache_of}")
                if self.run_order[step.cache_of].cache_of is not None:
                    raise ValueError(f"run_order[{s}].cache_of names an entry that owns no cache")


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part expects in the model folder.

    ``role`` decides the random initialisation and the storage rule:
      "matrix"     ~N(0, sigma); kept in the stored floating type (bfloat16 or float32)
      "embedding"  like "matrix"
      "norm"       1 + N(0, norm_jitter); held as float32 (exact from bfloat16)
      "bias"       ~N(0, sigma)
      "int_table"  integers, held as int32
    ``optional`` tensors may be absent from the folder. ``load=False`` marks a tensor that the folder
    may hold but the part does not use (a stored copy of a tied matrix): its shape is checked, it is
    not read, and the random-weights mode does not write it.
    """
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    optional: bool = False
    load: bool = True


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer asks of the paged cache for one run-order entry.

    kind "full": every earlier token's rows stay. kind "window": only the last ``window`` tokens'
    rows are read, pages wholly behind the window are given back.

    A token stores, for each of ``n_kv_heads`` heads, one row per plane; ``planes`` gives the rows'
    widths. The default () means two planes of ``head_dim`` each: keys and values. A mixer that caches
    one latent row per token asks for ``n_kv_heads=1, planes=(width,)``; keys and values of different
    widths are ``planes=(dk, dv)``. Within a page the rows of one (head, plane) are contiguous
    ([page_size, width]) and a head's planes follow one another.
    """
    kind: str
    n_kv_heads: int
    head_dim: int
    window: int = 0
    planes: Tuple[int, ...] = ()

    @property
    def plane_widths(self) -> Tuple[int, ...]:
        return tuple(self.planes) if self.planes else (self.head_dim, self.head_dim)

    def group_key(self) -> Tuple:
        return (self.kind, self.n_kv_heads, self.plane_widths, self.window)


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size per-request state of a mixer: named tensors of given shape, float32."""
    tensors: Mapping[str, Tuple[int, ...]]
