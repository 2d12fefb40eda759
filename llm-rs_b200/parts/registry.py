"""Registries of parts by kind: mixers, feed-forwards, norms, position encodings, blocks,
embeddings and heads. ``build(kind_of_part, spec, ...)`` makes the part a ``PartSpec`` names.

A part class is registered with ``@register("mixer", "gqa_attention")``. Tests register
toy parts the same way; the framework's files need no change for a new part.
"""
from __future__ import annotations

from typing import Any, Callable, Dict

_CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "lm_head")
_REGISTRY: Dict[str, Dict[str, Callable[..., Any]]] = {c: {} for c in _CATEGORIES}


def register(category: str, kind: str, *, replace: bool = False):
    if category not in _REGISTRY:
        raise KeyError(f"unknown part category {category!r}; known: {_CATEGORIES}")

    def deco(cls):
        if kind in _REGISTRY[category] and not replace:
            raise KeyError(f"{category} {kind!r} is already registered")
        _REGISTRY[category][kind] = cls
        return cls
    return deco


def unregister(category: str, kind: str) -> None:
    _REGISTRY[category].pop(kind, None)


def kinds(category: str):
    return sorted(_REGISTRY[category])


def build(category: str, spec, **context):
    """Construct the part ``spec`` names: ``cls(**spec.params, **context)``."""
    try:
        cls = _REGISTRY[category][spec.kind]
    except KeyError:
        raise KeyError(
            f"no {category} of kind {spec.kind!r} is registered; known: {kinds(category)}") from None
    return cls(**dict(spec.params), **context)
