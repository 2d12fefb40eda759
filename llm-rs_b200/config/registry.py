"""One registry from an architecture's name to its configuration class and model builder.

The reference has no registry by name: it classifies tensors by name pattern
(llm-core/src/graph/scan.rs:92-196) and branches on which tensors exist
(llm-core/src/graph/builder.rs:5-448); the ``arch`` string is informational
(llm-core/src/types.rs:67-68). Here the name in ``config.json`` (``architectures[0]``,
else ``model_type``) selects an entry; everything else follows from the entry.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional

from .errors import ConfigError


@dataclass(frozen=True)
class ArchitectureEntry:
    """What the framework needs to know about one architecture.

    name         the string found in config.json's ``architectures``
    model_type   config.json's ``model_type`` (used when ``architectures`` is absent)
    config_cls   a class with ``from_dict(dict) -> config`` and ``to_dict()``
    build_spec   ``config -> parts.ModelSpec``: the layer list, run order and part choices
    """
    name: str
    model_type: str
    config_cls: Any
    build_spec: Callable[[Any], Any]


_ARCHITECTURES: Dict[str, ArchitectureEntry] = {}


def register_architecture(entry: ArchitectureEntry, *, replace: bool = False) -> None:
    if entry.name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture {entry.name!r} is already registered")
    _ARCHITECTURES[entry.name] = entry


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def architecture_names() -> List[str]:
    return sorted(_ARCHITECTURES)


def resolve_architecture(raw: Dict[str, Any]) -> ArchitectureEntry:
    """Pick the registry entry for a parsed config.json."""
    names = raw.get("architectures")
    if isinstance(names, list) and names:
        name = names[0]
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {architecture_names()}")
    model_type: Optional[str] = raw.get("model_type")
    for entry in _ARCHITECTURES.values():
        if model_type and entry.model_type == model_type:
            return entry
    raise ConfigError(
        "config.json names no known architecture (architectures="
        f"{names!r}, model_type={model_type!r}); registered: {architecture_names()}")


def load_config(model_dir: str):
    """Read ``model_dir/config.json`` and return ``(entry, typed config)``."""
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json in {model_dir!r}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"failed to parse {path}: {e}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    entry = resolve_architecture(raw)
    return entry, entry.config_cls.from_dict(raw)
