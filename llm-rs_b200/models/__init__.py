"""Architectures: each module turns its typed configuration into a ``ModelSpec`` and
registers itself by the name found in config.json."""
from . import qwen3

__all__ = ["qwen3"]
