"""Typed model configurations and the architecture registry."""
from .errors import ConfigError
from .registry import (ArchitectureEntry, architecture_names, load_config,
                       register_architecture, resolve_architecture, unregister_architecture)
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "ArchitectureEntry", "architecture_names", "load_config",
           "register_architecture", "resolve_architecture", "unregister_architecture", "Qwen3Config"]
