"""llm-rs_b200: a single-GPU inference engine for NVIDIA B200 (sm_100a), with the
capabilities of mashriram/llm-rs's Qwen3 dense path: typed configuration and registry,
weights by name, layers composed from parts, a paged cache manager, one step function
for mixed batches, a scheduler, samplers, a command line and trace replay, on
hand-written CUDA kernels. Import as ``llm_rs_b200``.
"""
from . import config, parts, models  # noqa: F401  (models registers the architectures)

__version__ = "0.1.0"
