"""Sampling: parameters and the device sampler."""
from .params import GREEDY_BELOW, SamplingParams

__all__ = ["GREEDY_BELOW", "SamplingParams", "Sampler"]


def __getattr__(name):
    if name == "Sampler":
        from .sampler import Sampler
        return Sampler
    raise AttributeError(name)
