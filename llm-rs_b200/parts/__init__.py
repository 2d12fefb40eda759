"""Parts a model is put together from, their registries, and the generic decoder model."""
from .spec import CacheNeed, LayerSpec, ModelSpec, PartSpec, RunStep, StateNeed, WeightSpec
from .registry import build, kinds, register, unregister
from .base import Block, FeedForward, Mixer, Norm, Part, Plan, PositionEncoding, Runtime, StepInfo
from . import norm, position, attention, mlp, block, embedding  # registers the built-in parts
from .linear import Linear
from .model import DecoderModel

__all__ = ["Plan", "StepInfo", "CacheNeed", "LayerSpec", "ModelSpec", "PartSpec", "RunStep", "StateNeed", "WeightSpec",
           "build", "kinds", "register", "unregister", "Block", "FeedForward", "Mixer", "Norm", "Part",
           "PositionEncoding", "Runtime", "Linear", "DecoderModel"]
