"""The step function, the scheduler above it, and the engine a user talks to."""
from .runner import ModelRunner, StepContext, StepEntry, StepError

__all__ = ["ModelRunner", "StepContext", "StepEntry", "StepError"]
