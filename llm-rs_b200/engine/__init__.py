"""The step function, the scheduler above it, and the engine a user talks to."""
from .scheduler import Output, Request, Scheduled, Scheduler

__all__ = ["ModelRunner", "StepContext", "StepEntry", "StepError", "Output", "Request", "Scheduled", "Scheduler",
           "Engine", "EngineConfig", "ChatRequest", "GenerationResult", "create_engine", "send_request",
           "poll_token", "destroy_engine"]

_RUNNER = ("ModelRunner", "StepContext", "StepEntry", "StepError")
_ENGINE = ("Engine", "EngineConfig", "ChatRequest", "GenerationResult", "create_engine", "send_request",
           "poll_token", "destroy_engine")


def __getattr__(name):
    # The scheduler is host logic; the runner and the engine pull in torch and the kernels.
    if name in _RUNNER:
        from . import runner
        return getattr(runner, name)
    if name in _ENGINE:
        from . import engine
        return getattr(engine, name)
    raise AttributeError(name)
