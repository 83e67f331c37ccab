from .batch import StepEntry
from .engine import Engine, ExternalContext, device_tensor
from .runtime import parse_dtype
from .scheduler import Request, RequestState, Scheduler, StepPlan

__all__ = ["StepEntry", "Engine", "ExternalContext", "device_tensor", "parse_dtype", "Request", "RequestState",
           "Scheduler", "StepPlan", "LLM", "GenerationResult"]


def __getattr__(name):
    if name in ("LLM", "GenerationResult"):
        from . import llm
        return getattr(llm, name)
    raise AttributeError(name)
