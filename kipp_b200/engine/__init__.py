from .batch import StepEntry, StepMeta
from .engine import CacheView, Engine, StepContext
from .runtime import Runtime, Workspace, parse_dtype

__all__ = ["StepEntry", "StepMeta", "CacheView", "Engine", "StepContext", "Runtime", "Workspace",
           "parse_dtype"]
from .scheduler import Request, RequestState, Scheduler, StepPlan  # noqa: E402

__all__ += ["Request", "RequestState", "Scheduler", "StepPlan", "LLM", "GenerationResult"]


def __getattr__(name):
    if name in ("LLM", "GenerationResult"):
        from . import llm
        return getattr(llm, name)
    raise AttributeError(name)
