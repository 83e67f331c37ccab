from .batch import StepEntry, StepMeta
from .engine import CacheView, Engine, StepContext
from .runtime import Runtime, Workspace, parse_dtype

__all__ = ["StepEntry", "StepMeta", "CacheView", "Engine", "StepContext", "Runtime", "Workspace",
           "parse_dtype"]
