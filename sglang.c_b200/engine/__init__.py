from .engine import Engine, OutOfPages, StepError
from .runtime import Runtime
from .step import StepEntry

__all__ = ["Engine", "OutOfPages", "StepError", "Runtime", "StepEntry"]
