from .batch import StepContext, StepEntry
from .scheduler import Engine, EngineOptions, Request, uniform_for

__all__ = ["Engine", "EngineOptions", "Request", "StepContext", "StepEntry", "uniform_for"]
