from .batch import StateView, StepBuffers, StepContext
from .engine import Engine, StepEntry
from .scheduler import Request, Scheduler, StepOutput

__all__ = ["StateView", "StepBuffers", "StepContext", "Engine", "StepEntry", "Request", "Scheduler",
           "StepOutput"]
