from .batch import Step, StepBuffers, StepEntry
from .runner import ModelRunner
from .scheduler import FinishReason, Request, Scheduler
from .engine import Engine, GenerationResult

__all__ = ["Step", "StepBuffers", "StepEntry", "ModelRunner", "FinishReason", "Request", "Scheduler",
           "Engine", "GenerationResult"]
