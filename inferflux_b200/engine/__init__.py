"""Step function, scheduler and the Python entry point."""
from .batch import StepContext, StepEntry
from .runner import ModelRunner, StepError

__all__ = ["StepContext", "StepEntry", "ModelRunner", "StepError"]
