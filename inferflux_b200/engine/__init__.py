"""Step function, scheduler and the Python entry point."""
from .batch import StepContext, StepEntry
from .engine import Engine, EngineStats, GenerationResult
from .load_spec import ModelLoadSpec
from .runner import ModelRunner, StepError
from .scheduler import Request, Scheduler, SchedulerConfig, StepPlan

__all__ = ["StepContext", "StepEntry", "Engine", "EngineStats", "GenerationResult", "ModelLoadSpec", "ModelRunner", "StepError",
           "Request", "Scheduler", "SchedulerConfig", "StepPlan"]
