"""The step function, the scheduler above it, generation and trace replay."""
from .step import StepEntry, StepOutput, Stepper

__all__ = ["StepEntry", "StepOutput", "Stepper"]
from .scheduler import PlannedEntry, Request, RequestState, Scheduler, SchedulerStats, StepPlan
from .engine import Engine, EngineConfig, GenerationResult, GenerationStats, generate

__all__ += ["PlannedEntry", "Request", "RequestState", "Scheduler", "SchedulerStats", "StepPlan", "Engine",
            "EngineConfig", "GenerationResult", "GenerationStats", "generate"]
