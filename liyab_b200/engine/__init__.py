"""The step function, the scheduler above it, generation and trace replay."""
from .step import StepEntry, StepOutput, Stepper

__all__ = ["StepEntry", "StepOutput", "Stepper"]
