"""The step function, the scheduler above it, and the generation engine."""

from .context import StepContext, StepShape
from .runner import ModelRunner, OutOfPages, StepEntry

__all__ = ["ModelRunner", "OutOfPages", "StepContext", "StepEntry"]
