"""The step function, the scheduler above it, and the generation engine."""

from .context import StepContext
from .runner import ModelRunner, OutOfPages, StepEntry

__all__ = ["ModelRunner", "OutOfPages", "StepContext", "StepEntry"]
