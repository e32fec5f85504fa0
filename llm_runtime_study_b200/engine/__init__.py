from .step import StepContext, StepEntry, StepRunner

__all__ = ["StepContext", "StepEntry", "StepRunner"]
