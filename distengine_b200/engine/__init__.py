from .step import KernelStatusError, StepEntry, StepRunner

__all__ = ["KernelStatusError", "StepEntry", "StepRunner"]
