from . import attention, attention_plan, build, library, ops
from .library import KernelsUnavailable

__all__ = ["attention", "attention_plan", "build", "library", "ops", "KernelsUnavailable"]
