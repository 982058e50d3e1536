from .context import StepContext, StepEntry, StepInputError, build_context
from .runner import ModelRunner

__all__ = ["StepContext", "StepEntry", "StepInputError", "build_context", "ModelRunner"]
