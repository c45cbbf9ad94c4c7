from .batch import GroupView, StepContext, StepEntry, StepError, build_context
from .runner import ModelRunner, resolve_dtype

__all__ = ["GroupView", "StepContext", "StepEntry", "StepError", "build_context", "ModelRunner",
           "resolve_dtype"]
