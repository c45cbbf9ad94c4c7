from .batch import GroupView, StepContext, StepEntry, StepError, build_context
from .runner import ModelRunner, resolve_dtype

__all__ = ["GroupView", "StepContext", "StepEntry", "StepError", "build_context", "ModelRunner",
           "resolve_dtype"]
from .scheduler import PlannedEntry, Request, SamplingParams, Scheduler, StepPlan  # noqa: E402
from .engine import Engine  # noqa: E402

__all__ += ["PlannedEntry", "Request", "SamplingParams", "Scheduler", "StepPlan", "Engine"]
