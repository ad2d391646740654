"""The step function, the scheduler above it, and the Python entry point."""

from .engine import Engine, EngineStats, resolve_dtype
from .params import (Choice, FinishReason, GenerationOutput, GenerationParams, KvCacheOptions, RequestStatus, Usage)
from .runner import ModelRunner, StepEntry
from .scheduler import (PagedSchedulerConfig, ScheduledSequence, ScheduledStep, Scheduler, Sequence, SequenceState)

__all__ = [
    "Choice", "Engine", "EngineStats", "FinishReason", "GenerationOutput", "GenerationParams", "KvCacheOptions",
    "ModelRunner", "PagedSchedulerConfig", "RequestStatus", "ScheduledSequence", "ScheduledStep", "Scheduler",
    "Sequence", "SequenceState", "StepEntry", "Usage", "resolve_dtype",
]
