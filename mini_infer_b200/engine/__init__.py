"""The step function, the runner, the scheduler and the entry points."""

from .runner import ModelRunner  # noqa: F401
from .scheduler import (  # noqa: F401
    ContinuousScheduler,
    EngineFaultError,
    EngineNotRunningError,
    GenerationResult,
    Request,
    RequestHandle,
    RequestState,
    SchedulerLoad,
)
from .step import StepEntry, StepError, StepResult, StepRunner  # noqa: F401
