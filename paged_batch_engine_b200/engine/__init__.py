from .batch import StepContext, StepEntry, attention_work_arrays
from .scheduler import Request, Scheduler, SchedulerConfig, SchedulerOutput

__all__ = ["StepContext", "StepEntry", "attention_work_arrays", "ModelRunner", "build_model",
           "Request", "Scheduler", "SchedulerConfig", "SchedulerOutput", "Engine", "GenerationResult",
           "generate"]


def __getattr__(name):
    if name in ("ModelRunner", "build_model"):
        from . import runner
        return getattr(runner, name)
    if name in ("Engine", "GenerationResult", "generate"):
        from . import engine
        return getattr(engine, name)
    raise AttributeError(name)
