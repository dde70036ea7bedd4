"""The engine: step function, scheduler, generation entry point, trace replay."""

from .batch import BatchBuilder, StepContext, StepEntry

__all__ = ["BatchBuilder", "Engine", "GenerationOutput", "ModelRunner", "Scheduler", "StepContext", "StepEntry"]


def __getattr__(name):
    if name == "ModelRunner":
        from .runner import ModelRunner
        return ModelRunner
    if name in ("Engine", "GenerationOutput"):
        from . import engine
        return getattr(engine, name)
    if name == "Scheduler":
        from .scheduler import Scheduler
        return Scheduler
    raise AttributeError(name)
