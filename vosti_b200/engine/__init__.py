from .batch import StepContext, StepEntry
from .request import AdmissionStatus, Request
from .scheduler import PlanRow, Scheduler, SchedulerConfig, StepPlan

__all__ = ["StepContext", "StepEntry", "AdmissionStatus", "Request", "PlanRow", "Scheduler",
           "SchedulerConfig", "StepPlan", "Engine", "ModelRunner"]


def __getattr__(name):
    # Engine and ModelRunner pull in the CUDA library; load them on first use so that the
    # scheduler and cache manager import on a machine without a GPU.
    if name == "Engine":
        from .engine import Engine
        return Engine
    if name == "ModelRunner":
        from .runner import ModelRunner
        return ModelRunner
    raise AttributeError(name)
