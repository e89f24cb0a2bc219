from .batch import BatchEntry, StepBatch
from .scheduler import (AdmissionError, FinishReason, Request, RequestStatus, ScheduledRows,
                        Scheduler, SchedulerOutput)

__all__ = ["BatchEntry", "StepBatch", "AdmissionError", "FinishReason", "Request",
           "RequestStatus", "ScheduledRows", "Scheduler", "SchedulerOutput", "ModelRunner",
           "StepError", "LLM", "RequestOutput"]


def __getattr__(name):
    if name == "StepError":
        from .step_builder import StepError
        return StepError
    if name == "ModelRunner":
        from .runner import ModelRunner
        return ModelRunner
    if name in ("LLM", "RequestOutput"):
        from . import llm
        return getattr(llm, name)
    raise AttributeError(name)
