from .runner import ModelRunner, StepEntry, StepError
from .scheduler import FinishReason, Request, RequestOutput, RequestStatus, ScheduledRequest, Scheduler

__all__ = ["FinishReason", "ModelRunner", "Request", "RequestOutput", "RequestStatus", "ScheduledRequest",
           "Scheduler", "StepEntry", "StepError"]
