from .batch import Entry, StepBatch
from .engine import Engine
from .scheduler import Scheduled, Scheduler, SchedulerError
from .llm import LLM, RequestMetrics, RequestOutput, StepRecord

__all__ = ["Entry", "StepBatch", "Engine", "Scheduled", "Scheduler", "SchedulerError", "LLM",
           "RequestMetrics", "RequestOutput", "StepRecord"]
