from .core import EngineCore
from .llm import LLM
from .loading import load_model
from .runner import ModelRunner, StepEntry
from .scheduler import Piece, Request, RequestRejected, Scheduler, SchedulerStats

__all__ = ["EngineCore", "LLM", "load_model", "ModelRunner", "StepEntry", "Piece", "Request",
           "RequestRejected", "Scheduler", "SchedulerStats"]
