from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import Plan, Portion, Request, Scheduler
from .llm import Engine, Session

__all__ = ["StepEntry", "ModelRunner", "Plan", "Portion", "Request", "Scheduler", "Engine", "Session"]
