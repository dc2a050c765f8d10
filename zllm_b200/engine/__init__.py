from .batch import StepEntry
from .runner import ModelRunner

__all__ = ["StepEntry", "ModelRunner"]
