from .batch import Span, StepContext, StepEntry
from .core import EngineCore, EngineOptions
from .runner import ModelRunner, StepError

__all__ = ["Span", "StepContext", "StepEntry", "EngineCore", "EngineOptions", "ModelRunner", "StepError"]
