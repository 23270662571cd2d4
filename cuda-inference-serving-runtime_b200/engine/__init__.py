"""The engine: model assembly, the step function, the scheduler."""
from .batch import StepEntry
from .model import Model
from .scheduler import Engine, Request
from .step import Stepper

__all__ = ["Engine", "Model", "Request", "StepEntry", "Stepper"]
