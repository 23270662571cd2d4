"""The engine: model assembly, the step function, the scheduler."""
from .batch import StepEntry
from .model import Model
from .step import Stepper

__all__ = ["Model", "StepEntry", "Stepper"]
