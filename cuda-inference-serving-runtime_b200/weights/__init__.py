"""Weights: safetensors by tensor name, and seeded random weights."""
from .loader import WeightError, load_model_tensors
from .random_init import random_tensors, write_random_model

__all__ = ["WeightError", "load_model_tensors", "random_tensors", "write_random_model"]
