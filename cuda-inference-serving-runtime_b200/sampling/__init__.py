"""Sampling: greedy and temperature."""
from .sampler import DeviceSampler, sample_tokens, uniform

__all__ = ["DeviceSampler", "sample_tokens", "uniform"]
