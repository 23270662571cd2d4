"""Rotary position encoding with split-half pairing.

Parity: runtime/reference.py:9-15 and kernels/ops.cu:21-33: pair (i, i + D/2) turns
by pos * theta^(-2i/D); keys are cached already rotated.  The frequencies are taken
in float64 on the host and the angles in float64 on the device; the tables a step
uses are computed once per step and shared by all layers with the same constants.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from .base import POSITIONS, PositionEncoding, Rotation, register


@register(POSITIONS, "rotary_half")
class RotaryHalf(PositionEncoding):
    """params: theta, dim (rotated width, at most the head size)."""

    interleaved = False

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.theta = float(spec["theta"])
        self.dim = int(spec["dim"])
        if self.dim % 2:
            raise ValueError("rotary position encoding needs an even width")
        self._inv_freq = None

    def kernel_jobs(self):
        return [("elementwise.cu", {}, ())]

    def inv_freq(self, device) -> torch.Tensor:
        if self._inv_freq is None or self._inv_freq.device != device:
            half = self.dim // 2
            host = self.theta ** (-torch.arange(half, dtype=torch.float64) * 2.0 / self.dim)
            self._inv_freq = host.to(device)
        return self._inv_freq

    def rotation(self, ctx) -> Rotation:
        key = ("rotary", self.theta, self.dim, self.interleaved)
        cached = ctx.shared.get(key)
        if cached is None:
            half = self.dim // 2
            cos = torch.empty((ctx.n_tokens, half), dtype=torch.float32, device=ctx.device)
            sin = torch.empty_like(cos)
            kernels.rotary_tables(ctx.positions, self.inv_freq(ctx.device), cos, sin)
            cached = Rotation(cos, sin, half, self.interleaved)
            ctx.shared[key] = cached
        return cached


@register(POSITIONS, "none")
class NoPosition(PositionEncoding):
    def rotation(self, ctx):
        return None
