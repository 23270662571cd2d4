"""SwiGLU feed-forward: down(silu(gate(h)) * up(h)).

Parity: runtime/model.py:116-119, kernels/execution.cu:7-10.  gate_proj and up_proj
are stacked into one [2I, H] matrix at load so one product serves both.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels
from .base import FEED_FORWARDS, FeedForward, TensorNeed, register
from .linear import linear


@register(FEED_FORWARDS, "swiglu")
class SwiGLU(FeedForward):
    """params: hidden_size, intermediate_size."""

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.gate_up = None
        self.down = None

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        return {"gate_proj.weight": TensorNeed((self.inter, self.hidden)),
                "up_proj.weight": TensorNeed((self.inter, self.hidden)),
                "down_proj.weight": TensorNeed((self.hidden, self.inter))}

    def load(self, tensors):
        self.gate_up = torch.cat((tensors["gate_proj.weight"], tensors["up_proj.weight"]), dim=0).contiguous()
        self.down = tensors["down_proj.weight"].contiguous()

    def kernel_jobs(self):
        return [("elementwise.cu", {}, ())] + kernels.gemm_jobs(self.dtype)

    def forward(self, h, ctx):
        gate_up = linear(h, self.gate_up)
        act = torch.empty((h.shape[0], self.inter), dtype=self.dtype, device=h.device)
        kernels.swiglu(gate_up, act)
        return linear(act, self.down)
