"""SwiGLU feed-forward: down(silu(gate(h)) * up(h)).

Parity: runtime/model.py:116-119, kernels/execution.cu:7-10.  gate_proj and up_proj
are stacked into one [2I, H] matrix at load so one product serves both.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels
from .base import FEED_FORWARDS, FeedForward, TensorNeed, register
from .linear import as_tensor, linear, linear_to_stream, norm_fusable


@register(FEED_FORWARDS, "swiglu")
class SwiGLU(FeedForward):
    """params: hidden_size, intermediate_size."""

    accepts_pending_norm = True

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
        return ([("elementwise.cu", {}, ())] + kernels.gemm_jobs(self.dtype)
                + (kernels.skinny_jobs() if self.dtype == torch.bfloat16 else []))

    def forward(self, h, ctx):
        h0 = h
        tokens = h.x.shape[0] if not isinstance(h, torch.Tensor) else h.shape[0]
        device = h.x.device if not isinstance(h, torch.Tensor) else h.device
        act = torch.empty((tokens, self.inter), dtype=self.dtype, device=device)
        if kernels.skinny_ok(tokens, self.gate_up):
            # few tokens: (norm,) gate and up products and the activation in one launch
            if norm_fusable(h, tokens, self.gate_up):
                x_out = h.new_stream_buffer()
                kernels.skinny_gemm(self.gate_up, tokens, x=h.x, delta=h.delta, norm_w=h.weight, eps=h.eps, x_out=x_out,
                                    epilogue=kernels.EPI_SWIGLU, out=act)
                h.done(x_out)
            else:
                kernels.skinny_gemm(self.gate_up, tokens, act=as_tensor(h), epilogue=kernels.EPI_SWIGLU, out=act)
        else:
            hn = as_tensor(h)
            if kernels.tcgen05_ok(hn, self.gate_up):
                kernels.gemm_tcgen05_swiglu(hn, self.gate_up, act)      # many tokens: SwiGLU is the product's epilogue
            else:
                kernels.swiglu(linear(hn, self.gate_up), act)
        return linear_to_stream(act, self.down, h0)
