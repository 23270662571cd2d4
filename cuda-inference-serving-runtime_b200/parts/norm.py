"""RMSNorm, fused with the residual add that precedes it.

Parity: runtime/reference.py:5-6, kernels/ops.cu:3-19, kernels/execution.cu:12-24
(y = x * rsqrt(mean(x^2) + eps) * w; no bias, no 1+w offset).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import kernels
from .base import NORMS, Norm, TensorNeed, register


@register(NORMS, "rms_norm")
class RMSNorm(Norm):
    """params: size (width), eps."""

    fusable_into_product = True     # y = x * rsqrt(mean(x^2) + eps) * w is what the products' norm prologue computes

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight: Optional[torch.Tensor] = None

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        return {"weight": TensorNeed((self.size,), role="vector")}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def kernel_jobs(self):
        return [("elementwise.cu", {}, ())]

    def forward(self, x, delta, out_dtype, rows=None, write_back=True):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype, device=x.device)
        return kernels.add_rmsnorm(x, delta, self.weight, self.eps, out, rows=rows, write_back=write_back)
