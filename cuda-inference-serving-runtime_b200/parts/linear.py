"""Matrix products of the parts: out[M, N] (float) = a[M, K] @ w[N, K]^T.

Weights keep the checkpoint's [out, in] layout (runtime/model.py:1-5).  Products
always accumulate and return float; bfloat16 operands run on the tensor cores,
float operands as true 32-bit.
"""
from __future__ import annotations

import torch

from ..ops import kernels


def linear(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    out = torch.empty((a.shape[0], w.shape[0]), dtype=torch.float32, device=a.device)
    if a.shape[0] == 0:
        return out
    return kernels.gemm(a, w, out)
