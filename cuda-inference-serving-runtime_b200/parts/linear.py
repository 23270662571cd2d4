"""Matrix products of the parts: out[M, N] (float) = a[M, K] @ w[N, K]^T.

Weights keep the checkpoint's [out, in] layout (runtime/model.py:1-5).  Products
always accumulate and return float; bfloat16 operands run on the tensor cores,
float operands as true 32-bit.
"""
from __future__ import annotations

import torch

from ..ops import kernels


def linear(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Few tokens (a decode step): the weight-streaming kernel; otherwise the library product."""
    out = torch.empty((a.shape[0], w.shape[0]), dtype=torch.float32, device=a.device)
    if a.shape[0] == 0:
        return out
    if kernels.skinny_ok(a.shape[0], w) and a.dtype == torch.bfloat16:
        kernels.skinny_gemm(w, a.shape[0], act=a, epilogue=kernels.EPI_PLAIN, out=out)
        return out
    return kernels.gemm(a, w, out)


def norm_fusable(h, tokens: int, w: torch.Tensor) -> bool:
    """Whether `h` is a pending norm that this product can compute in its own prologue."""
    from .base import PendingNorm
    if not (isinstance(h, PendingNorm) and h.fusable() and tokens <= kernels.SKINNY_NORM_MAX_TOKENS
            and kernels.skinny_ok(tokens, w)):
        return False
    # The persistent streaming kernel would redo the norm of every token in each of its CTAs, in front of a full ring
    # of weights: beyond two tokens the norm kernel, once, and the activation prologue are faster.
    return not (kernels.stream_takes(tokens, w) and tokens > 2)


def as_tensor(h) -> torch.Tensor:
    from .base import PendingNorm
    return h.materialize_once() if isinstance(h, PendingNorm) else h


def stream_target(h, tokens: int, width: int):
    """The residual stream's own tensor, when a product may add its result to it in place: `h` is the part's input as a
    `PendingNorm` that is resolved by now (the norm has run, here or inside a product, so `h.stream.x` holds x + the
    output before and nothing is pending), float, contiguous and [tokens, width].  Otherwise None."""
    from .base import PendingNorm
    if not (isinstance(h, PendingNorm) and h.resolved and h.stream.pending is None):
        return None
    x = h.stream.x
    if x.dtype != torch.float32 or x.shape != (tokens, width) or not x.is_contiguous():
        return None
    return x


def linear_to_stream(a: torch.Tensor, w: torch.Tensor, h):
    """The last product of a sub-block, whose result the block adds to the residual stream: returns the float
    product for the block to add, or None after adding it to the stream in place.

    In place needs the stream's current tensor (`stream_target`) and a product kernel with the add as its epilogue:
    the weight-streaming kernels for few tokens, the tcgen05 product for many.  The sum is the same single float add
    per element that the next norm would otherwise make, so the logits do not change with the path; the norm after
    it then reads one tensor instead of two."""
    x = stream_target(h, a.shape[0], w.shape[0])
    if x is not None and a.shape[0] > 0:
        if kernels.skinny_ok(a.shape[0], w) and a.dtype == torch.bfloat16:
            kernels.skinny_gemm(w, a.shape[0], act=a, epilogue=kernels.EPI_PLAIN, out=x, accumulate=True)
            return None
        if kernels.tcgen05_ok(a, w):
            kernels.gemm_tcgen05(a, w, x, accumulate=True)
            return None
    return linear(a, w)
