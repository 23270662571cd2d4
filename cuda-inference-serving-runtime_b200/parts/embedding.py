"""Token embedding and the output head.

Parity: runtime/model.py:105 (lookup, no scaling) and runtime/model.py:120 (logits =
norm(x) @ head^T, no bias, no scaling); a tied head is the embedding table itself
(runtime/checkpoint.py:38-39), held once.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels
from .base import EMBEDDINGS, HEADS, Embedding, Head, TensorNeed, register
from .linear import linear


@register(EMBEDDINGS, "token_embedding")
class TokenEmbedding(Embedding):
    """params: vocab_size, hidden_size."""

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.vocab = int(spec["vocab_size"])
        self.hidden = int(spec["hidden_size"])
        self.table = None

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        return {"weight": TensorNeed((self.vocab, self.hidden))}

    def load(self, tensors):
        self.table = tensors["weight"]

    def kernel_jobs(self):
        return [("elementwise.cu", {}, ())]

    def forward(self, token_ids):
        out = torch.empty((token_ids.numel(), self.hidden), dtype=torch.float32, device=token_ids.device)
        return kernels.embedding(self.table, token_ids, out)


@register(HEADS, "linear_head")
class LinearHead(Head):
    """params: vocab_size, hidden_size, tied_to (full name of the tensor to share, or None)."""

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.vocab = int(spec["vocab_size"])
        self.hidden = int(spec["hidden_size"])
        self.tied_to = spec.get("tied_to")
        self.weight = None

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        return {"weight": TensorNeed((self.vocab, self.hidden), alias=self.tied_to)}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def kernel_jobs(self):
        return kernels.gemm_jobs(self.dtype) + (kernels.skinny_jobs() if self.dtype == torch.bfloat16 else [])

    def forward(self, h):
        return linear(h, self.weight)
