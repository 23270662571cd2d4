"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from a `PartSpec` (its registered kind plus sizes and constants)
and the compute dtype.  It says which tensors it needs under local names
(`tensor_needs`), receives them (`load`), and runs on the device (`forward`).
No part knows which model or which layer it is in: checkpoint names are made by
the model from the layer's prefix and the local name.

Registries: NORMS, POSITIONS, MIXERS, FEED_FORWARDS, ARRANGEMENTS, EMBEDDINGS, HEADS.
`register(registry, kind)` is a class decorator; registering a kind twice is an error.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch

from ..config.spec import CacheUse, PartSpec


@dataclass(frozen=True)
class TensorNeed:
    """A tensor a part loads: shape, and how it is kept.

    role "matrix": a GEMM operand, kept in the compute dtype.
    role "vector": a small per-channel tensor, kept as stored when stored in 32-bit, else in the compute dtype.
    role "table": an integer table, kept as int32.
    `alias` names a tensor (by full checkpoint name) to use when this one is absent (a tied head).
    """
    shape: Tuple[int, ...]
    role: str = "matrix"
    alias: Optional[str] = None


class Part:
    def __init__(self, spec: PartSpec, dtype: torch.dtype):
        self.spec = spec
        self.dtype = dtype

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass

    def kernel_jobs(self) -> List[tuple]:
        """Build jobs (source, defines, extra flags) of the kernel libraries this part launches."""
        return []

    def begin_step(self, ctx) -> None:
        """Called once per step for every part of the model, before the embedding: work that needs the step's metadata
        only (position tables) is launched here, ahead of the layers, instead of inside the first layer that uses it.
        What it makes goes to `ctx.shared`, where the part finds it again."""

    def plan_key(self) -> Optional[tuple]:
        """None: the part needs nothing but the step context.  Otherwise a hashable key naming the launch plan it
        derives from a step's shape (`step_plan`); parts with equal keys share one plan per step, which the engine
        sends to the device inside the step's one metadata copy (`ctx.plan_for(part)` reads it)."""
        return None

    def step_plan(self, host):
        """The `engine.batch.StepPlan` for a step described by `host` (`engine.batch.HostBatch`)."""
        raise NotImplementedError


class PendingNorm:
    """The input of a mixer or feed-forward that has not been normed yet: norm(x + pending).

    A part that can fuse the residual add and the norm into its first product (`accepts_pending_norm = True`)
    asks `fusable(tokens)`; if so it reads `x`, `delta`, `weight`, `eps`, runs its fused kernel with a fresh
    `x_out` buffer from `new_stream_buffer()`, and calls `done(x_out)`.  Otherwise it calls `materialize()`
    and gets the normed tensor from the norm's own kernel.
    """

    def __init__(self, stream, norm: "Norm", dtype: torch.dtype):
        self.stream, self.norm, self.dtype = stream, norm, dtype
        self.x = stream.x
        self.delta = stream.pending
        self.resolved = False      # the norm has run (here or inside a product): stream.x is the sum, nothing is pending

    def fusable(self) -> bool:
        return getattr(self.norm, "fusable_into_product", False)

    @property
    def weight(self) -> torch.Tensor:
        return self.norm.weight

    @property
    def eps(self) -> float:
        return self.norm.eps

    def new_stream_buffer(self) -> Optional[torch.Tensor]:
        """Where x + delta goes; None when nothing is pending (x stays as it is)."""
        return None if self.delta is None else torch.empty_like(self.x)

    def done(self, x_out: Optional[torch.Tensor]) -> None:
        self.stream.take_pending()
        if x_out is not None:
            self.stream.x = x_out
        self.resolved = True

    def materialize(self) -> torch.Tensor:
        out = self.norm.forward(self.stream.x, self.stream.take_pending(), self.dtype)
        self.resolved = True
        return out

    def materialize_once(self) -> torch.Tensor:
        """`materialize`, remembered: a part may ask for the normed tensor more than once while choosing its kernels."""
        if getattr(self, "_tensor", None) is None:
            self._tensor = self.materialize()
        return self._tensor


class Norm(Part):
    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor], out_dtype: torch.dtype,
                rows: Optional[torch.Tensor] = None, write_back: bool = True) -> torch.Tensor:
        """x += delta in place (if given), then return norm(x) in `out_dtype`; `rows` picks rows of x."""
        raise NotImplementedError


class PositionEncoding(Part):
    def rotation(self, ctx) -> Optional["Rotation"]:
        """Per-token rotation tables for this step, or None when the encoding does not rotate."""
        raise NotImplementedError


@dataclass
class Rotation:
    cos: torch.Tensor      # [tokens, rot_half] float
    sin: torch.Tensor
    rot_half: int          # 2 * rot_half leading coordinates of each head are rotated
    interleaved: bool      # pairs (2i, 2i+1) instead of (i, i + rot_half)


class Mixer(Part):
    # True when `forward` takes a `PendingNorm` in place of the normed tensor (and may fuse the norm into its product).
    accepts_pending_norm = False
    # True when `forward` reads the step only through device tensors of the context (never `ctx.host`), so that
    # a captured CUDA graph of it stays right when replayed with other requests, positions and lengths.
    graph_safe = False

    def cache_use(self) -> CacheUse:
        return CacheUse("none")

    def forward(self, h: torch.Tensor, ctx, cache) -> torch.Tensor:
        """h [tokens, hidden] in the compute dtype -> float [tokens, hidden] to add to the residual stream (a part that
        took a `PendingNorm` may instead add its output to `h.stream.x` itself and return None)."""
        raise NotImplementedError


class FeedForward(Part):
    accepts_pending_norm = False

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Embedding(Part):
    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        """int32 [tokens] -> float residual stream [tokens, hidden]."""
        raise NotImplementedError


class Head(Part):
    def forward(self, h: torch.Tensor) -> torch.Tensor:
        """[rows, hidden] in the compute dtype -> float logits [rows, vocab]."""
        raise NotImplementedError


NORMS: Dict[str, type] = {}
POSITIONS: Dict[str, type] = {}
MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
ARRANGEMENTS: Dict[str, type] = {}
EMBEDDINGS: Dict[str, type] = {}
HEADS: Dict[str, type] = {}


def register(registry: Dict[str, type], kind: str):
    def wrap(cls):
        if kind in registry:
            raise ValueError(f"part kind {kind!r} is already registered")
        registry[kind] = cls
        return cls
    return wrap


def build_part(registry: Dict[str, type], spec: PartSpec, dtype: torch.dtype, what: str) -> Any:
    if spec.kind not in registry:
        raise KeyError(f"no {what} registered as {spec.kind!r}; known: {', '.join(sorted(registry)) or 'none'}")
    return registry[spec.kind](spec, dtype)
