"""How a layer's parts are arranged around the residual stream.

"pre_norm" (runtime/model.py:109-119): x += mixer(norm1(x)); x += feed_forward(norm2(x)).
The add of one sub-block's output is fused into the next norm, so a layer leaves
its feed-forward output pending in the stream instead of adding it itself.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..config.spec import LayerSpec
from .base import ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, PendingNorm, build_part, register


class ResidualStream:
    """The float residual stream x [tokens, hidden] and an output not added to it yet."""

    def __init__(self, x: torch.Tensor):
        self.x = x
        self.pending: Optional[torch.Tensor] = None

    def take_pending(self) -> Optional[torch.Tensor]:
        pending, self.pending = self.pending, None
        return pending


@register(ARRANGEMENTS, "pre_norm")
class PreNormBlock:
    slots = ("mixer_norm", "mixer", "feed_forward_norm", "feed_forward")

    def __init__(self, spec: LayerSpec, dtype: torch.dtype):
        self.spec = spec
        self.dtype = dtype
        self.mixer_norm = build_part(NORMS, spec.mixer_norm, dtype, "norm")
        self.mixer = build_part(MIXERS, spec.mixer, dtype, "mixer")
        self.feed_forward_norm = build_part(NORMS, spec.feed_forward_norm, dtype, "norm")
        self.feed_forward = build_part(FEED_FORWARDS, spec.feed_forward, dtype, "feed-forward")

    def parts(self):
        return {slot: getattr(self, slot) for slot in self.slots}

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        h = PendingNorm(stream, self.mixer_norm, self.dtype)
        mixed = self.mixer.forward(h if self.mixer.accepts_pending_norm else h.materialize(), ctx, cache)
        stream.pending = mixed
        h = PendingNorm(stream, self.feed_forward_norm, self.dtype)
        stream.pending = self.feed_forward.forward(h if self.feed_forward.accepts_pending_norm else h.materialize(), ctx)
