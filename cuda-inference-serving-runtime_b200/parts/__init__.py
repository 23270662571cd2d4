"""Parts a model is assembled from: norms, position encodings, mixers, feed-forwards, arrangements."""
from .base import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Embedding, FeedForward,
                   Head, Mixer, Norm, Part, PendingNorm, PositionEncoding, Rotation, TensorNeed, build_part, register)
from . import attention, block, embedding, feedforward, norm, rotary  # noqa: F401  (registers the built-in parts)
from .block import ResidualStream

__all__ = ["ARRANGEMENTS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Embedding",
           "FeedForward", "Head", "Mixer", "Norm", "Part", "PendingNorm", "PositionEncoding", "Rotation", "TensorNeed", "build_part",
           "register", "ResidualStream"]
