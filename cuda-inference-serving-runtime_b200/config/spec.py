"""Architecture-neutral description of a model: parts, layers and the run list.

An architecture's configuration class turns its config.json into a `ModelSpec`.
Everything below the spec (parts, cache manager, step function, loader) reads
only the spec, never the architecture's name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: the key it is registered under and its sizes and constants."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a mixer and a feed-forward, each with its norm, and how they are arranged.

    `names` maps the four slots to the sub-prefix their tensors carry in the
    checkpoint below `prefix` (for Llama: mixer -> "self_attn.", ...).
    """
    prefix: str
    mixer: PartSpec
    mixer_norm: PartSpec
    feed_forward: PartSpec
    feed_forward_norm: PartSpec
    arrangement: str = "pre_norm"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run list.

    `layer` indexes `ModelSpec.layers`; naming a layer twice runs its weights
    twice.  Each entry owns a cache of its own unless `cache_of` names an earlier
    entry, whose cache it then reads without writing.
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class CacheUse:
    """What a mixer needs from the cache manager.

    kind "pages": keys and values in pages ([kv_heads, page, head_dim] per page);
    `window` None keeps every key, an integer keeps the last `window` of them.
    kind "state": a fixed-size tensor per request of `state_shape`/`state_dtype`.
    kind "none": nothing.
    """
    kind: str = "none"
    kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()
    state_dtype: str = "float32"

    def group_key(self) -> tuple:
        return (self.kind, self.kv_heads, self.head_dim, self.window, self.state_shape, self.state_dtype)


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    embedding_prefix: str
    layers: Sequence[LayerSpec]
    run: Sequence[RunEntry]
    final_norm: PartSpec
    final_norm_prefix: str
    head: PartSpec
    head_prefix: str
    eos_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        if not self.layers or not self.run:
            raise ValueError("a model needs at least one layer and one run entry")
        for i, entry in enumerate(self.run):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"run entry {i} names layer {entry.layer}, which does not exist")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < i:
                    raise ValueError(f"run entry {i} reads the cache of entry {entry.cache_of}, which must run earlier")
                if self.run[entry.cache_of].cache_of is not None:
                    raise ValueError(f"run entry {i} reads the cache of entry {entry.cache_of}, which owns none")
