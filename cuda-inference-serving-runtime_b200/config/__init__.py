"""Typed configurations, layer specifications and the architecture registry."""
from .spec import CacheUse, LayerSpec, ModelSpec, PartSpec, RunEntry
from .llama import LlamaConfig
from .registry import ARCHITECTURES, Architecture, architecture_for, register_architecture

__all__ = ["CacheUse", "LayerSpec", "ModelSpec", "PartSpec", "RunEntry", "LlamaConfig",
           "ARCHITECTURES", "Architecture", "architecture_for", "register_architecture"]
