"""Typed configurations, layer specifications and the architecture registry."""
from .errors import ConfigError
from .spec import CacheUse, LayerSpec, ModelSpec, PartSpec, RunEntry
from .registry import ARCHITECTURES, Architecture, architecture_for, register_architecture
from .llama import LlamaConfig      # registers LlamaForCausalLM
from .presets import preset, preset_dict, preset_names

__all__ = ["CacheUse", "ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "RunEntry", "LlamaConfig",
           "ARCHITECTURES", "Architecture", "architecture_for", "register_architecture",
           "preset", "preset_dict", "preset_names"]
