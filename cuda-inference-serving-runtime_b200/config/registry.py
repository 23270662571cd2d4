"""One registry from an architecture's name (config.json `architectures[0]`) to its model.

An entry gives the configuration class (with `from_dict(raw)`, `to_dict()` and `to_spec()`).
The model itself is always assembled by `engine.model.Model` from the spec, so adding an
architecture means adding a configuration class that emits a spec, and any parts the spec
names that are not registered yet.  This module knows no architecture: each one registers
itself where its configuration class is defined (config/llama.py does so for Llama).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping

from .errors import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any
    model_types: tuple = ()


ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Any, model_types: tuple = ()) -> None:
    if name in ARCHITECTURES:
        raise ValueError(f"architecture {name!r} is already registered")
    ARCHITECTURES[name] = Architecture(name, config_class, tuple(model_types))


def architecture_for(raw: Mapping[str, Any]) -> Architecture:
    """Pick the architecture by `architectures[0]`, else by `model_type`."""
    names = raw.get("architectures") or []
    for name in names:
        if name in ARCHITECTURES:
            return ARCHITECTURES[name]
    model_type = raw.get("model_type")
    for arch in ARCHITECTURES.values():
        if model_type is not None and model_type in arch.model_types:
            return arch
    raise ConfigError(f"no registered architecture for architectures={list(names)!r}, model_type={model_type!r}; "
                      f"known: {', '.join(sorted(ARCHITECTURES))}")

