"""Named shapes: config.json dicts kept as files under config/presets/.

A preset is only a config.json; which architecture it belongs to is decided by the
registry from its `architectures` / `model_type` keys, as for a checkpoint's own file.
"""
from __future__ import annotations

import json
from pathlib import Path

from .errors import ConfigError
from .registry import architecture_for

PRESET_DIR = Path(__file__).resolve().parent / "presets"


def preset_names() -> list:
    return sorted(p.stem for p in PRESET_DIR.glob("*.json"))


def preset_dict(name: str) -> dict:
    """config.json dict of a named shape."""
    path = PRESET_DIR / f"{name}.json"
    if not path.exists():
        raise ConfigError(f"unknown preset {name!r}; known: {', '.join(preset_names())}")
    return json.loads(path.read_text())


def preset(name: str):
    """The typed configuration of a named shape, built by the class its architecture registered."""
    raw = preset_dict(name)
    return architecture_for(raw).config_class.from_dict(raw)
