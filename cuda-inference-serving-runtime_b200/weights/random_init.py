"""Seeded random weights: in memory for a model, or written as a model folder.

Matrices are drawn N(0, 0.02), per-channel vectors (norm weights) 1 + N(0, 0.1).  Each
tensor has its own stream keyed by (seed, tensor name), so the values do not depend
on the order or on which other tensors exist.  The reference's `toy_weights`
(runtime/model.py:38-55) draws N(0,1)/sqrt(in) with unit norms from one stream; the
recipe here is the one the measurements are quoted on.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Dict, Mapping

import torch

from ..parts.base import TensorNeed

MATRIX_STD = 0.02
VECTOR_STD = 0.1
DEVICE_DRAW_THRESHOLD = 1 << 22   # tensors above this many elements are drawn on the device


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def draw(name: str, need: TensorNeed, seed: int, device=None) -> torch.Tensor:
    """float32 values of one tensor."""
    shape = tuple(need.shape)
    numel = 1
    for s in shape:
        numel *= s
    on_device = device is not None and numel > DEVICE_DRAW_THRESHOLD
    gen = torch.Generator(device=device if on_device else "cpu")
    gen.manual_seed(_tensor_seed(seed, name))
    if need.role == "table":
        return torch.zeros(shape, dtype=torch.int32)
    values = torch.randn(shape, generator=gen, dtype=torch.float32, device=device if on_device else "cpu")
    if need.role == "vector":
        return 1.0 + VECTOR_STD * values
    return MATRIX_STD * values


def random_tensors(needs: Mapping[str, TensorNeed], seed: int, dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    out = {}
    for name, need in needs.items():
        if need.alias is not None:
            continue
        value = draw(name, need, seed, device)
        kept = torch.int32 if need.role == "table" else (torch.float32 if need.role == "vector" else dtype)
        out[name] = value.to(device=device, dtype=kept).contiguous()
    return out


def write_random_model(directory, config, seed: int = 0, store_dtype: str = "bfloat16") -> Path:
    """Write config.json and model.safetensors for `config` (preset name, dict or configuration object)."""
    from safetensors.torch import save_file

    from ..config import architecture_for
    from ..config.presets import preset_dict
    from ..engine.model import Model, resolve_dtype

    raw = preset_dict(config) if isinstance(config, str) else (dict(config) if isinstance(config, dict) else config.to_dict())
    cfg = architecture_for(raw).config_class.from_dict(raw)
    kept = resolve_dtype(store_dtype)
    model = Model(cfg.to_spec(), kept, config=raw, device=None)
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    out_config = cfg.to_dict() if hasattr(cfg, "to_dict") else raw
    out_config["torch_dtype"] = "float32" if kept == torch.float32 else "bfloat16"
    (directory / "config.json").write_text(json.dumps(out_config, indent=1))
    tensors = {}
    for name, need in model.tensor_needs().items():
        if need.alias is not None:
            continue
        value = draw(name, need, seed)
        tensors[name] = value if need.role == "table" else value.to(kept).contiguous()
    save_file(tensors, str(directory / "model.safetensors"))
    return directory
