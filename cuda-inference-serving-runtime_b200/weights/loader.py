"""Read safetensors by tensor name into the tensors a model asked for.

Parity: runtime/checkpoint.py:18-41 (every *.safetensors of the folder, duplicate
names refused, missing or wrongly shaped tensors refused, tied head taken from the
embedding).  Differences: tensors are not widened to float32 (matrices are kept in
the compute dtype, a vector stored in 32-bit stays 32-bit, integer tables become
int32), and one error lists everything that is wrong instead of the first name.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Mapping

import torch

from ..parts.base import TensorNeed


class WeightError(ValueError):
    """The checkpoint does not fit the model; the message lists every problem."""


def _index_files(directory: Path) -> Dict[str, Path]:
    from safetensors import safe_open

    index = directory / "model.safetensors.index.json"
    if index.exists():
        files = sorted({directory / f for f in json.loads(index.read_text())["weight_map"].values()})
    else:
        files = sorted(directory.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors checkpoint found in {directory}")
    where: Dict[str, Path] = {}
    for path in files:
        with safe_open(str(path), framework="pt") as handle:
            for name in handle.keys():
                if name in where:
                    raise WeightError(f"duplicate tensor {name} in {where[name].name} and {path.name}")
                where[name] = path
    return where


def _kept_dtype(need: TensorNeed, stored: torch.dtype, dtype: torch.dtype) -> torch.dtype:
    if need.role == "table":
        return torch.int32
    if need.role == "vector" and stored == torch.float32:
        return torch.float32
    return dtype


def load_model_tensors(directory, needs: Mapping[str, TensorNeed], dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    from safetensors import safe_open

    directory = Path(directory)
    where = _index_files(directory)
    aliased = {name for name, need in needs.items() if need.alias is not None}
    wanted = {name: need for name, need in needs.items() if need.alias is None}
    missing = sorted(n for n in wanted if n not in where)
    unexpected = sorted(n for n in where if n not in wanted and n not in aliased)
    wrong = []
    by_file: Dict[Path, list] = {}
    for name in wanted:
        if name in where:
            by_file.setdefault(where[name], []).append(name)
    for path, names in by_file.items():
        with safe_open(str(path), framework="pt") as handle:
            for name in names:
                shape = tuple(handle.get_slice(name).get_shape())
                if shape != tuple(wanted[name].shape):
                    wrong.append(f"{name}: checkpoint has {list(shape)}, model needs {list(wanted[name].shape)}")
    if missing or unexpected or wrong:
        parts = [f"checkpoint in {directory} does not fit the model"]
        if missing:
            parts.append(f"missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            parts.append(f"unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            parts.append(f"wrong shapes ({len(wrong)}): " + "; ".join(sorted(wrong)))
        raise WeightError("\n".join(parts))
    out: Dict[str, torch.Tensor] = {}
    for path, names in by_file.items():
        with safe_open(str(path), framework="pt") as handle:
            for name in names:
                tensor = handle.get_tensor(name)
                if tensor.dtype not in (torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.int64):
                    raise WeightError(f"unsupported weight dtype {tensor.dtype} of {name}")
                out[name] = tensor.to(device=device, dtype=_kept_dtype(wanted[name], tensor.dtype, dtype)).contiguous()
    return out
