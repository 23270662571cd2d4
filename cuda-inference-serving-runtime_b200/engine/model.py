"""A model assembled from a `ModelSpec`: embedding, layers run in the order of the
run list, final norm, head.  Nothing here names an architecture.

Parity: runtime/model.py:58-120 (`Model`): there the forward pass is one monolithic
loop with string-built weight names; here each layer is an arrangement of registered
parts and the run list is data.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional, Union

import torch

from ..cache import CacheManager
from ..config import ModelSpec, architecture_for
from ..parts import ARRANGEMENTS, EMBEDDINGS, HEADS, NORMS, ResidualStream, TensorNeed, build_part
from ..ops import build as kernel_build

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, torch.float32: torch.float32,
          torch.bfloat16: torch.bfloat16}


def resolve_dtype(dtype) -> torch.dtype:
    if dtype not in DTYPES:
        raise ValueError(f"dtype must be float32 or bfloat16, not {dtype!r}")
    return DTYPES[dtype]


def require_cuda() -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device: this engine runs its own sm_100a kernels and has no CPU path")
    return torch.device("cuda", torch.cuda.current_device())


class Model:
    def __init__(self, spec: ModelSpec, dtype, config: Optional[dict] = None, device: Optional[torch.device] = None):
        spec.validate()
        self.spec = spec
        self.dtype = resolve_dtype(dtype)
        self.config = config or {}
        self.device = device
        self.embedding = build_part(EMBEDDINGS, spec.embedding, self.dtype, "embedding")
        self.layers = []
        for layer_spec in spec.layers:
            if layer_spec.arrangement not in ARRANGEMENTS:
                raise KeyError(f"no layer arrangement registered as {layer_spec.arrangement!r}")
            self.layers.append(ARRANGEMENTS[layer_spec.arrangement](layer_spec, self.dtype))
        self.final_norm = build_part(NORMS, spec.final_norm, self.dtype, "norm")
        self.head = build_part(HEADS, spec.head, self.dtype, "head")
        self.loaded = False

    # ---------------------------------------------------------------- tensors
    def _named_parts(self):
        yield self.spec.embedding_prefix, self.embedding
        for layer_spec, layer in zip(self.spec.layers, self.layers):
            for slot, part in layer.parts().items():
                yield layer_spec.prefix + layer_spec.names.get(slot, slot + "."), part
        yield self.spec.final_norm_prefix, self.final_norm
        yield self.spec.head_prefix, self.head

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        """Checkpoint name -> need, for every tensor of the model."""
        needs: Dict[str, TensorNeed] = {}
        for prefix, part in self._named_parts():
            for local, need in part.tensor_needs().items():
                needs[prefix + local] = need
        return needs

    def load_tensors(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Hand each part its tensors (already on the device, in their kept dtype)."""
        for prefix, part in self._named_parts():
            local = {}
            for name, need in part.tensor_needs().items():
                full = prefix + name
                local[name] = tensors[need.alias] if need.alias is not None else tensors[full]
            part.load(local)
        self.loaded = True

    def kernel_jobs(self) -> List[tuple]:
        jobs, seen = [], set()
        for _, part in self._named_parts():
            for job in part.kernel_jobs():
                key = repr(job)
                if key not in seen:
                    seen.add(key)
                    jobs.append(job)
        jobs.append(("sampling.cu", {}, ()))
        return jobs

    def planners(self) -> list:
        """The parts whose launch plans travel with every step's metadata, one per plan key."""
        from .batch import unique_planners

        return unique_planners(part for _, part in self._named_parts())

    def compile_kernels(self) -> None:
        """Build, in parallel, exactly the kernel libraries this model launches."""
        kernel_build.compile_many(self.kernel_jobs())

    # ---------------------------------------------------------------- cache
    def cache_uses(self) -> list:
        uses = []
        for entry in self.spec.run:
            if entry.cache_of is not None:
                uses.append(entry.cache_of)
            else:
                uses.append(self.layers[entry.layer].mixer.cache_use())
        return uses

    def make_cache(self, n_pages: int, page_size: int = 16, max_slots: int = 64) -> CacheManager:
        return CacheManager(self.cache_uses(), n_pages, page_size, max_slots, self.spec.max_positions,
                            dtype=self.dtype, device=self.device)

    # ---------------------------------------------------------------- forward
    def step_beginners(self) -> list:
        """The parts of the layers that run, in run order, whose class has a `begin_step` of its own."""
        found = getattr(self, "_step_beginners", None)
        if found is None:
            from ..parts.base import Part
            found, seen = [], set()
            for entry in self.spec.run:
                for part in self.layers[entry.layer].parts().values():
                    if id(part) not in seen and getattr(type(part), "begin_step", Part.begin_step) is not Part.begin_step:
                        seen.add(id(part))
                        found.append(part)
            self._step_beginners = found
        return found

    def forward(self, ctx, cache: CacheManager) -> torch.Tensor:
        """Run the step's tokens through every run entry; float logits [wanted rows, vocab]."""
        for part in self.step_beginners():
            part.begin_step(ctx)
        stream = ResidualStream(self.embedding.forward(ctx.token_ids))
        for index, entry in enumerate(self.spec.run):
            self.layers[entry.layer].forward(stream, ctx, cache.binding(index, reads_from=entry.cache_of))
        if ctx.logit_rows.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        h = self.final_norm.forward(stream.x, stream.take_pending(), self.dtype, rows=ctx.logit_rows, write_back=False)
        return self.head.forward(h)

    # ---------------------------------------------------------------- construction
    @classmethod
    def from_pretrained(cls, directory: Union[str, Path], dtype="bfloat16") -> "Model":
        """Load a folder with config.json and safetensors; the model is chosen by config.json."""
        from ..weights import load_model_tensors

        directory = Path(directory)
        config_path = directory / "config.json"
        if not config_path.exists():
            raise FileNotFoundError(f"{config_path} does not exist")
        raw = json.loads(config_path.read_text())
        arch = architecture_for(raw)
        config = arch.config_class.from_dict(raw)
        device = require_cuda()
        model = cls(config.to_spec(), dtype, config=raw, device=device)
        model.compile_kernels()
        model.load_tensors(load_model_tensors(directory, model.tensor_needs(), model.dtype, device))
        return model

    @classmethod
    def from_config(cls, config, seed: int = 0, dtype="bfloat16") -> "Model":
        """A model with seeded random weights, made on the device without touching the disk.

        `config` is a preset name, a config.json dict, or a configuration object.
        """
        from ..config.presets import preset_dict
        from ..weights import random_tensors

        raw = preset_dict(config) if isinstance(config, str) else (config if isinstance(config, dict) else config.to_dict())
        arch = architecture_for(raw)
        cfg = arch.config_class.from_dict(raw)
        device = require_cuda()
        model = cls(cfg.to_spec(), dtype, config=raw, device=device)
        model.compile_kernels()
        model.load_tensors(random_tensors(model.tensor_needs(), seed, model.dtype, device))
        return model
