"""Typed configuration of the Llama dense decoder, read from its config.json keys.

Parity: runtime/model.py:11-35 (fields and checks) and runtime/checkpoint.py:12-17
(what a checkpoint's config.json may and may not say).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .errors import ConfigError
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

# Head sizes the attention kernels are built for (csrc/attention*.cu are specialised by HEAD_DIM in steps of 16).
HEAD_DIM_STEP, HEAD_DIM_MAX = 16, 256


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None

    REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads")

    def __post_init__(self) -> None:
        sizes = (self.vocab_size, self.hidden_size, self.intermediate_size, self.num_hidden_layers,
                 self.num_attention_heads, self.num_key_value_heads, self.head_dim, self.max_position_embeddings)
        if min(sizes) <= 0:
            raise ConfigError("model dimensions must be positive")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.head_dim % 2:
            raise ConfigError("rotary position encoding needs an even head_dim")
        if self.head_dim % HEAD_DIM_STEP or self.head_dim > HEAD_DIM_MAX:
            # the reference takes any even size up to 256 (runtime/model.py:31-32); the kernels here are specialised
            # in steps of 16, and a size between the steps is refused before any weight is read
            raise ConfigError(f"head_dim {self.head_dim} is not supported: the attention kernels take multiples of "
                              f"{HEAD_DIM_STEP} up to {HEAD_DIM_MAX}")
        if not self.rms_norm_eps > 0 or not self.rope_theta > 0:
            raise ConfigError("rms_norm_eps and rope_theta must be positive")

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "LlamaConfig":
        """Build from a config.json dict; unknown keys are ignored, unsupported options refused."""
        if raw.get("model_type", "llama") != "llama":
            raise ConfigError(f"model_type {raw.get('model_type')!r} is not llama")
        if raw.get("rope_scaling"):
            raise ConfigError("rope_scaling is not implemented (plain rotary positions only)")
        if raw.get("attention_bias") or raw.get("mlp_bias"):
            raise ConfigError("biased projections are not implemented")
        if raw.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act {raw.get('hidden_act')!r} is not implemented (silu only)")
        missing = [k for k in cls.REQUIRED if k not in raw]
        if missing:
            raise ConfigError("config.json lacks " + ", ".join(missing))
        heads = int(raw["num_attention_heads"])
        hidden = int(raw["hidden_size"])
        head_dim = raw.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError("hidden_size must be a multiple of num_attention_heads when head_dim is not given")
            head_dim = hidden // heads
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(
            vocab_size=int(raw["vocab_size"]), hidden_size=hidden, intermediate_size=int(raw["intermediate_size"]),
            num_hidden_layers=int(raw["num_hidden_layers"]), num_attention_heads=heads,
            num_key_value_heads=int(raw.get("num_key_value_heads", heads)), head_dim=int(head_dim),
            rms_norm_eps=float(raw.get("rms_norm_eps", 1e-6)), rope_theta=float(raw.get("rope_theta", 10000.0)),
            max_position_embeddings=int(raw.get("max_position_embeddings", 2048)),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)), eos_token_ids=eos_ids,
            bos_token_id=raw.get("bos_token_id"), torch_dtype=raw.get("torch_dtype") or raw.get("dtype"),
        )

    def to_dict(self) -> dict:
        """The config.json dict of this configuration."""
        out = {
            "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads, "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim, "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
        }
        if self.eos_token_ids:
            out["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if self.torch_dtype:
            out["torch_dtype"] = self.torch_dtype
        return out

    def to_spec(self) -> ModelSpec:
        """Every layer: RMSNorm -> grouped-query attention with rotary positions -> RMSNorm -> SwiGLU."""
        norm = PartSpec("rms_norm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        position = PartSpec("rotary_half", {"theta": self.rope_theta, "dim": self.head_dim})
        mixer = PartSpec("gqa_attention", {
            "hidden_size": self.hidden_size, "num_heads": self.num_attention_heads,
            "num_kv_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "position": position, "window": None, "scale": self.head_dim ** -0.5,
        })
        ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size})
        names = {"mixer": "self_attn.", "mixer_norm": "input_layernorm.",
                 "feed_forward": "mlp.", "feed_forward_norm": "post_attention_layernorm."}
        layers = tuple(
            LayerSpec(prefix=f"model.layers.{i}.", mixer=mixer, mixer_norm=norm, feed_forward=ffn,
                      feed_forward_norm=norm, arrangement="pre_norm", names=names)
            for i in range(self.num_hidden_layers))
        spec = ModelSpec(
            hidden_size=self.hidden_size, vocab_size=self.vocab_size, max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size}),
            embedding_prefix="model.embed_tokens.", layers=layers,
            run=tuple(RunEntry(layer=i) for i in range(self.num_hidden_layers)),
            final_norm=norm, final_norm_prefix="model.norm.",
            head=PartSpec("linear_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                                          "tied_to": "model.embed_tokens.weight" if self.tie_word_embeddings else None}),
            head_prefix="lm_head.", eos_token_ids=self.eos_token_ids)
        spec.validate()
        return spec


register_architecture("LlamaForCausalLM", LlamaConfig, model_types=("llama",))
