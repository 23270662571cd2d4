"""Tiny random Llama models for tests: config.json dicts and seeded weights.

Two configurations that differ in every size and option (layers, widths, head
counts and grouping, head size, vocabulary, eps, theta, tied or untied head).
Weights are drawn with NumPy only, so the plain implementation, the golden
script and the engine all see the same numbers without sharing engine code.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

TINY_A = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 256,
    "hidden_size": 64,
    "intermediate_size": 176,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0,
    "max_position_embeddings": 512,
    "tie_word_embeddings": True,
    "hidden_act": "silu",
    "eos_token_id": 2,
}

TINY_B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 384,
    "hidden_size": 96,
    "intermediate_size": 250,
    "num_hidden_layers": 3,
    "num_attention_heads": 3,
    "num_key_value_heads": 1,
    "head_dim": 32,
    "rms_norm_eps": 1e-6,
    "rope_theta": 500000.0,
    "max_position_embeddings": 1024,
    "tie_word_embeddings": False,
    "hidden_act": "silu",
    "eos_token_id": 5,
}

# A third shape with sizes that are no power of two anywhere (48-wide heads, 5 query heads).
TINY_C = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 301,
    "hidden_size": 240,
    "intermediate_size": 334,
    "num_hidden_layers": 2,
    "num_attention_heads": 5,
    "num_key_value_heads": 5,
    "head_dim": 48,
    "rms_norm_eps": 3e-6,
    "rope_theta": 25000.0,
    "max_position_embeddings": 1024,
    "tie_word_embeddings": False,
    "hidden_act": "silu",
}

# A fourth shape with 64-wide heads, three query heads to a key head: the head geometry for which the engine has its
# tensor-map decode attention, its tcgen05 prompt attention and the rotation epilogue of the tcgen05 product.
TINY_D = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 173,
    "hidden_size": 384,
    "intermediate_size": 272,
    "num_hidden_layers": 2,
    "num_attention_heads": 6,
    "num_key_value_heads": 2,
    "head_dim": 64,
    "rms_norm_eps": 2e-5,
    "rope_theta": 50000.0,
    "max_position_embeddings": 2048,
    "tie_word_embeddings": True,
    "hidden_act": "silu",
}


def tensor_shapes(cfg: dict) -> dict:
    """Name -> shape of every tensor of a Llama checkpoint (runtime/checkpoint.py:45-56)."""
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hq, hkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or h // hq
    shapes = {"model.embed_tokens.weight": (v, h), "model.norm.weight": (h,)}
    if not cfg.get("tie_word_embeddings", False):
        shapes["lm_head.weight"] = (v, h)
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        shapes[p + "input_layernorm.weight"] = (h,)
        shapes[p + "post_attention_layernorm.weight"] = (h,)
        shapes[p + "self_attn.q_proj.weight"] = (hq * d, h)
        shapes[p + "self_attn.k_proj.weight"] = (hkv * d, h)
        shapes[p + "self_attn.v_proj.weight"] = (hkv * d, h)
        shapes[p + "self_attn.o_proj.weight"] = (h, hq * d)
        shapes[p + "mlp.gate_proj.weight"] = (i, h)
        shapes[p + "mlp.up_proj.weight"] = (i, h)
        shapes[p + "mlp.down_proj.weight"] = (h, i)
    return shapes


def make_weights(cfg: dict, seed: int, scale: float = 0.02, bf16_exact: bool = False) -> dict:
    """Seeded weights as float32 NumPy arrays: matrices N(0, scale), norm weights 1 + N(0, 0.1).

    With `bf16_exact` every value is rounded to a bfloat16-representable number, so
    a bfloat16 engine and a float oracle start from identical weights.
    """
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if len(shape) == 1:
            value = 1.0 + 0.1 * rng.standard_normal(shape)
        else:
            value = scale * rng.standard_normal(shape)
        value = value.astype(np.float32)
        if bf16_exact:
            value = torch.from_numpy(value).to(torch.bfloat16).to(torch.float32).numpy()
        out[name] = value
    return out


def torch_weights(weights: dict) -> dict:
    return {k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in weights.items()}


def write_model_dir(path, cfg: dict, weights: dict, store_dtype=torch.float32) -> Path:
    """Write config.json and model.safetensors (tensors stored in `store_dtype`)."""
    from safetensors.torch import save_file

    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg, indent=1))
    tensors = {k: torch.from_numpy(np.ascontiguousarray(v)).to(store_dtype).contiguous() for k, v in weights.items()}
    save_file(tensors, str(path / "model.safetensors"))
    return path


def random_tokens(cfg: dict, n: int, seed: int) -> list:
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, cfg["vocab_size"], size=n)]
