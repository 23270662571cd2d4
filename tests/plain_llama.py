"""Plain, slow Llama forward pass: the oracle every engine test compares with.

Whole sequences, no cache, no batching, one function per part, torch on the CPU.
It shares no code with the engine package.  Every function cites the reference
formula it restates (paths are inside nehanmohammed19/cuda-inference-serving-runtime).

`tests/golden/` holds logits of the reference's own NumPy model for two tiny random
models; `tests/test_plain_vs_golden.py` compares this file with them, so this file
rests on the reference's code, not only on a reading of its formulas.

Weights are a dict of torch tensors under Hugging Face Llama names with [out, in]
linear layout (runtime/model.py:1-5, runtime/checkpoint.py:45-56).  `dtype` selects
the arithmetic: float64 (default, the tightest oracle) or float32.

`storage` (None or torch.bfloat16) restates the reference's 16-bit modes (runtime/model.py:3-4,
docs/RUNTIME.md:16-19: activations between kernels and the cache are stored in 16 bits, every sum is
taken in 32): with it, the values that the engine's bfloat16 path keeps in bfloat16 (the norm's output,
the rotated queries and keys, the values, the attention output, the SwiGLU output) are rounded to that
type where they are produced and the arithmetic goes on in `dtype`; the residual stream and the logits
are not rounded.  Against this twin a bfloat16 engine differs only by what is left: the order of its
sums and the rounding of the attention probabilities.
"""
from __future__ import annotations

import math

import torch


def stored(x: torch.Tensor, storage) -> torch.Tensor:
    """x as it reads back after being stored in `storage` (None: unchanged)."""
    return x if storage is None else x.to(storage).to(x.dtype)


def embed(table: torch.Tensor, tokens) -> torch.Tensor:
    """x[t, :] = table[token[t], :], no scaling (runtime/model.py:105)."""
    return table[torch.as_tensor(list(tokens), dtype=torch.long)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w (runtime/reference.py:5-6)."""
    return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def rotary(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Split-half rotation of [T, heads, D] (runtime/reference.py:9-15).

    Pair (i, i + D/2) turns by angle pos * theta^(-2i/D).
    """
    d = x.shape[-1]
    half = d // 2
    inv = theta ** (-torch.arange(half, dtype=torch.float64) * 2.0 / d)
    angle = positions.to(torch.float64)[:, None] * inv[None, :]
    cos = torch.cos(angle)[:, None, :].to(x.dtype)
    sin = torch.sin(angle)[:, None, :].to(x.dtype)
    a, b = x[..., :half], x[..., half:]
    return torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int | None = None) -> torch.Tensor:
    """Causal grouped-query attention over a whole sequence.

    q [T, Hq, D], k and v [T, Hkv, D].  Consecutive query heads share a KV head
    (runtime/reference.py:18-27); scores are scaled by 1/sqrt(D); token t sees
    tokens 0..t (runtime/reference.py:30-31).  `window`, when given, keeps only
    the last `window` keys (t - window < s <= t); the reference has no window.
    """
    t, hq, d = q.shape
    groups = hq // k.shape[1]
    index = torch.arange(hq) // groups
    kk, vv = k[:, index], v[:, index]  # [T, Hq, D]
    scores = torch.einsum("thd,shd->hts", q, kk) / math.sqrt(d)
    row = torch.arange(t)[:, None]
    col = torch.arange(t)[None, :]
    mask = col > row
    if window is not None:
        mask = mask | (col <= row - window)
    scores = scores.masked_fill(mask[None], float("-inf"))
    scores = scores - scores.max(dim=-1, keepdim=True).values
    p = torch.exp(scores)
    p = p / p.sum(dim=-1, keepdim=True)
    return torch.einsum("hts,shd->thd", p, vv)


def swiglu_mlp(h: torch.Tensor, gate_w: torch.Tensor, up_w: torch.Tensor, down_w: torch.Tensor, storage=None) -> torch.Tensor:
    """down(silu(gate(h)) * up(h)), silu(g) = g / (1 + exp(-g)) (runtime/model.py:117-119, kernels/execution.cu:7-10)."""
    gate = h @ gate_w.T
    return stored(gate / (1 + torch.exp(-gate)) * (h @ up_w.T), storage) @ down_w.T


def attention_block(h, w, prefix, positions, cfg, window=None, storage=None):
    """q/k/v projections, rotation of q and k, attention, output projection (runtime/model.py:110-115)."""
    hq, hkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // hq
    q = (h @ w[prefix + "self_attn.q_proj.weight"].T).reshape(-1, hq, d)
    k = (h @ w[prefix + "self_attn.k_proj.weight"].T).reshape(-1, hkv, d)
    v = stored((h @ w[prefix + "self_attn.v_proj.weight"].T).reshape(-1, hkv, d), storage)
    q = stored(rotary(q, positions, cfg["rope_theta"]), storage)
    k = stored(rotary(k, positions, cfg["rope_theta"]), storage)       # keys are cached rotated
    out = stored(causal_attention(q, k, v, window).reshape(-1, hq * d), storage)
    return out @ w[prefix + "self_attn.o_proj.weight"].T


def decoder_layer(x, w, layer, positions, cfg, storage=None):
    """Pre-norm residual block (runtime/model.py:109-119)."""
    p = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    h = stored(rms_norm(x, w[p + "input_layernorm.weight"], eps), storage)
    x = x + attention_block(h, w, p, positions, cfg, storage=storage)
    h = stored(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps), storage)
    return x + swiglu_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"], storage)


def forward(cfg: dict, weights: dict, tokens, dtype=torch.float64, storage=None) -> torch.Tensor:
    """Logits [T, V] at every position of one whole sequence (runtime/model.py:105-120).

    `cfg` is the config.json dict.  A tied head uses the embedding table
    (runtime/checkpoint.py:38-39).  `storage`: see the head of this file.
    """
    w = {k: v.to(dtype) for k, v in weights.items()}
    positions = torch.arange(len(tokens))
    x = embed(w["model.embed_tokens.weight"], tokens)
    for layer in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, layer, positions, cfg, storage)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return stored(rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"]), storage) @ head.T


def greedy(logits: torch.Tensor) -> int:
    """argmax, lowest index on ties (runtime/engine.py:99)."""
    return int(torch.argmax(logits.to(torch.float64)).item())


def generate_greedy(cfg: dict, weights: dict, prompt, new_tokens: int, eos=None, dtype=torch.float64):
    """Greedy generation by re-running the whole sequence for each token (runtime/engine.py:97-110).

    The first new token comes from the last prompt position; generation stops after
    `new_tokens` tokens or when a token equals `eos`.
    """
    seq = list(prompt)
    out = []
    for _ in range(new_tokens):
        token = greedy(forward(cfg, weights, seq, dtype)[-1])
        out.append(token)
        seq.append(token)
        if eos is not None and token == eos:
            break
    return out


def temperature_probabilities(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """softmax(logits / T) in float64; the reference samples greedily only, this is the textbook form."""
    z = logits.to(torch.float64) / temperature
    z = z - z.max()
    p = torch.exp(z)
    return p / p.sum()


def sample_inverse_cdf(logits: torch.Tensor, temperature: float, u: float) -> int:
    """First index whose cumulative probability exceeds u (u uniform in [0, 1))."""
    c = torch.cumsum(temperature_probabilities(logits, temperature), dim=0)
    idx = int(torch.searchsorted(c, torch.tensor(u, dtype=torch.float64), right=True).item())
    return min(idx, logits.numel() - 1)
