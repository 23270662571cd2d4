"""New parts and a new architecture, defined here and registered without touching the engine's files.

A toy mixer that carries a fixed-size state per request (an exponential running mean),
a toy architecture whose layers use different mixers, whose run list names a layer
twice and lets one entry read another entry's cache.  None of this is a model of
anyone's; it shows that the interfaces carry parts the engine does not ship.
"""
import json

import numpy as np
import pytest
import torch
from safetensors.torch import save_file

import plain_llama as pl
import replay

pytestmark = pytest.mark.gpu

HIDDEN, HEADS, KV, DIM, INTER, VOCAB, DECAY = 48, 3, 1, 16, 80, 97, 0.75


def register_toys():
    from cisr_b200.config import (ARCHITECTURES, CacheUse, LayerSpec, ModelSpec, PartSpec, RunEntry,
                                  register_architecture)
    from cisr_b200.parts import MIXERS, Mixer, TensorNeed, register
    from cisr_b200.parts.linear import linear

    if "toy_running_mean" not in MIXERS:
        @register(MIXERS, "toy_running_mean")
        class ToyRunningMean(Mixer):
            """state <- decay * state + (1 - decay) * h_t per token; output = W @ state.  State: [hidden] per request."""

            def __init__(self, spec, dtype):
                super().__init__(spec, dtype)
                self.hidden, self.decay = int(spec["hidden_size"]), float(spec["decay"])

            def tensor_needs(self):
                return {"mix.weight": TensorNeed((self.hidden, self.hidden))}

            def load(self, tensors):
                self.w = tensors["mix.weight"]

            def cache_use(self):
                return CacheUse("state", state_shape=(self.hidden,), state_dtype="float32")

            def forward(self, h, ctx, cache):
                states = torch.empty((h.shape[0], self.hidden), dtype=torch.float32, device=h.device)
                for r, slot in enumerate(ctx.host.slots):
                    s = cache.state[slot]
                    for t in range(ctx.host.q_start[r], ctx.host.q_start[r] + ctx.host.q_len[r]):
                        s = self.decay * s + (1 - self.decay) * h[t].float()
                        states[t] = s
                    cache.state[slot] = s
                return linear(states.to(self.dtype), self.w)

    if "ToyMixedForCausalLM" not in ARCHITECTURES:
        class ToyConfig:
            def __init__(self, raw):
                self.raw = raw

            @classmethod
            def from_dict(cls, raw):
                return cls(dict(raw))

            def to_dict(self):
                return dict(self.raw)

            def to_spec(self):
                r = self.raw
                norm = PartSpec("rms_norm", {"size": r["width"], "eps": r["eps"]})
                attention = PartSpec("gqa_attention", {"hidden_size": r["width"], "num_heads": r["heads"], "num_kv_heads": r["kv_heads"],
                                                       "head_dim": r["head_dim"], "window": None,
                                                       "position": PartSpec("rotary_half", {"theta": r["theta"], "dim": r["head_dim"]})})
                toy = PartSpec("toy_running_mean", {"hidden_size": r["width"], "decay": r["decay"]})
                ffn = PartSpec("swiglu", {"hidden_size": r["width"], "intermediate_size": r["inner"]})
                names = {"mixer": "mixer.", "mixer_norm": "norm1.", "feed_forward": "ffn.", "feed_forward_norm": "norm2."}
                layers = tuple(LayerSpec(prefix=f"blocks.{i}.", mixer=m, mixer_norm=norm, feed_forward=ffn, feed_forward_norm=norm, names=names)
                               for i, m in enumerate((attention, toy)))
                run = tuple(RunEntry(**e) for e in r["run"])
                return ModelSpec(hidden_size=r["width"], vocab_size=r["vocab"], max_positions=r["max_len"],
                                 embedding=PartSpec("token_embedding", {"vocab_size": r["vocab"], "hidden_size": r["width"]}),
                                 embedding_prefix="embed.", layers=layers, run=run, final_norm=norm, final_norm_prefix="final_norm.",
                                 head=PartSpec("linear_head", {"vocab_size": r["vocab"], "hidden_size": r["width"], "tied_to": None}),
                                 head_prefix="head.")

        register_architecture("ToyMixedForCausalLM", ToyConfig)


RUN = [{"layer": 0}, {"layer": 1}, {"layer": 0}, {"layer": 1}, {"layer": 0, "cache_of": 0}]
CONFIG = {"architectures": ["ToyMixedForCausalLM"], "width": HIDDEN, "heads": HEADS, "kv_heads": KV, "head_dim": DIM, "inner": INTER,
          "vocab": VOCAB, "eps": 1e-5, "theta": 5000.0, "decay": DECAY, "max_len": 256, "run": RUN}


def make_weights(seed):
    g = torch.Generator().manual_seed(seed)
    w = {"embed.weight": 0.5 * torch.randn(VOCAB, HIDDEN, generator=g), "head.weight": 0.2 * torch.randn(VOCAB, HIDDEN, generator=g),
         "final_norm.weight": 1 + 0.1 * torch.randn(HIDDEN, generator=g)}
    for i in range(2):
        p = f"blocks.{i}."
        w[p + "norm1.weight"] = 1 + 0.1 * torch.randn(HIDDEN, generator=g)
        w[p + "norm2.weight"] = 1 + 0.1 * torch.randn(HIDDEN, generator=g)
        w[p + "ffn.gate_proj.weight"] = 0.15 * torch.randn(INTER, HIDDEN, generator=g)
        w[p + "ffn.up_proj.weight"] = 0.15 * torch.randn(INTER, HIDDEN, generator=g)
        w[p + "ffn.down_proj.weight"] = 0.15 * torch.randn(HIDDEN, INTER, generator=g)
    w["blocks.0.mixer.q_proj.weight"] = 0.15 * torch.randn(HEADS * DIM, HIDDEN, generator=g)
    w["blocks.0.mixer.k_proj.weight"] = 0.15 * torch.randn(KV * DIM, HIDDEN, generator=g)
    w["blocks.0.mixer.v_proj.weight"] = 0.3 * torch.randn(KV * DIM, HIDDEN, generator=g)
    w["blocks.0.mixer.o_proj.weight"] = 0.3 * torch.randn(HIDDEN, HEADS * DIM, generator=g)
    w["blocks.1.mixer.mix.weight"] = 0.3 * torch.randn(HIDDEN, HIDDEN, generator=g)
    return {k: v.to(torch.bfloat16).float() for k, v in w.items()}


def plain_forward(w, tokens):
    """The toy model on a whole sequence with the plain functions, following the run list."""
    w = {k: v.double() for k, v in w.items()}
    positions = torch.arange(len(tokens))
    x = pl.embed(w["embed.weight"], tokens)
    kept = {}
    for index, entry in enumerate(RUN):
        p = f"blocks.{entry['layer']}."
        h = pl.rms_norm(x, w[p + "norm1.weight"], 1e-5)
        if entry["layer"] == 0:
            q = pl.rotary((h @ w[p + "mixer.q_proj.weight"].T).reshape(-1, HEADS, DIM), positions, 5000.0)
            if "cache_of" in entry:
                k, v = kept[entry["cache_of"]]
            else:
                k = pl.rotary((h @ w[p + "mixer.k_proj.weight"].T).reshape(-1, KV, DIM), positions, 5000.0)
                v = (h @ w[p + "mixer.v_proj.weight"].T).reshape(-1, KV, DIM)
                kept[index] = (k, v)
            mixed = pl.causal_attention(q, k, v).reshape(-1, HEADS * DIM) @ w[p + "mixer.o_proj.weight"].T
        else:
            state = torch.zeros(HIDDEN, dtype=torch.float64)
            states = []
            for t in range(len(tokens)):
                state = DECAY * state + (1 - DECAY) * h[t]
                states.append(state)
            mixed = torch.stack(states) @ w[p + "mixer.mix.weight"].T
        x = x + mixed
        h = pl.rms_norm(x, w[p + "norm2.weight"], 1e-5)
        x = x + pl.swiglu_mlp(h, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"], w[p + "ffn.down_proj.weight"])
    return (pl.rms_norm(x, w["final_norm.weight"], 1e-5) @ w["head.weight"].T).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_a_stateful_mixer_steps_like_its_plain_form(dtype, tmp_path):
    from cisr_b200 import Model, Stepper

    register_toys()
    weights = make_weights(3)
    (tmp_path / "config.json").write_text(json.dumps(CONFIG))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(tmp_path / "model.safetensors"))
    model = Model.from_pretrained(tmp_path, dtype=dtype)
    uses = model.cache_uses()
    assert [u if isinstance(u, int) else u.kind for u in uses] == ["pages", "state", "pages", "state", 0]
    rng = np.random.default_rng(5)
    requests = {rid: [int(t) for t in rng.integers(0, VOCAB, n)] for rid, n in (("a", 60), ("b", 25), ("c", 41))}
    reference = {rid: plain_forward(weights, t) for rid, t in requests.items()}
    for steps in (replay.trace_whole(requests), replay.trace_portions(requests, (5, 2, 11, 1, 3)), replay.trace_mixed(requests, 2, max_live=3, decode_tail=8)):
        stepper = Stepper(model, n_pages=replay.max_live_tokens(steps) // 16, page_size=16, max_slots=3)
        cache = stepper.cache
        assert len(cache.page_groups) == 1 and cache.page_groups[0].entries == [0, 2] and cache.state_groups[0].entries == [1, 3]
        got = replay.run_steps(stepper, steps)
        replay.compare(got, requests, reference, dtype)
        assert cache.page_groups[0].pool.n_free == cache.page_groups[0].pool.n_pages
