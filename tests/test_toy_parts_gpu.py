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


# ---------------------------------------------------------------------------------------------------------------
# A second toy architecture: a feed-forward that routes each token to two of three small experts, a position
# encoding that turns only the first pairs of each head, interleaved and with frequencies of its own, a norm with a
# mean and a bias, and an arrangement in which mixer and feed-forward read the same normed input.
# ---------------------------------------------------------------------------------------------------------------
R_WIDTH, R_HEADS, R_KV, R_DIM, R_PAIRS, R_BASE, R_EXPERTS, R_TOP, R_INNER, R_VOCAB, R_EPS = 40, 2, 2, 32, 6, 90.0, 3, 2, 24, 61, 1e-4
MARGIN = 0.12          # the least gap between the last chosen and the first unchosen router logit that the seed must give


def register_routed_toys():
    from cisr_b200.config import ARCHITECTURES, LayerSpec, ModelSpec, PartSpec, RunEntry, register_architecture
    from cisr_b200.parts import (ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, FeedForward, Norm, PositionEncoding,
                                 Rotation, TensorNeed, build_part, register)

    if "toy_top_k_experts" not in FEED_FORWARDS:
        @register(FEED_FORWARDS, "toy_top_k_experts")
        class ToyExperts(FeedForward):
            """Router logits in 32-bit; the top k experts' weights are a softmax over their logits; expert: W2 relu(W1 h)."""

            def __init__(self, spec, dtype):
                super().__init__(spec, dtype)
                self.hidden, self.inner, self.n, self.k = (int(spec[key]) for key in ("hidden_size", "inner", "experts", "top"))

            def tensor_needs(self):
                return {"router.weight": TensorNeed((self.n, self.hidden)), "w1": TensorNeed((self.n, self.inner, self.hidden)),
                        "w2": TensorNeed((self.n, self.hidden, self.inner))}

            def load(self, tensors):
                self.router, self.w1, self.w2 = tensors["router.weight"], tensors["w1"], tensors["w2"]

            def forward(self, h, ctx):
                logits = h.float() @ self.router.float().T
                top, chosen = torch.topk(logits, self.k, dim=-1)
                gates = torch.zeros_like(logits).scatter_(1, chosen, torch.softmax(top, dim=-1))
                out = torch.zeros((h.shape[0], self.hidden), dtype=torch.float32, device=h.device)
                for e in range(self.n):
                    rows = torch.nonzero(gates[:, e] > 0).flatten()          # only the tokens routed here run the expert
                    if rows.numel():
                        inner = torch.relu(h[rows].float() @ self.w1[e].float().T).to(self.dtype).float()
                        out[rows] += gates[rows, e, None] * (inner @ self.w2[e].float().T)
                return out

    if "toy_interleaved_pairs" not in POSITIONS:
        @register(POSITIONS, "toy_interleaved_pairs")
        class ToyPairs(PositionEncoding):
            """Pairs (2i, 2i + 1), i < pairs, turn by pos * base^(-(i + 1) / pairs); the rest of the head is left alone."""

            def __init__(self, spec, dtype):
                super().__init__(spec, dtype)
                self.pairs, self.base = int(spec["pairs"]), float(spec["base"])

            def rotation(self, ctx):
                key = ("toy_pairs", self.pairs, self.base)
                if key not in ctx.shared:
                    freq = self.base ** (-(torch.arange(self.pairs, dtype=torch.float64, device=ctx.device) + 1) / self.pairs)
                    angle = ctx.positions.double()[:, None] * freq[None, :]
                    ctx.shared[key] = Rotation(torch.cos(angle).float().contiguous(), torch.sin(angle).float().contiguous(),
                                               self.pairs, True)
                return ctx.shared[key]

    if "toy_layer_norm" not in NORMS:
        @register(NORMS, "toy_layer_norm")
        class ToyLayerNorm(Norm):
            """(x - mean) / sqrt(var + eps) * weight + bias; not of the form the products' prologue computes."""

            def __init__(self, spec, dtype):
                super().__init__(spec, dtype)
                self.size, self.eps = int(spec["size"]), float(spec["eps"])

            def tensor_needs(self):
                return {"weight": TensorNeed((self.size,), role="vector"), "bias": TensorNeed((self.size,), role="vector")}

            def load(self, tensors):
                self.weight, self.bias = tensors["weight"], tensors["bias"]

            def forward(self, x, delta, out_dtype, rows=None, write_back=True):
                if delta is not None and write_back:
                    x += delta
                    delta = None
                picked = x if rows is None else x[rows.long()]
                if delta is not None:
                    picked = picked + (delta if rows is None else delta[rows.long()])
                mean = picked.mean(-1, keepdim=True)
                var = ((picked - mean) ** 2).mean(-1, keepdim=True)
                return ((picked - mean) * torch.rsqrt(var + self.eps) * self.weight.float() + self.bias.float()).to(out_dtype)

    if "toy_parallel" not in ARRANGEMENTS:
        @register(ARRANGEMENTS, "toy_parallel")
        class ToyParallel:
            """x += mixer(norm(x)) + feed_forward(norm(x)): one norm, read by both."""
            slots = ("mixer_norm", "mixer", "feed_forward")

            def __init__(self, spec, dtype):
                self.dtype = dtype
                self.mixer_norm = build_part(NORMS, spec.mixer_norm, dtype, "norm")
                self.mixer = build_part(MIXERS, spec.mixer, dtype, "mixer")
                self.feed_forward = build_part(FEED_FORWARDS, spec.feed_forward, dtype, "feed-forward")

            def parts(self):
                return {slot: getattr(self, slot) for slot in self.slots}

            def forward(self, stream, ctx, cache):
                h = self.mixer_norm.forward(stream.x, stream.take_pending(), self.dtype)
                stream.pending = self.mixer.forward(h, ctx, cache) + self.feed_forward.forward(h, ctx)

    if "ToyRoutedForCausalLM" not in ARCHITECTURES:
        class ToyRoutedConfig:
            def __init__(self, raw):
                self.raw = raw

            @classmethod
            def from_dict(cls, raw):
                return cls(dict(raw))

            def to_dict(self):
                return dict(self.raw)

            def to_spec(self):
                r = self.raw
                norm = PartSpec("toy_layer_norm", {"size": r["width"], "eps": r["eps"]})
                attention = PartSpec("gqa_attention", {"hidden_size": r["width"], "num_heads": r["heads"], "num_kv_heads": r["kv_heads"],
                                                       "head_dim": r["head_dim"], "window": r["window"],
                                                       "position": PartSpec("toy_interleaved_pairs", {"pairs": r["pairs"], "base": r["base"]})})
                ffn = PartSpec("toy_top_k_experts", {"hidden_size": r["width"], "inner": r["inner"], "experts": r["experts"], "top": r["top"]})
                names = {"mixer": "attn.", "mixer_norm": "ln1.", "feed_forward": "moe.", "feed_forward_norm": "ln2."}
                layers = tuple(LayerSpec(prefix=f"h.{i}.", mixer=attention, mixer_norm=norm, feed_forward=ffn, feed_forward_norm=norm,
                                         arrangement=a, names=names) for i, a in enumerate(r["arrangements"]))
                return ModelSpec(hidden_size=r["width"], vocab_size=r["vocab"], max_positions=r["max_len"],
                                 embedding=PartSpec("token_embedding", {"vocab_size": r["vocab"], "hidden_size": r["width"]}),
                                 embedding_prefix="wte.", layers=layers, run=tuple(RunEntry(layer=i) for i in range(len(layers))),
                                 final_norm=norm, final_norm_prefix="ln_f.",
                                 head=PartSpec("linear_head", {"vocab_size": r["vocab"], "hidden_size": r["width"], "tied_to": "wte.weight"}),
                                 head_prefix="lm_head.")

        register_architecture("ToyRoutedForCausalLM", ToyRoutedConfig)


ROUTED_ARRANGEMENTS = ["pre_norm", "toy_parallel"]
ROUTED_CONFIG = {"architectures": ["ToyRoutedForCausalLM"], "width": R_WIDTH, "heads": R_HEADS, "kv_heads": R_KV, "head_dim": R_DIM,
                 "pairs": R_PAIRS, "base": R_BASE, "experts": R_EXPERTS, "top": R_TOP, "inner": R_INNER, "vocab": R_VOCAB, "eps": R_EPS,
                 "window": 12, "max_len": 128, "arrangements": ROUTED_ARRANGEMENTS}


def make_routed_weights(seed):
    g = torch.Generator().manual_seed(seed)
    w = {"wte.weight": 0.6 * torch.randn(R_VOCAB, R_WIDTH, generator=g),
         "ln_f.weight": 1 + 0.1 * torch.randn(R_WIDTH, generator=g), "ln_f.bias": 0.1 * torch.randn(R_WIDTH, generator=g)}
    for i, arrangement in enumerate(ROUTED_ARRANGEMENTS):
        p = f"h.{i}."
        for ln in ("ln1.",) if arrangement == "toy_parallel" else ("ln1.", "ln2."):
            w[p + ln + "weight"] = 1 + 0.1 * torch.randn(R_WIDTH, generator=g)
            w[p + ln + "bias"] = 0.1 * torch.randn(R_WIDTH, generator=g)
        w[p + "attn.q_proj.weight"] = 0.2 * torch.randn(R_HEADS * R_DIM, R_WIDTH, generator=g)
        w[p + "attn.k_proj.weight"] = 0.2 * torch.randn(R_KV * R_DIM, R_WIDTH, generator=g)
        w[p + "attn.v_proj.weight"] = 0.3 * torch.randn(R_KV * R_DIM, R_WIDTH, generator=g)
        w[p + "attn.o_proj.weight"] = 0.2 * torch.randn(R_WIDTH, R_HEADS * R_DIM, generator=g)
        w[p + "moe.router.weight"] = 0.6 * torch.randn(R_EXPERTS, R_WIDTH, generator=g)
        w[p + "moe.w1"] = 0.25 * torch.randn(R_EXPERTS, R_INNER, R_WIDTH, generator=g)
        w[p + "moe.w2"] = 0.25 * torch.randn(R_EXPERTS, R_WIDTH, R_INNER, generator=g)
    return {k: v.to(torch.bfloat16).float() for k, v in w.items()}


def routed_plain_forward(w, tokens):
    """The routed toy model on a whole sequence in float64; also the least routing margin it met."""
    w = {k: v.double() for k, v in w.items()}
    n = len(tokens)
    positions = torch.arange(n, dtype=torch.float64)
    freq = R_BASE ** (-(torch.arange(R_PAIRS, dtype=torch.float64) + 1) / R_PAIRS)
    cos, sin = torch.cos(positions[:, None] * freq)[:, None, :], torch.sin(positions[:, None] * freq)[:, None, :]
    margin = [float("inf")]

    def layer_norm(x, p):
        mean = x.mean(-1, keepdim=True)
        var = ((x - mean) ** 2).mean(-1, keepdim=True)
        return (x - mean) / torch.sqrt(var + R_EPS) * w[p + "weight"] + w[p + "bias"]

    def turn(x):
        out = x.clone()
        even, odd = x[..., 0:2 * R_PAIRS:2], x[..., 1:2 * R_PAIRS:2]
        out[..., 0:2 * R_PAIRS:2] = even * cos - odd * sin
        out[..., 1:2 * R_PAIRS:2] = odd * cos + even * sin
        return out

    def attention(h, p):
        q = turn((h @ w[p + "q_proj.weight"].T).reshape(n, R_HEADS, R_DIM))
        k = turn((h @ w[p + "k_proj.weight"].T).reshape(n, R_KV, R_DIM))
        v = (h @ w[p + "v_proj.weight"].T).reshape(n, R_KV, R_DIM)
        return pl.causal_attention(q, k, v, window=ROUTED_CONFIG["window"]).reshape(n, R_HEADS * R_DIM) @ w[p + "o_proj.weight"].T

    def experts(h, p):
        logits = h @ w[p + "router.weight"].T
        ordered = torch.sort(logits, dim=-1, descending=True).values
        margin[0] = min(margin[0], float((ordered[:, R_TOP - 1] - ordered[:, R_TOP]).min()))
        top, chosen = torch.topk(logits, R_TOP, dim=-1)
        gates = torch.softmax(top, dim=-1)
        out = torch.zeros(n, R_WIDTH, dtype=torch.float64)
        for t in range(n):
            for j in range(R_TOP):
                e = int(chosen[t, j])
                out[t] += gates[t, j] * (w[p + "w2"][e] @ torch.relu(w[p + "w1"][e] @ h[t]))
        return out

    x = pl.embed(w["wte.weight"], tokens)
    for i, arrangement in enumerate(ROUTED_ARRANGEMENTS):
        p = f"h.{i}."
        h = layer_norm(x, p + "ln1.")
        if arrangement == "toy_parallel":
            x = x + attention(h, p + "attn.") + experts(h, p + "moe.")
        else:
            x = x + attention(h, p + "attn.")
            x = x + experts(layer_norm(x, p + "ln2."), p + "moe.")
    return (layer_norm(x, "ln_f.") @ w["wte.weight"].T).numpy(), margin[0]


ROUTED_SEED, ROUTED_TOKENS_SEED = 11, 6


def routed_requests():
    rng = np.random.default_rng(ROUTED_TOKENS_SEED)
    return {rid: [int(t) for t in rng.integers(0, R_VOCAB, n)] for rid, n in (("a", 37), ("b", 11), ("c", 20))}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_experts_position_norm_and_arrangement(dtype, tmp_path):
    from cisr_b200 import Model, Stepper

    register_routed_toys()
    weights = make_routed_weights(ROUTED_SEED)
    (tmp_path / "config.json").write_text(json.dumps(ROUTED_CONFIG))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(tmp_path / "model.safetensors"))
    model = Model.from_pretrained(tmp_path, dtype=dtype)
    assert "h.1.ln2.weight" not in model.tensor_needs() and "h.0.ln2.bias" in model.tensor_needs()
    requests = routed_requests()
    reference = {}
    for rid, tokens in requests.items():
        reference[rid], margin = routed_plain_forward(weights, tokens)
        # a choice of experts that hangs on a hair would differ between precisions and say nothing about the engine
        assert margin > MARGIN, f"the seeds give a routing margin of {margin:.4f}; pick others"
    for steps in (replay.trace_whole(requests), replay.trace_portions(requests, (7, 2, 4, 1, 9)), replay.trace_mixed(requests, 3, max_live=3, decode_tail=6)):
        stepper = Stepper(model, n_pages=replay.max_live_tokens(steps) // 16, page_size=16, max_slots=3)
        got = replay.run_steps(stepper, steps)
        replay.compare(got, requests, reference, dtype)
        pool = stepper.cache.page_groups[0].pool
        assert pool.n_free == pool.n_pages


# ---------------------------------------------------------------------------------------------------------------
# A toy architecture of the engine's own parts whose second layer attends to a window of keys: its pages have a pool
# of their own and go back to it as the window passes them, also while decode steps come from captured graphs (the
# block-table entries of the passed pages are cleared by the update kernel at the head of the captured step).
W_WINDOW, W_LAYERS = 40, 2
W_CFG = {"hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 112,
         "vocab_size": 131, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "num_hidden_layers": W_LAYERS, "tie_word_embeddings": True}
W_CONFIG = dict(W_CFG, architectures=["ToyWindowedForCausalLM"], window=W_WINDOW, max_len=512)


def register_windowed_toy():
    from cisr_b200.config import ARCHITECTURES, LayerSpec, ModelSpec, PartSpec, RunEntry, register_architecture

    if "ToyWindowedForCausalLM" in ARCHITECTURES:
        return

    class WindowedConfig:
        def __init__(self, raw):
            self.raw = raw

        @classmethod
        def from_dict(cls, raw):
            return cls(dict(raw))

        def to_dict(self):
            return dict(self.raw)

        def to_spec(self):
            r = self.raw
            norm = PartSpec("rms_norm", {"size": r["hidden_size"], "eps": r["rms_norm_eps"]})
            def attention(window):
                return PartSpec("gqa_attention", {"hidden_size": r["hidden_size"], "num_heads": r["num_attention_heads"],
                                                  "num_kv_heads": r["num_key_value_heads"], "head_dim": r["head_dim"], "window": window,
                                                  "scale": r["head_dim"] ** -0.5,
                                                  "position": PartSpec("rotary_half", {"theta": r["rope_theta"], "dim": r["head_dim"]})})
            ffn = PartSpec("swiglu", {"hidden_size": r["hidden_size"], "intermediate_size": r["intermediate_size"]})
            names = {"mixer": "self_attn.", "mixer_norm": "input_layernorm.", "feed_forward": "mlp.", "feed_forward_norm": "post_attention_layernorm."}
            layers = tuple(LayerSpec(prefix=f"model.layers.{i}.", mixer=attention(None if i == 0 else r["window"]), mixer_norm=norm,
                                     feed_forward=ffn, feed_forward_norm=norm, names=names) for i in range(r["num_hidden_layers"]))
            return ModelSpec(hidden_size=r["hidden_size"], vocab_size=r["vocab_size"], max_positions=r["max_len"],
                             embedding=PartSpec("token_embedding", {"vocab_size": r["vocab_size"], "hidden_size": r["hidden_size"]}),
                             embedding_prefix="model.embed_tokens.", layers=layers, run=tuple(RunEntry(layer=i) for i in range(len(layers))),
                             final_norm=norm, final_norm_prefix="model.norm.",
                             head=PartSpec("linear_head", {"vocab_size": r["vocab_size"], "hidden_size": r["hidden_size"],
                                                           "tied_to": "model.embed_tokens.weight"}), head_prefix="lm_head.")

    register_architecture("ToyWindowedForCausalLM", WindowedConfig)


def windowed_plain_forward(weights, tokens):
    """plain_llama's layer with the window handed to the second layer's attention."""
    w = {k: v.double() for k, v in weights.items()}
    positions = torch.arange(len(tokens))
    x = pl.embed(w["model.embed_tokens.weight"], tokens)
    for layer in range(W_LAYERS):
        p = f"model.layers.{layer}."
        h = pl.rms_norm(x, w[p + "input_layernorm.weight"], W_CFG["rms_norm_eps"])
        x = x + pl.attention_block(h, w, p, positions, W_CFG, window=None if layer == 0 else W_WINDOW)
        h = pl.rms_norm(x, w[p + "post_attention_layernorm.weight"], W_CFG["rms_norm_eps"])
        x = x + pl.swiglu_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return pl.rms_norm(x, w["model.norm.weight"], W_CFG["rms_norm_eps"]) @ w["model.embed_tokens.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_window_group_inside_captured_decode_steps(dtype, tmp_path):
    import tiny_models as tm
    from cisr_b200 import Model, StepEntry, Stepper

    register_windowed_toy()
    weights = {k: torch.from_numpy(v) if isinstance(v, np.ndarray) else v for k, v in tm.make_weights(W_CFG, 77, scale=0.08, bf16_exact=True).items()}
    (tmp_path / "config.json").write_text(json.dumps(W_CONFIG))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(tmp_path / "model.safetensors"))
    model = Model.from_pretrained(tmp_path, dtype=dtype)
    rng = np.random.default_rng(5)
    requests = {rid: [int(t) for t in rng.integers(0, W_CFG["vocab_size"], n)] for rid, n in (("a", 150), ("b", 97), ("c", 61))}
    reference = {rid: windowed_plain_forward(weights, tokens).numpy() for rid, tokens in requests.items()}
    page = 8
    stepper = Stepper(model, n_pages=64, page_size=page, max_slots=4, graph=True)
    groups = stepper.cache.page_groups
    assert len(groups) == 2 and sorted(g.use.window or 0 for g in groups) == [0, W_WINDOW]
    windowed = next(g for g in groups if g.use.window)
    got = {}
    prompt = {"a": 30, "b": 20, "c": 9}                       # the rest of each request is decoded, one token per step, from graphs
    for rid, tokens in requests.items():
        stepper.create(rid)
        logits = stepper.step([StepEntry(rid, tokens[:prompt[rid]], list(range(prompt[rid])))]).cpu().numpy()
        for i in range(prompt[rid]):
            got[(rid, i)] = logits[i]
    longest = max(len(t) for t in requests.values())
    for at in range(longest):
        entries = [StepEntry(rid, [tokens[prompt[rid] + at]], [0]) for rid, tokens in requests.items() if prompt[rid] + at < len(tokens)]
        if not entries:
            break
        logits = stepper.step(entries).cpu().numpy()
        for row, e in enumerate(entries):
            got[(e.key, prompt[e.key] + at)] = logits[row]
        # the windowed layer never holds more pages per request than its window spans
        assert windowed.pool.n_used <= len(entries) * (-(-W_WINDOW // page) + 1) + (len(requests) - len(entries)) * (-(-W_WINDOW // page) + 1)
    assert stepper.graphs.report()["hits"] > 50
    replay.compare(got, requests, reference, dtype)
    for rid in requests:
        stepper.release(rid)
    assert all(g.pool.n_free == g.pool.n_pages for g in groups)
