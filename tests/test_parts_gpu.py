"""Each part of a layer alone, built through its registry, against the plain functions."""
import numpy as np
import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu
DEV = "cuda"


def part(registry_name, kind, params, dtype):
    from cisr_b200 import parts
    from cisr_b200.config import PartSpec
    return parts.build_part(getattr(parts, registry_name), PartSpec(kind, params), dtype, kind)


def close(a, b, atol, rtol):
    torch.testing.assert_close(a.double().cpu(), b.double().cpu(), atol=atol, rtol=rtol)


def close_for(dtype, a, b):
    """float32: element by element; bfloat16: relative RMS error of the whole result and no single wild element."""
    if dtype == torch.float32:
        return close(a, b, *TOL[dtype])
    a, b = a.double().cpu(), b.double().cpu()
    assert torch.isfinite(a).all()
    assert float(((a - b) ** 2).mean().sqrt() / (b ** 2).mean().sqrt()) < 0.02
    assert float((a - b).abs().max()) < 0.1 * float(b.abs().max())


TOL = {torch.float32: (3e-6, 2e-5), torch.bfloat16: (3e-2, 3e-2)}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rms_norm_part(dtype):
    norm = part("NORMS", "rms_norm", {"size": 100, "eps": 2e-6}, dtype)
    assert norm.tensor_needs()["weight"].shape == (100,) and norm.tensor_needs()["weight"].role == "vector"
    g = torch.Generator().manual_seed(0)
    w, x, d = 1 + 0.1 * torch.randn(100, generator=g), torch.randn(6, 100, generator=g), torch.randn(6, 100, generator=g)
    norm.load({"weight": w.to(DEV)})                     # a 32-bit vector stays 32-bit in either mode
    xd = x.to(DEV)
    out = norm.forward(xd, d.to(DEV), dtype)
    assert out.dtype == dtype
    close(xd, x + d, 1e-6, 1e-6)
    close(out, pl.rms_norm((x + d).double(), w.double(), 2e-6), 3e-6 if dtype == torch.float32 else 0, 3e-6 if dtype == torch.float32 else 2 ** -8)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_embedding_and_head_parts(dtype):
    g = torch.Generator().manual_seed(1)
    ffn = part("FEED_FORWARDS", "swiglu", {"hidden_size": 70, "intermediate_size": 150}, dtype)
    assert set(ffn.tensor_needs()) == {"gate_proj.weight", "up_proj.weight", "down_proj.weight"}
    ws = {n: (0.2 * torch.randn(*need.shape, generator=g)).to(dtype) for n, need in ffn.tensor_needs().items()}
    ffn.load({n: w.to(DEV) for n, w in ws.items()})
    h = torch.randn(9, 70, generator=g).to(dtype)
    out = ffn.forward(h.to(DEV), None)
    ref = pl.swiglu_mlp(h.double(), ws["gate_proj.weight"].double(), ws["up_proj.weight"].double(), ws["down_proj.weight"].double())
    assert out.dtype == torch.float32
    close_for(dtype, out, ref)

    emb = part("EMBEDDINGS", "token_embedding", {"vocab_size": 300, "hidden_size": 70}, dtype)
    table = torch.randn(300, 70, generator=g).to(dtype)
    emb.load({"weight": table.to(DEV)})
    ids = torch.tensor([3, 299, 0], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ids).cpu(), table[[3, 299, 0]].float())
    head = part("HEADS", "linear_head", {"vocab_size": 300, "hidden_size": 70, "tied_to": "model.embed_tokens.weight"}, dtype)
    assert head.tensor_needs()["weight"].alias == "model.embed_tokens.weight"
    head.load({"weight": table.to(DEV)})
    close(head.forward(h.to(DEV)), h.double() @ table.double().T, 1e-4 if dtype == torch.float32 else 0.15, 1e-5 if dtype == torch.float32 else 2e-2)


class MiniStep:
    """A cache manager and step contexts for one mixer, without a model."""

    def __init__(self, mixer, n_pages, page_size, dtype):
        from cisr_b200.cache import CacheManager
        from cisr_b200.engine.batch import PinnedRing
        self.cache = CacheManager([mixer.cache_use()], n_pages, page_size, 4, 512, dtype=dtype, device=torch.device(DEV))
        self.ring = PinnedRing()

    def run(self, fn, entries):
        from cisr_b200 import StepEntry
        from cisr_b200.engine.step import commit_step, prepare_step
        entries = [StepEntry(k, [0] * n) for k, n in entries]
        ctx, _, _ = prepare_step(self.cache, self.ring, torch.device(DEV), entries, 1)
        out = fn(ctx, self.cache.binding(0))
        commit_step(self.cache, entries)
        return out


def test_rotary_part_matches_plain_and_is_computed_once_per_step():
    rot = part("POSITIONS", "rotary_half", {"theta": 500000.0, "dim": 32}, torch.float32)
    mixer = part("MIXERS", "gqa_attention", {"hidden_size": 64, "num_heads": 2, "num_kv_heads": 1, "head_dim": 32, "window": None,
                                              "position": rot.spec}, torch.float32)
    mini = MiniStep(mixer, 8, 16, torch.float32)
    mini.cache.create("a"); mini.cache.create("b")
    mini.run(lambda ctx, cache: None, [("a", 37)])

    def check(ctx, cache):
        r1 = rot.rotation(ctx)
        assert rot.rotation(ctx) is r1 and r1.rot_half == 16 and not r1.interleaved
        positions = torch.tensor(list(range(37, 40)) + list(range(5)))
        x = torch.randn(8, 2, 32, dtype=torch.float64)
        ref = pl.rotary(x, positions, 500000.0)
        c, s = r1.cos.double().cpu()[:, None], r1.sin.double().cpu()[:, None]
        ours = torch.cat((x[..., :16] * c - x[..., 16:] * s, x[..., 16:] * c + x[..., :16] * s), dim=-1)
        close(ours, ref, 1e-6, 0)
    mini.run(check, [("a", 3), ("b", 5)])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 24])
def test_attention_part_over_portions(dtype, window):
    """The mixer alone: a sequence fed in portions (with another request beside it) equals the plain block on the whole."""
    from cisr_b200.config import PartSpec
    hidden, hq, hkv, d, theta = 96, 6, 2, 32, 10000.0
    mixer = part("MIXERS", "gqa_attention", {"hidden_size": hidden, "num_heads": hq, "num_kv_heads": hkv, "head_dim": d, "window": window,
                                              "position": PartSpec("rotary_half", {"theta": theta, "dim": d})}, dtype)
    use = mixer.cache_use()
    assert (use.kind, use.kv_heads, use.head_dim, use.window) == ("pages", hkv, d, window)
    g = torch.Generator().manual_seed(4)
    ws = {n: (0.15 * torch.randn(*need.shape, generator=g)).to(dtype) for n, need in mixer.tensor_needs().items()}
    mixer.load({n: w.to(DEV) for n, w in ws.items()})
    total = 90
    h = {k: torch.randn(total, hidden, generator=g).to(dtype) for k in ("a", "b")}
    cfg = {"num_attention_heads": hq, "num_key_value_heads": hkv, "head_dim": d, "hidden_size": hidden, "rope_theta": theta}
    mini = MiniStep(mixer, 32, 8, dtype)
    mini.cache.create("a"); mini.cache.create("b")
    got = {"a": [], "b": []}
    at = {"a": 0, "b": 0}
    for na, nb in ((40, 1), (1, 1), (7, 30), (2, 1), (40, 57)):
        both = torch.cat((h["a"][at["a"]:at["a"] + na], h["b"][at["b"]:at["b"] + nb])).to(DEV)
        out = mini.run(lambda ctx, cache: mixer.forward(both, ctx, cache), [("a", na), ("b", nb)])
        got["a"].append(out[:na].cpu()); got["b"].append(out[na:].cpu())
        at["a"] += na; at["b"] += nb
    for k in ("a", "b"):
        weights = {"L.self_attn." + n: w.double() for n, w in ws.items()}
        ref = pl.attention_block(h[k].double(), weights, "L.", torch.arange(total), cfg, window)
        close_for(dtype, torch.cat(got[k]), ref)
    if window is not None:
        assert mini.cache.page_groups[0].pool.n_used <= 2 * (-(-window // 8) + 1)     # passed pages came back


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pre_norm_block_arrangement(dtype):
    """The arrangement alone: its output pending + x equals the plain decoder layer."""
    from cisr_b200.config import LayerSpec, PartSpec
    from cisr_b200.parts import ARRANGEMENTS, ResidualStream
    hidden, hq, hkv, d, inter = 64, 4, 4, 16, 100
    norm = PartSpec("rms_norm", {"size": hidden, "eps": 1e-5})
    spec = LayerSpec(prefix="model.layers.0.", mixer_norm=norm, feed_forward_norm=norm,
                     mixer=PartSpec("gqa_attention", {"hidden_size": hidden, "num_heads": hq, "num_kv_heads": hkv, "head_dim": d, "window": None,
                                                      "position": PartSpec("rotary_half", {"theta": 10000.0, "dim": d})}),
                     feed_forward=PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": inter}),
                     names={"mixer": "self_attn.", "mixer_norm": "input_layernorm.", "feed_forward": "mlp.", "feed_forward_norm": "post_attention_layernorm."})
    block = ARRANGEMENTS["pre_norm"](spec, dtype)
    g = torch.Generator().manual_seed(9)
    weights = {}
    for slot, p in block.parts().items():
        local = {}
        for n, need in p.tensor_needs().items():
            w = (1 + 0.1 * torch.randn(*need.shape, generator=g)) if need.role == "vector" else (0.15 * torch.randn(*need.shape, generator=g)).to(dtype).float()
            local[n] = w.to(DEV) if need.role == "vector" else w.to(dtype).to(DEV)
            weights[spec.prefix + spec.names[slot] + n] = w.double()
        p.load(local)
    x = torch.randn(21, hidden, generator=g)
    pending = torch.randn(21, hidden, generator=g)
    mini = MiniStep(block.mixer, 8, 16, dtype)
    mini.cache.create("a")
    stream = ResidualStream(x.to(DEV).clone())
    stream.pending = pending.to(DEV)
    mini.run(lambda ctx, cache: block.forward(stream, ctx, cache), [("a", 21)])
    cfg = {"num_attention_heads": hq, "num_key_value_heads": hkv, "head_dim": d, "hidden_size": hidden, "rope_theta": 10000.0, "rms_norm_eps": 1e-5}
    ref = pl.decoder_layer((x + pending).double(), weights, 0, torch.arange(21), cfg)
    close_for(dtype, stream.x + stream.pending, ref)


def test_unknown_parts_are_named_in_the_error():
    from cisr_b200 import parts
    from cisr_b200.config import PartSpec
    with pytest.raises(KeyError, match="no mixer registered as 'hyena'.*gqa_attention"):
        parts.build_part(parts.MIXERS, PartSpec("hyena", {}), torch.float32, "mixer")
    with pytest.raises(ValueError, match="head_dim 40"):
        part("MIXERS", "gqa_attention", {"hidden_size": 80, "num_heads": 2, "num_kv_heads": 1, "head_dim": 40, "window": None,
                                          "position": PartSpec("none", {})}, torch.float32)
