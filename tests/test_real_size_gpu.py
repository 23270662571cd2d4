"""The engine at real layer sizes against the plain implementation, under every way of cutting the work.

The tiny configurations never reach the kernels that only real sizes select: the persistent weight-streaming
product (matrices of 8 MB and more: the 49,152-row head at the SmolLM2-135M sizes, every product at the
Llama-3.1-8B sizes, with its 3-D and 4-D tensor maps for the gated and the rotating epilogue), 128 x 256 tiles
of the tcgen05 product, K = 576 (nine 64-wide blocks), thirty layers of accumulated rounding, the tcgen05
attention at head size 128, and decode graphs whose context crosses a bucket.  Here they run inside the engine
and their logits are compared with plain_llama in float64 on the same bfloat16-exact weights.  Parity: the
reference's tests/test_model.py:8-26 (paged token-by-token equals the dense whole sequence) and
tests/test_execution.py:14-40, at size.

Bounds.  float32: those of tests/replay.py.  bfloat16: at thirty layers the rounding of values stored in bfloat16
(six per layer) is itself as large as the 0.03 that tests/replay.py allows a row: plain_llama with bfloat16 storage
and float64 arithmetic (no engine involved) is 0.017 (median) to 0.033 (worst row) away from its exact self at these
sizes, and the engine measures the same, 0.017 to 0.033, under every way of cutting, because its rounding noise is
that noise.  So a bfloat16 row is held to the reference's own bound for bfloat16 logits, 0.04
(tests/test_precision.py:27-28), and the engine's median error over all rows must not exceed the median error of
that plain bfloat16-storage twin by more than a quarter: a loss of precision anywhere in the engine would lift it.
"""
import gc

import numpy as np
import pytest
import torch

import replay
import tiny_models as tm

pytestmark = pytest.mark.gpu

# The SmolLM2-135M sizes, all thirty layers (config/presets/smollm2-135m.json; the context limit cut to what the test uses).
SMOLLM2_135M = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu", "vocab_size": 49152, "hidden_size": 576,
    "intermediate_size": 1536, "num_hidden_layers": 30, "num_attention_heads": 9, "num_key_value_heads": 3, "head_dim": 64,
    "rms_norm_eps": 1e-5, "rope_theta": 100000.0, "max_position_embeddings": 1024, "tie_word_embeddings": True,
}
# Two layers with the Llama-3.1-8B layer geometry; the vocabulary is cut to 4096 so that the plain side stays small.
LLAMA_8B_LAYERS = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu", "vocab_size": 4096, "hidden_size": 4096,
    "intermediate_size": 14336, "num_hidden_layers": 2, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 1024, "tie_word_embeddings": False,
}
# name -> configuration, seed, scale of the matrices (about one over the root of the width), request lengths.
# The longest request's last 32 tokens start below 256 and end above it, so its decode graph changes context bucket.
# The short requests come first, so that in the mixed trace (four live at a time) the long ones start in pages that
# the short ones have given back.
CASES = {
    "smollm2_135m": (SMOLLM2_135M, 61, 0.04, {"d": 33, "f": 20, "e": 47, "c": 70, "g": 64, "h": 100, "b": 129, "a": 280}),
    "llama_8b_layers": (LLAMA_8B_LAYERS, 62, 0.015, {"d": 20, "e": 33, "c": 40, "f": 64, "b": 70, "g": 90, "a": 270}),
}
RRMS16_AT_DEPTH = 0.04         # the reference's own bound for bfloat16 logits (tests/test_precision.py:27-28)
MEDIAN_OVER_TWIN = 1.25        # engine median error / plain bfloat16-storage twin's median error, at most
_made = {}


def case(name, tmp_path_factory):
    """Weights, model folder, requests and float64 plain logits of a case, made once."""
    if name not in _made:
        _made.clear()                      # one case's weights at a time
        gc.collect()
        cfg, seed, scale, lengths = CASES[name]
        weights = tm.make_weights(cfg, seed, scale=scale, bf16_exact=True)
        path = tm.write_model_dir(tmp_path_factory.mktemp(name), cfg, weights, store_dtype=torch.bfloat16)
        requests = {rid: tm.random_tokens(cfg, n, 500 + i) for i, (rid, n) in enumerate(lengths.items())}
        reference = {rid: replay.plain_logits(cfg, weights, tokens) for rid, tokens in requests.items()}
        # what bfloat16 storage alone does to this model: the plain twin's error against its exact self, row by row
        twin_errors = []
        for rid, tokens in requests.items():
            twin = replay.plain_logits(cfg, weights, tokens, storage=torch.bfloat16)
            twin_errors += [replay.relative_rms(twin[pos], reference[rid][pos]) for pos in range(len(tokens))]
        _made[name] = (cfg, path, requests, reference, {}, float(np.median(twin_errors)))
    return _made[name]


def model_for(name, dtype, tmp_path_factory):
    from cisr_b200 import Model

    cfg, path, requests, reference, models, twin_median = case(name, tmp_path_factory)
    if dtype not in models:
        models.clear()
        gc.collect(); torch.cuda.empty_cache()
        models[dtype] = Model.from_pretrained(path, dtype=dtype)
    return cfg, models[dtype], requests, reference, twin_median


def traces(requests):
    return {"whole": replay.trace_whole(requests), "tail": replay.trace_tail_decode(requests, 32),
            "portions": replay.trace_portions(requests, (7, 2, 13, 5, 2, 31, 64, 3)),
            "mixed": replay.trace_mixed(requests, seed=5, max_live=4)}


def test_a_wrong_page_would_show(tmp_path_factory):
    """The comparison above can fail: the same run with one block-table entry of one request pointing at another
    request's page gives logits outside the bound."""
    from cisr_b200 import StepEntry, Stepper

    cfg, model, requests, reference, _ = model_for("smollm2_135m", "float32", tmp_path_factory)
    stepper = Stepper(model, n_pages=32, page_size=16, max_slots=2)
    a, c = requests["c"], requests["d"]
    assert len(a) >= 48 and len(c) >= 30
    stepper.create("x"); stepper.create("y")
    stepper.step([StepEntry("x", a[:40], []), StepEntry("y", c[:30], [])])
    group = stepper.cache.page_groups[0]
    tx, ty = stepper.cache.requests["x"].tables[0], stepper.cache.requests["y"].tables[0]
    group.set_entry(stepper.cache.requests["x"].slot, 1, ty[0])          # x's second page now reads y's first
    logits = stepper.step([StepEntry("x", a[40:48], list(range(8)))]).cpu().numpy()
    with pytest.raises(AssertionError):
        replay.compare({("c", 40 + j): logits[j] for j in range(8)}, None, reference, "float32")
    group.set_entry(stepper.cache.requests["x"].slot, 1, tx[1])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CASES))
def test_real_size_logits_under_every_cut(name, dtype, tmp_path_factory):
    from cisr_b200 import Stepper
    from cisr_b200.ops import kernels

    cfg, model, requests, reference, twin_median = model_for(name, dtype, tmp_path_factory)
    total = sum(len(t) for t in requests.values())
    before = dict(kernels.LAUNCHES)
    for mode, steps in traces(requests).items():
        for graph in (False, True):
            if graph and mode in ("whole", "portions"):
                continue                                  # no single-token steps in these: nothing would run from a graph
            pages = replay.max_live_tokens(steps) // 16
            stepper = Stepper(model, n_pages=pages, page_size=16, max_slots=4, graph=graph)
            got = replay.run_steps(stepper, steps)
            assert len(got) == total, (mode, graph)
            try:
                replay.compare(got, requests, reference, dtype, rrms=RRMS16_AT_DEPTH)
            except AssertionError as err:
                raise AssertionError(f"{name} {dtype} {mode} graph={graph}: {err}") from None
            if dtype == "bfloat16":
                median = float(np.median([replay.relative_rms(row, reference[rid][pos]) for (rid, pos), row in got.items()]))
                assert median <= MEDIAN_OVER_TWIN * twin_median, \
                    f"{name} {mode} graph={graph}: median error {median:.4f}, the plain bfloat16-storage twin's is {twin_median:.4f}"
            pool = stepper.cache.page_groups[0].pool
            assert pool.n_free == pool.n_pages and not stepper.cache.requests
            if mode == "mixed":
                assert pool.taken > pool.n_pages, "the pool was to be small enough for pages to be used again"
            if graph:
                report = stepper.graphs.report()
                assert report["hits"] > 0
                if mode == "tail":
                    assert len({k.split("x")[1] for k in report["replays"]}) >= 2, "the decode graphs were to cross a context bucket"
            del stepper
    stepper = None
    kernels.raise_if_kernel_gave_up()
    assert kernels.LAUNCHES["own"] > before["own"]
