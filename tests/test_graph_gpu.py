"""Decode steps replayed from CUDA graphs: same logits and tokens as direct launches."""
import numpy as np
import pytest
import torch

import plain_llama as pl
import replay
import tiny_models as tm

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    cfg = tm.TINY_B
    weights = tm.make_weights(cfg, 41, scale=0.08, bf16_exact=True)
    return cfg, weights, tm.write_model_dir(tmp_path_factory.mktemp("graph"), cfg, weights)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_steps_rebind_requests_and_match_plain(model_dir, dtype):
    """Batch composition changes from step to step (a,b) -> (a) -> (a,b,c) -> (c,a) -> (b): graphs are reused with new contents."""
    from cisr_b200 import Model, StepEntry, Stepper

    cfg, weights, path = model_dir
    model = Model.from_pretrained(path, dtype=dtype)
    stepper = Stepper(model, n_pages=24, page_size=8, max_slots=4, graph=True)
    assert stepper.graphs is not None
    tokens = {k: tm.random_tokens(cfg, 60, i) for i, k in enumerate("abc")}
    reference = {k: replay.plain_logits(cfg, weights, t) for k, t in tokens.items()}
    cursor = {}
    for k, n in (("a", 9), ("b", 1), ("c", 17)):
        stepper.create(k)
        stepper.step([StepEntry(k, tokens[k][:n], [])])           # a prompt portion: launched directly
        cursor[k] = n
    got = {}
    for keys in [("a", "b"), ("a",), ("a", "b", "c"), ("c", "a"), ("b",)] * 6:
        logits = stepper.step([StepEntry(k, [tokens[k][cursor[k]]], [0]) for k in keys]).cpu().numpy()
        for row, k in enumerate(keys):
            got[(k, cursor[k])] = logits[row].copy()
            cursor[k] += 1
        stepper.cache.check()
    replay.compare(got, tokens, reference, dtype)
    report = stepper.graphs.report()
    assert report["hits"] > 0 and report["entries"] == 3 and report["misses"] == 3      # buckets of 1, 2 and 4 rows
    for k in "abc":
        stepper.release(k)
    assert stepper.cache.page_groups[0].pool.n_free == 24


def test_graph_generation_equals_plain_and_direct_launches(model_dir):
    from cisr_b200 import Engine, Model, Request

    cfg, weights, path = model_dir
    model = Model.from_pretrained(path, dtype="float32")
    prompts = {f"r{n}": tm.random_tokens(cfg, n, n) for n in (1, 7, 3, 30)}
    expected = {k: pl.generate_greedy(cfg, tm.torch_weights(weights), p, 10) for k, p in prompts.items()}
    outputs = []
    for graph in (False, True):
        engine = Engine.for_model(model, pages=32, page_size=8, max_active=4, token_budget=16, prefill_chunk=8,
                                  policy="decode_first", graph=graph)
        for k, p in prompts.items():
            engine.submit(Request(k, p, max_new_tokens=10))
        outputs.append({r.key: r.generated for r in engine.run()})
    assert outputs[0] == expected and outputs[1] == expected


def test_temperature_sampling_inside_the_graph_matches_direct_launches(model_dir):
    from cisr_b200 import Engine, Model, Request

    cfg, weights, path = model_dir
    model = Model.from_pretrained(path, dtype="float32")
    outputs = []
    for graph in (False, True):
        engine = Engine.for_model(model, pages=32, page_size=8, max_active=4, token_budget=16, prefill_chunk=8, graph=graph)
        for i, n in enumerate((5, 12, 2)):
            engine.submit(Request(f"t{n}", tm.random_tokens(cfg, n, n), max_new_tokens=9, temperature=0.0 if i == 1 else 0.9, seed=77 + i))
        outputs.append({r.key: r.generated for r in engine.run()})
    assert outputs[0] == outputs[1]


def test_decode_ahead_feeds_tokens_back_on_the_device(model_dir):
    from cisr_b200 import Model, StepEntry, Stepper

    cfg, weights, path = model_dir
    model = Model.from_pretrained(path, dtype="float32")
    stepper = Stepper(model, n_pages=40, page_size=8, max_slots=3, graph=True)
    prompts = {"a": tm.random_tokens(cfg, 11, 1), "b": tm.random_tokens(cfg, 4, 2), "c": tm.random_tokens(cfg, 19, 3)}
    expected = {k: pl.generate_greedy(cfg, tm.torch_weights(weights), p, 14) for k, p in prompts.items()}
    first = {}
    for k, p in prompts.items():
        stepper.create(k)
        first[k] = int(stepper.step([StepEntry(k, p, [len(p) - 1])]).argmax())
    assert first == {k: v[0] for k, v in expected.items()}
    stepper.step([StepEntry(k, [first[k]], [0]) for k in prompts])
    second = stepper.last_tokens.cpu().tolist()
    ahead = stepper.decode_ahead(12).cpu().numpy()
    assert ahead.shape == (12, 3)
    for col, k in enumerate(prompts):
        assert [first[k], second[col]] + ahead[:, col].tolist() == expected[k]
        assert stepper.cache.length(k) == len(prompts[k]) + 13
    stepper.cache.check()
    with pytest.raises(RuntimeError, match="decode_ahead follows"):
        stepper.step([StepEntry("a", [1, 2], [])]); stepper.decode_ahead(2)


def test_staged_tokens_are_read_one_step_behind_the_device(model_dir):
    """Step k + 1 is launched before the host reads step k's tokens from the ring slot that step wrote; the ring has four
    slots and the run is longer than that, so slots are used again."""
    from cisr_b200 import Model, StepEntry, Stepper

    cfg, weights, path = model_dir
    model = Model.from_pretrained(path, dtype="float32")
    stepper = Stepper(model, n_pages=40, page_size=8, max_slots=3, graph=True)
    prompts = {"a": tm.random_tokens(cfg, 9, 4), "b": tm.random_tokens(cfg, 17, 5)}
    expected = {k: pl.generate_greedy(cfg, tm.torch_weights(weights), p, 13) for k, p in prompts.items()}
    first = {}
    for k, p in prompts.items():
        stepper.create(k)
        first[k] = int(stepper.step([StepEntry(k, p, [len(p) - 1])]).argmax())
    stepper.step([StepEntry(k, [first[k]], [0]) for k in prompts])
    got = [stepper.stage_last_tokens().read()]            # the first graph step: staged from its own copy
    pending = None
    for _ in range(11):
        assert stepper.decode_ahead(1, history=False) == 1
        handle = stepper.stage_last_tokens()
        if pending is not None:
            got.append(pending.read())
        pending = handle
    got.append(pending.read())
    for col, k in enumerate(prompts):
        assert [first[k]] + [row[col] for row in got] == expected[k]
    stepper.cache.check()


def test_a_mixer_that_reads_host_values_turns_graphs_off(model_dir):
    from cisr_b200 import Model, Stepper
    from cisr_b200.parts import Mixer

    assert Mixer.graph_safe is False
    cfg, weights, path = model_dir
    model = Model.from_pretrained(path, dtype="float32")
    model.layers[0].mixer.graph_safe = False
    try:
        assert Stepper(model, n_pages=4, page_size=8, max_slots=2, graph=True).graphs is None
    finally:
        del model.layers[0].mixer.graph_safe


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_repeated_step_shapes_replay_from_a_graph_with_new_contents(model_dir, dtype):
    """Portions of the same lengths recur (prompts cut by a fixed budget): from the second time on the step is a graph
    replay whose tokens, positions, requests, pages and wanted rows are rebound."""
    from cisr_b200 import Model, StepEntry, Stepper

    cfg, weights, path = model_dir
    model = Model.from_pretrained(path, dtype=dtype)
    stepper = Stepper(model, n_pages=40, page_size=8, max_slots=4, graph=True)
    tokens = {k: tm.random_tokens(cfg, 75, 10 + i) for i, k in enumerate("abcd")}
    reference = {k: replay.plain_logits(cfg, weights, t) for k, t in tokens.items()}
    got = {}
    for k in "abcd":
        stepper.create(k)
    # shape (30,) five times (a, b, c, d at position 0, then a at 30), shape (15, 1) three times with changing partners
    plan = [[("a", 0, 30)], [("b", 0, 30)], [("c", 0, 30)], [("d", 0, 30)], [("a", 30, 30)],
            [("b", 30, 15), ("a", 60, 1)], [("c", 30, 15), ("a", 61, 1)], [("d", 30, 15), ("b", 45, 1)]]
    for step in plan:
        entries = [StepEntry(k, tokens[k][at:at + n], [n - 1, 0] if n > 1 else [0]) for k, at, n in step]
        logits = stepper.step(entries).cpu().numpy()
        row = 0
        for k, at, n in step:
            for w in ([n - 1, 0] if n > 1 else [0]):
                got[(k, at + w)] = logits[row].copy()
                row += 1
        stepper.cache.check()
    replay.compare(got, tokens, reference, dtype)
    report = stepper.graphs.report()
    assert report["shape_entries"] == 2 and report["hits"] >= 4
    assert sorted(g.replays for g in stepper.graphs.shapes.values()) == [2, 4]


@pytest.mark.parametrize("dtype", ["float32"])
def test_steps_of_one_shape_queued_behind_a_busy_device_keep_their_own_metadata(model_dir, dtype):
    """Steps of a repeated shape run from one captured graph whose metadata sits in one pinned buffer.  When the host
    queues several such steps without reading anything in between (prompt portions with nothing wanted) while the
    device is still busy, a step's copy of that buffer has not run yet when the host prepares the next step: the
    buffer may only be rewritten once its copy has left it, or earlier steps run with later steps' positions, pages
    and tokens.  The device is kept busy by a spin kernel here so that the host does run ahead."""
    from cisr_b200 import Model, StepEntry, Stepper

    cfg, weights, path = model_dir
    model = Model.from_pretrained(path, dtype=dtype)
    stepper = Stepper(model, n_pages=64, page_size=8, max_slots=4, graph=True)
    tokens = {k: tm.random_tokens(cfg, 61, 20 + i) for i, k in enumerate("abcd")}
    reference = {k: replay.plain_logits(cfg, weights, t) for k, t in tokens.items()}
    for k in tokens:
        stepper.create(k)
    # every request in portions of 12 tokens: the shape (12,) repeats, so from its second appearance it is a graph
    stepper.step([StepEntry("a", tokens["a"][:12], [])])
    stepper.step([StepEntry("b", tokens["b"][:12], [])])
    torch.cuda.synchronize()
    torch.cuda._sleep(int(0.2 * 1.9e9))              # about a tenth of a second of device time
    order = [("c", 0), ("d", 0), ("a", 12), ("b", 12), ("c", 12), ("d", 12), ("a", 24), ("b", 24), ("c", 24), ("d", 24),
             ("a", 36), ("b", 36), ("c", 36), ("d", 36), ("a", 48), ("b", 48), ("c", 48), ("d", 48)]
    for k, at in order:                              # all queued while the device still spins
        stepper.step([StepEntry(k, tokens[k][at:at + 12], [])])
    assert stepper.graphs.report()["shape_entries"] >= 1
    got = {}
    for k in tokens:                                 # the last token of each: its logits depend on everything before
        got[(k, 60)] = stepper.step([StepEntry(k, [tokens[k][60]], [0])]).cpu().numpy()[0].copy()
    replay.compare(got, tokens, reference, dtype)
    stepper.cache.check()
