"""Generation through the public entry point: greedy tokens equal the plain implementation's;
temperature sampling is reproducible and independent of batching; the command line works."""
import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama as pl
import replay
import tiny_models as tm

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    out = {}
    for name, cfg, seed in (("a", tm.TINY_A, 31), ("b", tm.TINY_B, 32)):
        weights = tm.make_weights(cfg, seed, scale=0.08, bf16_exact=True)
        out[name] = (cfg, weights, tm.write_model_dir(tmp_path_factory.mktemp("gen_" + name), cfg, weights))
    return out


@pytest.mark.parametrize("name", ["a", "b"])
def test_greedy_generation_equals_the_plain_implementation(tiny, name):
    from cisr_b200 import Engine, Model, Request

    cfg, weights, path = tiny[name]
    model = Model.from_pretrained(path, dtype="float32")
    prompts = {f"r{n}": tm.random_tokens(cfg, n, n) for n in (1, 7, 3, 40, 17)}
    expected = {k: pl.generate_greedy(cfg, tm.torch_weights(weights), p, 8) for k, p in prompts.items()}
    outputs = []
    for kw in (dict(policy="serial"), dict(policy="chunked", token_budget=3, prefill_chunk=2),
               dict(policy="decode_first", token_budget=32, prefill_chunk=8),
               dict(policy="decode_first", token_budget=6, prefill_chunk=5, reserve="lazy", pages=6)):
        kw.setdefault("pages", 24)
        engine = Engine.for_model(model, page_size=16, max_active=4, **kw)
        for k, p in prompts.items():
            engine.submit(Request(k, p, max_new_tokens=8))
        outputs.append({r.key: r.generated for r in engine.run()})
        pool = engine.stepper.cache.page_groups[0].pool
        assert pool.n_free == pool.n_pages
        engine.stepper.cache.check()
    assert all(o == expected for o in outputs), (outputs, expected)


def test_eos_stops_generation(tiny):
    from cisr_b200 import Engine, Model, Request

    cfg, weights, path = tiny["a"]
    prompt = tm.random_tokens(cfg, 9, 5)
    full = pl.generate_greedy(cfg, tm.torch_weights(weights), prompt, 8)
    engine = Engine.for_model(Model.from_pretrained(path, dtype="float32"), pages=8)
    eos = full[2]
    engine.submit(Request("e", prompt, max_new_tokens=8, eos_token_id=[eos, 999]))
    assert engine.run()[0].generated == full[:full.index(eos) + 1]


def test_temperature_sampling_is_reproducible_and_independent_of_batching(tiny):
    from cisr_b200 import Engine, Model, Request
    from cisr_b200.sampling import uniform

    cfg, weights, path = tiny["b"]
    model = Model.from_pretrained(path, dtype="float32")
    prompts = {f"r{n}": tm.random_tokens(cfg, n, n) for n in (3, 17, 33, 61)}

    def run(**kw):
        engine = Engine.for_model(model, pages=32, page_size=8, max_active=4, **kw)
        for i, (k, p) in enumerate(prompts.items()):
            engine.submit(Request(k, p, max_new_tokens=6, temperature=0.8, seed=1234 + i))
        return {r.key: r.generated for r in engine.run()}

    first = run(policy="decode_first", token_budget=16, prefill_chunk=8)
    assert first == run(policy="decode_first", token_budget=16, prefill_chunk=8)
    assert first == run(policy="serial", token_budget=64, prefill_chunk=64)
    greedy = {k: pl.generate_greedy(cfg, tm.torch_weights(weights), p, 6) for k, p in prompts.items()}
    assert first != greedy
    # every sampled token is the inverse-CDF choice of the plain softmax at the request's own uniform
    for i, (k, p) in enumerate(prompts.items()):
        seq = list(p)
        for n, token in enumerate(first[k]):
            logits = pl.forward(cfg, tm.torch_weights(weights), seq)[-1]
            cdf = torch.cumsum(pl.temperature_probabilities(logits, 0.8), dim=0)
            u = uniform(1234 + i, n)
            lo = cdf[token - 1].item() if token else 0.0
            assert lo - 1e-4 <= u <= cdf[token].item() + 1e-4
            seq.append(token)


def test_bfloat16_generation_stays_within_the_logits_bound(tiny):
    """bfloat16 through the entry point: a request's first token is chosen from logits that must lie within the replay
    tests' bfloat16 bound of the plain ones, so it must be the plain choice wherever the plain margin between the best
    two logits is wider than that bound allows the logits to move; and from there on every token must again be the plain
    choice for the sequence generated so far, under the same condition."""
    from cisr_b200 import Engine, Model, Request, StepEntry, Stepper

    cfg, weights, path = tiny["a"]
    model = Model.from_pretrained(path, dtype="bfloat16")
    prompts = {f"r{n}": tm.random_tokens(cfg, n, n) for n in (5, 23, 40)}
    engine = Engine.for_model(model, pages=16)
    for k, p in prompts.items():
        engine.submit(Request(k, p, max_new_tokens=8))
    got = {r.key: r.generated for r in engine.run()}
    stepper = Stepper(model, n_pages=16, page_size=16, max_slots=4)
    first = {}
    for k, p in prompts.items():
        stepper.create(k)
        first[k] = stepper.step([StepEntry(k, p, [len(p) - 1])]).cpu().numpy()[0]
    assert all(len(got[k]) == 8 and all(0 <= t < cfg["vocab_size"] for t in got[k]) for k in prompts)
    assert replay.check_generated_tokens(cfg, weights, prompts, got, first) >= 12, "too few tokens had a clear plain choice"


def tiny_tokenizer(folder, words):
    """A word-level tokenizer.json: token id = index in `words`; written with the tokenizers package as a checkpoint's would be."""
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace

    tok = Tokenizer(WordLevel({w: i for i, w in enumerate(words)}, unk_token=words[0]))
    tok.pre_tokenizer = Whitespace()
    tok.save(str(folder / "tokenizer.json"))


def test_command_line_with_a_checkpoint_and_its_tokenizer(tiny, tmp_path):
    """--checkpoint DIR --prompt TEXT: the prompt goes through DIR/tokenizer.json, the generated ids come back as text
    (runtime/__main__.py:29-32,47), and the ids are the plain implementation's greedy choice for the encoded prompt."""
    import shutil

    cfg, weights, path = tiny["a"]
    folder = tmp_path / "checkpoint"
    shutil.copytree(path, folder)
    words = ["<unk>"] + [f"w{i}" for i in range(1, cfg["vocab_size"])]
    tiny_tokenizer(folder, words)
    prompt_ids = [7, 200, 31, 7]
    cmd = [sys.executable, "-m", "cisr_b200", "--dtype", "float32", "--checkpoint", str(folder), "--prompt",
           " ".join(words[i] for i in prompt_ids), "--max-new-tokens", "5", "--pages", "8"]
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=str(replay.ROOT), timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    out = json.loads(proc.stdout)
    assert out["weights"] == "pretrained-local"
    request = out["requests"][0]
    expected = pl.generate_greedy(cfg, tm.torch_weights(weights), prompt_ids, 5, eos=cfg["eos_token_id"])
    assert request["generated"] == expected
    assert request["text"] is not None and request["text"].split() == [words[t] for t in expected]


def test_command_line_prints_the_reference_fields(tiny, tmp_path):
    cfg, weights, path = tiny["a"]
    requests = [{"key": "short", "prompt": [1, 2, 3], "max_new_tokens": 4}, {"key": "later", "prompt": [4, 5, 6, 7], "max_new_tokens": 3, "arrival_s": 0.01}]
    (tmp_path / "requests.json").write_text(json.dumps(requests))
    cmd = [sys.executable, "-m", "cisr_b200", "--dtype", "float32", "--config", "tiny-b", "--seed", "3", "--requests",
           str(tmp_path / "requests.json"), "--policy", "decode_first", "--token-budget", "2", "--pages", "16", "--page-size", "8"]
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=str(replay.ROOT), timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    out = json.loads(proc.stdout)
    assert out["device"] == "cuda" and out["dtype"] == "float32" and out["weights"] == "random-tiny-b"
    assert [r["key"] for r in out["requests"]] == ["short", "later"]
    assert [len(r["generated"]) for r in out["requests"]] == [4, 3]
    assert all(r["status"] == "finished" and r["ttft_ms"] > 0 and r["text"] is None for r in out["requests"])
    single = subprocess.run([sys.executable, "-m", "cisr_b200", "--dtype", "bfloat16", "--tokens", "5,6,7", "--max-new-tokens", "3"],
                            capture_output=True, text=True, cwd=str(replay.ROOT), timeout=600)
    assert single.returncode == 0, single.stderr[-3000:]
    assert len(json.loads(single.stdout)["requests"][0]["generated"]) == 3


def test_kernel_timeline_records_every_launch_of_a_step(tiny):
    """A development build of the kernels (CISR_TRACE=1 in the environment of a fresh process) records when each CTA
    entered and left; a step of the tiny model leaves records of known kernels in launch order, and the Trace Event
    file is valid JSON."""
    cfg, weights, path = tiny["a"]
    script = f"""
import json, os, sys, tempfile
sys.path.insert(0, {str(replay.ROOT)!r})
from cisr_b200 import Model, StepEntry, Stepper
from cisr_b200.ops import trace
import torch
model = Model.from_pretrained({str(path)!r}, dtype="float32")
stepper = Stepper(model, n_pages=8, page_size=16, max_slots=2)
stepper.create("a")
stepper.step([StepEntry("a", [1, 2, 3, 4, 5], [4])])
torch.cuda.synchronize()
records = trace.read()
names = [trace.KERNEL_NAMES[int(k)] for k in records["kernel"]]
assert records.size > 0 and (records["left"] >= records["entered"]).all()
assert names[0] in ("table_update", "embedding", "rotary_table"), names[:3]
assert "attention (CUDA cores)" in names and "add_rmsnorm" in names
launches = trace.summary(records)
assert [l["begin"] for l in launches] == sorted(l["begin"] for l in launches)
out = os.path.join(tempfile.mkdtemp(), "step.json")
trace.write_chrome_trace(records, out)
events = json.load(open(out))["traceEvents"]
assert len(events) >= records.size
assert trace.read().size == 0          # reading empties the buffers
print("timeline ok", records.size, len(launches))
"""
    import os
    env = dict(os.environ, CISR_TRACE="1")
    done = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=env, timeout=240)
    assert done.returncode == 0, done.stdout + done.stderr
    assert "timeline ok" in done.stdout
