"""Helpers of the replay tests: build traces, run them through the engine, compare with the plain implementation."""
from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

import plain_llama
import tiny_models

ROOT = Path(__file__).resolve().parent.parent


def plain_logits(cfg: dict, weights: dict, tokens: Sequence[int], dtype=torch.float64, storage=None) -> np.ndarray:
    return plain_llama.forward(cfg, tiny_models.torch_weights(weights), list(tokens), dtype, storage).to(torch.float64).numpy()


# ------------------------------------------------------------------ traces
def trace_whole(requests: Dict[str, List[int]]) -> List[dict]:
    """Each request alone, its whole prompt in one step, logits everywhere."""
    steps = []
    for i, (rid, tokens) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": tokens, "want": list(range(len(tokens)))}], "end": [rid]})
    return steps


def trace_tail_decode(requests: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Most of a request in one step, then its last `tail` tokens one by one."""
    steps = []
    n = 0
    for rid, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": tokens[:head], "want": list(range(head))}], "end": []})
        n += 1
        for t in range(head, len(tokens)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [tokens[t]], "want": [0]}],
                          "end": [rid] if t == len(tokens) - 1 else []})
            n += 1
        if head == len(tokens):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(requests: Dict[str, List[int]], sizes: Sequence[int]) -> List[dict]:
    """Portions of changing size (cycled from `sizes`), down to two tokens."""
    steps = []
    n = 0
    for rid, tokens in requests.items():
        at, k = 0, 0
        while at < len(tokens):
            size = min(sizes[k % len(sizes)], len(tokens) - at)
            k += 1
            end = at + size
            steps.append({"step": n, "entries": [{"id": rid, "tokens": tokens[at:end], "want": list(range(size))}],
                          "end": [rid] if end == len(tokens) else []})
            at = end
            n += 1
    return steps


def trace_mixed(requests: Dict[str, List[int]], seed: int, max_live: int = 4, decode_tail: int = 12,
                sizes: Sequence[int] = (9, 2, 17, 5, 3, 30, 2, 11)) -> List[dict]:
    """Up to `max_live` live requests; portions of some beside single tokens of others; requests
    start as earlier ones end, and a request is sometimes left out of a step."""
    rng = np.random.default_rng(seed)
    waiting = list(requests.items())
    live: List[list] = []    # [rid, tokens, cursor]
    steps = []
    n = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, tokens = waiting.pop(0)
            live.append([rid, tokens, 0])
        entries, ended = [], []
        for item in live:
            rid, tokens, cursor = item
            if len(live) > 1 and rng.random() < 0.2:
                continue   # left out of this step, goes on later
            remaining = len(tokens) - cursor
            if remaining <= decode_tail:
                size = 1
            else:
                size = int(min(sizes[int(rng.integers(len(sizes)))], remaining - decode_tail))
            entries.append({"id": rid, "tokens": tokens[cursor:cursor + size], "want": list(range(size))})
            item[2] += size
            if item[2] == len(tokens):
                ended.append(rid)
        if not entries:
            continue
        steps.append({"step": n, "entries": entries, "end": ended})
        live = [item for item in live if item[0] not in ended]
        n += 1
    return steps


def max_live_tokens(steps: List[dict], round_to: int = 64) -> int:
    """The --max-tokens a trace needs: most tokens held at any time, each request rounded up."""
    held: Dict[str, int] = {}
    peak = 0
    for step in steps:
        for e in step["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-v // round_to) * round_to for v in held.values()))
        for rid in step["end"]:
            held.pop(rid, None)
    return peak


# ------------------------------------------------------------------ running
def run_steps(stepper, steps: List[dict]) -> Dict[Tuple[str, int], np.ndarray]:
    """Drive a Stepper with a trace in process; logits keyed by (request, position)."""
    from cisr_b200 import StepEntry

    out: Dict[Tuple[str, int], np.ndarray] = {}
    cursor: Dict[str, int] = {}
    for step in steps:
        entries = []
        for e in step["entries"]:
            if e["id"] not in stepper.cache.requests:
                stepper.create(e["id"])
                cursor[e["id"]] = 0
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        logits = stepper.step(entries).to("cpu").numpy()
        row = 0
        for e in step["entries"]:
            for w in e["want"]:
                out[(e["id"], cursor[e["id"]] + w)] = logits[row]
                row += 1
            cursor[e["id"]] += len(e["tokens"])
        for rid in step["end"]:
            stepper.release(rid)
        stepper.cache.check()
    return out


def run_trace_program(model_dir, dtype: str, steps: List[dict], out_dir, max_tokens: int, vocab: int,
                      env=None, timeout: int = 900) -> Dict[Tuple[str, int], np.ndarray]:
    """Drive bin/trace_run as a user would; logits keyed by (request, position)."""
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", str(max_tokens)], input=text, capture_output=True,
                          text=True, timeout=timeout, env=env)
    if proc.returncode != 0:
        raise RuntimeError(f"trace_run exited with {proc.returncode}\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}")
    done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps], "one 'done <step>' line per step, in order"
    out: Dict[Tuple[str, int], np.ndarray] = {}
    cursor: Dict[str, int] = {}
    for step in steps:
        wanted = sum(len(e["want"]) for e in step["entries"])
        path = Path(out_dir) / f"{step['step']}.f32"
        if wanted:
            data = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
        row = 0
        for e in step["entries"]:
            cursor.setdefault(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], cursor[e["id"]] + w)] = data[row]
                row += 1
            cursor[e["id"]] += len(e["tokens"])
    return out


# ------------------------------------------------------------------ comparing
# Tolerances, fixed when the first kernels passed and never widened since:
# float32: every logit within ATOL32 * max|reference row| + RTOL32 * |reference| of the float64 plain
#          implementation (the plain implementation run in float32 differs from its float64 self by up to
#          a quarter of this on the same models).
# bfloat16: relative RMS error of each logits row below RRMS16, against the plain implementation
#           run in float64 on the same (bfloat16-exact) weights (the reference's own bound for bfloat16
#           logits is 0.04, tests/test_precision.py:27-28).
ATOL32, RTOL32 = 1.5e-5, 1.5e-5
RRMS16 = 0.03


def relative_rms(row: np.ndarray, ref: np.ndarray) -> float:
    return float(np.sqrt(np.mean((row.astype(np.float64) - ref) ** 2) / max(np.mean(ref ** 2), 1e-30)))


def compare(got: Dict[Tuple[str, int], np.ndarray], requests: Dict[str, List[int]], reference: Dict[str, np.ndarray],
            dtype: str, scale: float = 1.0, rrms: float = None) -> None:
    """`rrms`: another bound than RRMS16 for the bfloat16 rows (a test that uses one says why)."""
    assert got, "nothing was compared"
    rrms = RRMS16 if rrms is None else rrms
    worst = 0.0
    for (rid, pos), row in sorted(got.items()):
        ref = reference[rid][pos]
        assert row.shape == ref.shape
        assert np.isfinite(row).all(), f"non-finite logits for {rid} at position {pos}"
        if dtype == "float32":
            err = np.abs(row.astype(np.float64) - ref)
            bound = scale * ATOL32 * max(1.0, float(np.abs(ref).max())) + RTOL32 * np.abs(ref)
            if not (err <= bound).all():
                i = int(np.argmax(err - bound))
                raise AssertionError(f"float32 logits differ for request {rid} at position {pos}, vocab index {i}: "
                                     f"got {row[i]!r}, plain {ref[i]!r}, |diff| {err[i]:.3e} (first wrong place in order)")
        else:
            rel = relative_rms(row, ref)
            worst = max(worst, rel)
            if not rel < rrms:
                raise AssertionError(f"bfloat16 logits differ for request {rid} at position {pos}: relative RMS error "
                                     f"{rel:.4f} >= {rrms}")


def check_generated_tokens(cfg: dict, weights: dict, prompts: Dict[str, List[int]], generated: Dict[str, List[int]],
                           first_logits: Dict[str, np.ndarray]) -> int:
    """Greedy bfloat16 generation against the plain implementation, without asking for luck.

    `first_logits[k]`: the engine's logits at the last prompt position of request k, which must be within the bfloat16
    bound of the plain ones.  Then every generated token must be the plain choice for the sequence generated so far
    wherever the plain margin between the two best logits is wider than that bound lets a logit move (a relative RMS
    error of RRMS16 over a row moves single logits by a few times RRMS16 * rms(row)).  Returns how many tokens had
    such a margin and were checked."""
    tw = tiny_models.torch_weights(weights)
    reference = {k: plain_llama.forward(cfg, tw, p).numpy() for k, p in prompts.items()}
    compare({(k, len(prompts[k]) - 1): row for k, row in first_logits.items()}, prompts, reference, "bfloat16")
    checked = 0
    for k, p in prompts.items():
        seq = list(p)
        for n, token in enumerate(generated[k]):
            logits = reference[k][-1] if n == 0 else plain_llama.forward(cfg, tw, seq)[-1].numpy()
            best = np.sort(logits)[-2:]
            if best[1] - best[0] > 8 * RRMS16 * float(np.sqrt(np.mean(logits ** 2))):
                assert token == int(np.argmax(logits)), f"request {k}: generated token {n} is {token}, the plain choice is {int(np.argmax(logits))}"
                checked += 1
            seq.append(token)          # follow the engine's own sequence
    return checked
