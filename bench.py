"""Decode and prefill throughput of the engine on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--preset smollm2-135m] [--batch 8] [--context 4096] [--dtype bfloat16] [--layers L]

Default run: the SmolLM2-135M layer sizes with seeded random weights, bfloat16, batch 8,
every request holding about 4096 tokens of context while it decodes.  Prints ONE JSON line:

  value        decoded tokens per second, K decode steps timed on the device with CUDA events; the steps
               run from the captured decode graph with sampled tokens fed back on the device
  e2e          the same through the Python entry point (Engine.tick): every step copies its inputs from
               pinned host memory and reads its chosen tokens back to the host
  prefill      one 2048-token prompt in one step: tokens/s, ms, and flops / time / tensor peak
  roofline     bytes a decode step must read (every weight once + the live cache) / time, against the
               measured copy bandwidth
  points       decode tokens/s at batch 1 and 64 at the same context
  gpu_launches kernels of this package launched in the timed region (library matrix products not counted)

Peaks come from MEASURED_PEAKS.json beside this file when the driver wrote it, else 6.65 TB/s and
1.59 PFLOP/s.  No L2 flush is needed: a decode step reads several hundred MB (weights + cache), more than
the 126 MB L2, which `config.l2` records.  Inputs are seeded synthetic token ids, uniform over the vocabulary.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
PUBLISHED_DECODE_B1_TOKS = 203.9      # the reference's own best decode figure (batch 1, float32, RTX 4060 Laptop)
PREFILL_TOKENS = 2048


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            raw = json.loads(path.read_text())
            return float(raw["hbm_gbs"]), float(raw.get("bf16_tflops_sustained") or raw["bf16_tflops"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


class ClockSampler:
    """nvidia-smi in the background, sampling clocks and throttle reasons every 200 ms."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            index = os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0] or "0"
            self.proc = subprocess.Popen(["nvidia-smi", "-i", index, f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [line.split(",") for line in Path(self.file.name).read_text().splitlines() if line.count(",") >= 6]
        os.unlink(self.file.name)
        clocks, maxes, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in rows:
            try:
                clocks.append(float(row[0])); maxes.append(float(row[1]))
            except ValueError:
                continue
            for name, cell in zip(names, row[3:7]):
                if cell.strip().lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max(maxes) if maxes else None,
                "reasons": sorted(reasons), "samples": len(clocks)}


def model_bytes_and_flops(cfg, layers: int, dtype_bytes: int):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hq, hkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = h * (hq + 2 * hkv) * d + hq * d * h + 3 * h * i
    weight_bytes = (layers * per_layer + v * h) * dtype_bytes + (2 * layers + 1) * h * 4   # matrices once (head = tied table), norms
    kv_bytes_per_token = layers * 2 * hkv * d * dtype_bytes
    return per_layer, weight_bytes, kv_bytes_per_token


def prefill_flops(cfg, layers: int, tokens: int) -> float:
    per_layer, _, _ = model_bytes_and_flops(cfg, layers, 2)
    hq, d = cfg["num_attention_heads"], cfg["head_dim"]
    gemm = 2.0 * tokens * per_layer * layers + 2.0 * cfg["vocab_size"] * cfg["hidden_size"]   # the head runs on one row
    attention = layers * 2 * 2.0 * hq * d * tokens * (tokens + 1) / 2                          # QK^T and PV over the causal half
    return gemm + attention


def make_model(args):
    from cisr_b200 import Model
    from cisr_b200.config.llama import preset_dict

    raw = preset_dict(args.preset)
    full_layers = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = min(args.layers, full_layers)
    model = Model.from_config(raw, seed=args.seed, dtype=args.dtype)
    return model, raw, full_layers


def fill_requests(stepper, keys, context: int, vocab: int, seed: int, chunk: int = 2048):
    """Give every request `context` tokens of cache by running real prompt portions through the engine."""
    import numpy as np
    from cisr_b200 import StepEntry

    rng = np.random.default_rng(seed)
    last = {}
    for key in keys:
        stepper.create(key)
        tokens = rng.integers(0, vocab, size=context).tolist()
        for at in range(0, context, chunk):
            stepper.step([StepEntry(key, tokens[at:at + chunk], [])])
        last[key] = int(rng.integers(0, vocab))
    return last


PAGE_SIZE = 16       # --page-size changes it for every run of the process


def device_decode(model, batch: int, context: int, steps: int, warmup: int, seed: int):
    """tokens/s of `steps` decode steps ending at `context` tokens per request, timed with CUDA events."""
    import torch
    from cisr_b200 import StepEntry, Stepper

    page = PAGE_SIZE
    start_ctx = context - steps - warmup - 1
    pages = batch * (-(-context // page) + 1)
    stepper = Stepper(model, n_pages=pages, page_size=page, max_slots=batch, graph=True)
    keys = [f"r{i}" for i in range(batch)]
    last = fill_requests(stepper, keys, start_ctx, model.spec.vocab_size, seed)
    stepper.step([StepEntry(k, [last[k]], [0]) for k in keys])          # captures the graph, runs one step
    stepper.decode_ahead(warmup)
    graph = stepper._ahead[0]
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()     # a profiler started with --profile-from-start off sees only the timed steps
    begin.record()
    ran = stepper.decode_ahead(steps).shape[0]
    end.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    assert ran == steps, f"only {ran} of {steps} steps fit below the graph's context limit"
    ms = begin.elapsed_time(end)
    final_ctx = stepper.cache.length(keys[0])
    launches = graph.launches
    for k in keys:
        stepper.release(k)
    del stepper
    torch.cuda.empty_cache()
    return batch * steps / (ms / 1e3), ms / steps, final_ctx, launches


def entry_point_decode(model, batch: int, context: int, steps: int, warmup: int, seed: int):
    """The same through Engine.tick: host token ids in (pinned copy per step), chosen tokens out (read per step)."""
    import numpy as np
    import torch
    from cisr_b200 import Engine, Request

    page = PAGE_SIZE
    prompt_len = context - steps - warmup - 2
    engine = Engine.for_model(model, pages=batch * (-(-context // page) + 2), page_size=page, max_active=batch,
                              token_budget=max(2048, batch), prefill_chunk=2048, policy="decode_first", graph=True)
    rng = np.random.default_rng(seed + 1)
    for i in range(batch):
        engine.submit(Request(f"e{i}", rng.integers(0, model.spec.vocab_size, size=prompt_len).tolist(),
                              max_new_tokens=steps + warmup + 2))
    while any(r.status != "decode" for r in engine.requests.values()):
        engine.tick()
    for _ in range(warmup):
        engine.tick()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.tick()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    decoded = sum(t["decode_tokens"] for t in engine.trace[-steps:])
    graph = engine.stepper._ahead[0] if engine.stepper._ahead else None
    # per step the host sends the block-table update lists (tokens are fed back on the device) and reads the sampled
    # tokens with the kernels' status word
    h2d = (graph.dev.numel() - graph.upd_start) * 4 if graph is not None else 0
    d2h = (graph.rows + 1) * 4 if graph is not None else batch * 4
    for r in list(engine.active):
        engine.cancel(r.key)
    del engine
    torch.cuda.empty_cache()
    return decoded / seconds, h2d, d2h


def prefill_run(model, tokens: int, seed: int, reps: int = 5, profile: bool = False):
    import numpy as np
    import torch
    from cisr_b200 import StepEntry, Stepper

    rng = np.random.default_rng(seed + 2)
    ids = rng.integers(0, model.spec.vocab_size, size=tokens).tolist()
    stepper = Stepper(model, n_pages=-(-tokens // PAGE_SIZE) + 1, page_size=PAGE_SIZE, max_slots=1, graph=True)
    times = []
    for rep in range(reps + 3):
        stepper.create("p")
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        stepper.step([StepEntry("p", ids, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        stepper.release("p")
        if rep >= 3:
            times.append(begin.elapsed_time(end))
        if rep == 2 and profile:
            torch.cuda.profiler.start()
        if rep == 3 and profile:
            torch.cuda.profiler.stop()
    ms = statistics.median(times)
    del stepper
    torch.cuda.empty_cache()
    return ms


def decode_timeline(model, batch: int, context: int, seed: int, path: str) -> int:
    """The last of a few decode steps, launch by launch, from the kernels' own clock stamps (a development build of the
    kernels, about a tenth slower than the ordinary one: compare shares and gaps, not absolutes)."""
    import numpy as np
    import torch
    from cisr_b200 import StepEntry, Stepper
    from cisr_b200.ops import trace

    if not trace.enabled():
        print("--timeline needs CISR_TRACE=1 in the environment (the kernels are then built with their recording code)")
        return 2
    page, steps, warmup = PAGE_SIZE, 3, 4
    stepper = Stepper(model, n_pages=batch * (-(-context // page) + 1), page_size=page, max_slots=batch, graph=True)
    keys = [f"r{i}" for i in range(batch)]
    last = fill_requests(stepper, keys, context - steps - warmup - 1, model.spec.vocab_size, seed)
    stepper.step([StepEntry(k, [last[k]], [0]) for k in keys])
    stepper.decode_ahead(warmup)
    torch.cuda.synchronize()
    trace.read()                                     # drop what the prompt and the warm-up recorded
    stepper.decode_ahead(steps)
    torch.cuda.synchronize()
    records = trace.read()
    start = records[records["kernel"] == 1]["entered"].max() - 20000      # the last step: from just before its embedding launch
    step = records[records["entered"] >= start]
    previous_end = None
    print(f"{'kernel':28s} {'CTAs':>5s} {'first entry':>12s} {'released':>10s} {'last exit':>10s} {'after the one before':>21s}   (ns)")
    for launch in trace.summary(step):
        gap = "" if previous_end is None else str(launch["end"] - previous_end)
        released = "" if launch["released"] is None else str(launch["released"])
        print(f"{launch['kernel']:28s} {launch['ctas']:5d} {launch['begin']:12d} {released:>10s} {launch['end']:10d} {gap:>21s}")
        previous_end = launch["end"]
    trace.write_chrome_trace(step, path)
    print(f"wrote {path}: {step.size} CTAs of one decode step")
    return 0


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--preset", default="smollm2-135m")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    parser.add_argument("--layers", type=int, default=0, help="run fewer layers than the preset has (both numbers are reported)")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--no-points", action="store_true", help="skip the batch 1 and batch 64 points")
    parser.add_argument("--only", choices=["all", "decode", "prefill"], default="all",
                        help="decode: only the device-timed decode steps; prefill: only the 2048-token prompt (for profiling)")
    parser.add_argument("--page-size", type=int, default=16, help="tokens per cache page (the trace program uses 16)")
    parser.add_argument("--timeline", metavar="FILE", default=None,
                        help="with CISR_TRACE=1 in the environment: run a few decode steps with kernels that record when each "
                             "CTA entered, got past its wait and left; print the last step launch by launch and write it "
                             "to FILE in the Trace Event format (chrome://tracing, Perfetto)")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference has no setup.py or pyproject.toml, so pip cannot "
                          "install it, and its CUDA path imports cupy, which is neither in this image nor in the wheelhouse"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine is single-GPU by design (--gpus {args.gpus} is not run)")
        return 2
    args.warmup = max(args.warmup, 3)
    global PAGE_SIZE
    PAGE_SIZE = args.page_size

    import torch

    hbm_gbs, bf16_tflops, peak_source = peaks()
    model, raw, full_layers = make_model(args)
    layers = raw["num_hidden_layers"]
    dtype_bytes = 2 if args.dtype == "bfloat16" else 4

    if args.timeline:
        return decode_timeline(model, args.batch, args.context, args.seed, args.timeline)
    if args.only == "prefill":
        ms = prefill_run(model, PREFILL_TOKENS, args.seed, reps=2, profile=True)
        print(json.dumps({"only": "prefill", "tokens": PREFILL_TOKENS, "ms": round(ms, 3)}))
        return 0
    if args.only == "decode":
        value, ms_per_step, _, launches = device_decode(model, args.batch, args.context, args.steps, args.warmup, args.seed)
        print(json.dumps({"only": "decode", "value": round(value, 1), "ms_per_step": round(ms_per_step, 4), "launches_per_step": launches}))
        return 0
    sampler = ClockSampler().start()
    value, ms_per_step, final_ctx, launches = device_decode(model, args.batch, args.context, args.steps, args.warmup, args.seed)
    clocks = sampler.stop()
    e2e, h2d, d2h = entry_point_decode(model, args.batch, args.context, min(args.steps, 128), args.warmup, args.seed)
    prefill_ms = prefill_run(model, PREFILL_TOKENS, args.seed)
    points = {}
    if not args.no_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(device_decode(model, b, args.context, min(args.steps, 128), args.warmup, args.seed)[0], 1)

    _, weight_bytes, kv_per_token = model_bytes_and_flops(raw, layers, dtype_bytes)
    mean_ctx = final_ctx - args.steps / 2
    step_bytes = weight_bytes + args.batch * mean_ctx * kv_per_token
    achieved_gbs = step_bytes / (ms_per_step / 1e3) / 1e9
    flops = prefill_flops(raw, layers, PREFILL_TOKENS)
    peak_flops = bf16_tflops * 1e12 if args.dtype == "bfloat16" else 75e12
    line = {
        "metric": "decode tok/s (SmolLM2-135M shape, batch 8, context 4096)" if args.preset == "smollm2-135m" else f"decode tok/s ({args.preset})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic token ids, seeded random weights",
        "config": {"model": args.preset, "global_batch": args.batch, "seq_len": args.context, "parallelism": "single-gpu",
                   "layers": layers, "layers_of_preset": full_layers, "hidden_size": raw["hidden_size"],
                   "intermediate_size": raw["intermediate_size"], "heads": raw["num_attention_heads"],
                   "kv_heads": raw["num_key_value_heads"], "head_dim": raw["head_dim"], "vocab_size": raw["vocab_size"],
                   "page_size": PAGE_SIZE, "decode": "cuda graph, tokens fed back on device", "peaks": peak_source,
                   "l2": "inputs larger than L2 (weights + cache per step), no flush"},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches["own"] * args.steps, "library_gemm_launches": launches["library"] * args.steps,
        "clocks": clocks,
        "prefill": {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms / 1e3) / peak_flops, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved_gbs, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved_gbs / hbm_gbs, 4)},
        "points": points,
        "published_reference_decode_b1": PUBLISHED_DECODE_B1_TOKS,
    }
    if "decode_b1" in points:
        line["decode_b1_vs_published"] = round(points["decode_b1"] / PUBLISHED_DECODE_B1_TOKS, 1)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
