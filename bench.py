"""Decode and prefill throughput of the engine on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--preset smollm2-135m] [--batch 8] [--context 4096] [--dtype bfloat16] [--layers L]
                    [--workload decode|mixed]

Default run: the SmolLM2-135M layer sizes with seeded random weights, bfloat16, batch 8,
every request holding about 4096 tokens of context while it decodes.  Prints ONE JSON line:

  value        decoded tokens per second: windows of K decode steps, each timed on the device with CUDA events,
               repeated back to back until at least half a second has been timed; the median window counts
               (`ms_per_step_spread` gives the fastest and slowest).  The steps run from the captured decode
               graph with sampled tokens fed back on the device
  e2e          the same through the Python entry point (Engine.tick): every step copies its inputs from
               pinned host memory and reads its chosen tokens back to the host
  prefill      one 2048-token prompt in one step: tokens/s, ms, and flops / time / tensor peak
  roofline     bytes a decode step must read (every weight once + the live cache) / time, against the
               measured copy bandwidth
  points       decode at batch 1 and 64 at the same context: tokens/s, and how many kernels of this package
               and how many vendor-library products one step launches
  kernels      the kernels a decode step and the prompt spend most time in, each launched alone (outside graphs,
               bracketed by CUDA events): time per launch, the bytes it must move or the flops it must do, and the
               fraction of the measured peak (copy bandwidth; burst bfloat16 product) that this comes to
  gpu_launches kernels of this package launched in the timed region (library matrix products are counted
               apart, in library_gemm_launches)

--workload mixed: the continuous-batching workload (by default the SmolLM2-1.7B sizes, 64 requests with prompts
of 128 to 2048 tokens, 256 generated tokens each) through the scheduler with graphs on; prints total, prefill
and decode tokens per second, launch counts, graph statistics and a roofline for the whole run.
--impl reference: the reference's own stock code on the same decode workload (see reference_arm).

Peaks come from MEASURED_PEAKS.json beside this file when the driver wrote it, else 6.65 TB/s and
1.59 PFLOP/s; the float32 product peak is measured here (the pedantic library product, 8192^3).  No L2 flush is
needed: a decode step reads several hundred MB (weights + cache), more than the 126 MB L2, which `config.l2`
records.  Inputs are seeded synthetic token ids, uniform over the vocabulary.
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
    """(copy bandwidth GB/s, bfloat16 product TFLOP/s sustained, the same as a burst, where they come from)."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            raw = json.loads(path.read_text())
            burst = float(raw["bf16_tflops"])
            return float(raw["hbm_gbs"]), float(raw.get("bf16_tflops_sustained") or burst), burst, "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, FALLBACK_BF16_TFLOPS, "fallback"


def measure_fp32_peak() -> float:
    """TFLOP/s of the true 32-bit library product (cublasGemmEx, 32-bit compute, pedantic math: what the float32
    path of the engine runs) on 8192^3, best of three: the denominator of the float32 prefill fraction."""
    import torch
    from cisr_b200.ops import kernels

    n = 8192
    a = torch.randn(n, n, device="cuda"); w = torch.randn(n, n, device="cuda"); out = torch.empty(n, n, device="cuda")
    kernels.gemm_library(a, w, out)
    best = float("inf")
    for _ in range(3):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(); kernels.gemm_library(a, w, out); end.record()
        torch.cuda.synchronize()
        best = min(best, begin.elapsed_time(end))
    del a, w, out
    torch.cuda.empty_cache()
    return 2.0 * n ** 3 / (best / 1e3) / 1e12


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
    from cisr_b200.config import preset_dict

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


MIN_TIMED_SECONDS = 0.5      # every decode figure is timed at least this long, whatever --steps says


def device_decode(model, batch: int, context: int, steps: int, warmup: int, seed: int, min_seconds: float = MIN_TIMED_SECONDS):
    """Decode steps ending at `context` tokens per request: windows of `steps` steps, each timed with CUDA events, back to
    back until `min_seconds` have been timed.  Returns tokens/s and ms per step of the median window, the spread over the
    windows, the mean context of the timed steps and the kernels one step launches."""
    import torch
    from cisr_b200 import StepEntry, Stepper

    page = PAGE_SIZE
    probe = 8                                            # steps timed first to learn how many windows half a second takes
    # a first guess of the number of windows from a rough step time; corrected after the probe
    stepper = None
    windows = 1
    for attempt in range(2):
        total_steps = windows * steps + warmup + probe + 1
        start_ctx = max(1, context - total_steps)
        pages = batch * (-(-context // page) + 1)
        stepper = Stepper(model, n_pages=pages, page_size=page, max_slots=batch, graph=True)
        keys = [f"r{i}" for i in range(batch)]
        last = fill_requests(stepper, keys, start_ctx, model.spec.vocab_size, seed)
        stepper.step([StepEntry(k, [last[k]], [0]) for k in keys])          # captures the graph, runs one step
        stepper.decode_ahead(warmup)
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(); stepper.decode_ahead(probe); end.record()
        torch.cuda.synchronize()
        step_ms = begin.elapsed_time(end) / probe
        needed = max(1, min(int(min_seconds * 1e3 / (step_ms * steps)) + 1, max(1, (context - 64) // steps)))
        if attempt == 1 or needed <= windows:
            break
        windows = needed                                  # start again further back, so that the last window ends at `context`
        for k in keys:
            stepper.release(k)
        del stepper
        torch.cuda.empty_cache()
    graph = stepper._ahead[0]
    times, contexts = [], []
    torch.cuda.profiler.start()     # a profiler started with --profile-from-start off sees only the timed steps
    for _ in range(windows):
        before = stepper.cache.length(keys[0])
        if before + steps > context:
            break
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        ran = stepper.decode_ahead(steps).shape[0] if stepper.can_run_ahead() else 0
        end.record()
        torch.cuda.synchronize()
        if ran == steps:
            times.append(begin.elapsed_time(end))
            contexts.append(before + steps / 2)
            continue
        # the edge of the graph's context bucket: this window does not count; one ordinary step with the tokens just
        # sampled captures the next bucket's graph, a few more warm it up
        tokens = stepper.last_tokens.tolist()
        stepper.step([StepEntry(k, [int(t)], [0]) for k, t in zip(keys, tokens)])
        stepper.decode_ahead(min(warmup, context - stepper.cache.length(keys[0]) - 1))
        torch.cuda.synchronize()
        graph = stepper._ahead[0]
    torch.cuda.profiler.stop()
    assert times, f"not one window of {steps} steps fit below the graph's context limit"
    order = sorted(range(len(times)), key=times.__getitem__)
    mid = order[len(order) // 2]
    launches = dict(graph.launches)
    final_ctx = stepper.cache.length(keys[0])
    for k in keys:
        stepper.release(k)
    del stepper
    torch.cuda.empty_cache()
    return {"value": batch * steps / (times[mid] / 1e3), "ms_per_step": times[mid] / steps, "windows": len(times),
            "spread": (min(times) / steps, max(times) / steps), "mean_ctx": contexts[mid], "final_ctx": final_ctx, "launches": launches}


def entry_point_decode(model, batch: int, context: int, steps: int, warmup: int, seed: int, min_seconds: float = MIN_TIMED_SECONDS):
    """The same through Engine.tick: host token ids in (pinned copy per step), chosen tokens out (read per step).
    Windows of `steps` ticks timed by the host clock around synchronisations, until `min_seconds`; the median counts."""
    import numpy as np
    import torch
    from cisr_b200 import Engine, Request

    page = PAGE_SIZE
    windows = max(1, min(int(min_seconds / (steps * 1e-3)) + 1, (context - 256) // steps))     # about a millisecond a step
    total = windows * steps + warmup + 2
    prompt_len = max(1, context - total)
    engine = Engine.for_model(model, pages=batch * (-(-context // page) + 2), page_size=page, max_active=batch,
                              token_budget=max(2048, batch), prefill_chunk=2048, policy="decode_first", graph=True)
    rng = np.random.default_rng(seed + 1)
    for i in range(batch):
        engine.submit(Request(f"e{i}", rng.integers(0, model.spec.vocab_size, size=prompt_len).tolist(), max_new_tokens=total))
    while any(r.status != "decode" for r in engine.requests.values()):
        engine.tick()
    for _ in range(warmup):
        engine.tick()
    rates = []
    spent = 0.0
    for _ in range(windows):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            engine.tick()
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        rates.append(sum(t["decode_tokens"] for t in engine.trace[-steps:]) / seconds)
        spent += seconds
        if spent >= min_seconds:
            break
    graph = engine.stepper._ahead[0] if engine.stepper._ahead else None
    # per step the host sends the block-table update lists (tokens are fed back on the device) and reads the sampled
    # tokens with the kernels' status word
    h2d = (graph.dev.numel() - graph.upd_start) * 4 if graph is not None else 0
    d2h = (graph.rows + 1) * 4 if graph is not None else batch * 4
    for r in list(engine.active):
        engine.cancel(r.key)
    del engine
    torch.cuda.empty_cache()
    return statistics.median(rates), h2d, d2h


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


# ------------------------------------------------------------------ per-kernel rooflines
EPILOGUE_NAMES = {0: "plain", 1: "swiglu", 2: "rope"}


def kernel_need(name: str, shape: tuple, cfg: dict, dtype_bytes: int, cache_tokens: int, causal_tokens: int):
    """(bytes a launch must move, flops it must do, a label) from the kernel's name and the shape it was called with.
    `cache_tokens`: tokens of context the step's single-token requests hold together (what the decode attention reads);
    `causal_tokens`: the length of the one prompt the prompt attention runs over."""
    hq, hkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    if name == "skinny_gemm":
        tokens, n, k, epilogue, normed = shape
        label = f"weight-streaming product {EPILOGUE_NAMES[epilogue]}{' +norm' if normed else ''} [{tokens}x{k}]x[{n}x{k}]"
        return n * k * 2 + tokens * k * (8 if normed else 2), 2.0 * tokens * n * k, label
    if name in ("gemm_tcgen05", "gemm_tcgen05_swiglu", "gemm_tcgen05_rope", "gemm_library"):
        m, n, k = shape
        out_bytes = m * n * (4 if name in ("gemm_tcgen05", "gemm_library") else 2)
        label = {"gemm_tcgen05": "tcgen05 product", "gemm_tcgen05_swiglu": "tcgen05 product + SwiGLU",
                 "gemm_tcgen05_rope": "tcgen05 product + rotation + cache write", "gemm_library": "library product"}[name]
        return (m * k + n * k) * dtype_bytes + out_bytes, 2.0 * m * n * k, f"{label} [{m}x{k}]x[{n}x{k}]"
    if name == "attn_decode":
        n_dec = shape[0]
        return cache_tokens * 2 * hkv * d * dtype_bytes, 4.0 * cache_tokens * hq * d, f"decode attention + merge, {n_dec} requests"
    if name in ("attn_prefill_wide", "attn_prefill"):
        tokens = shape[0]
        label = "prompt attention (tcgen05)" if name == "attn_prefill_wide" else "prompt attention"
        return 2 * tokens * (hq + 2 * hkv) * d * dtype_bytes, 4.0 * hq * d * causal_tokens * (causal_tokens + 1) / 2, f"{label}, {tokens} tokens"
    if name == "add_rmsnorm":
        rows, hidden, added = shape
        return rows * hidden * (4 + (8 if added else 0) + dtype_bytes), 0.0, f"{'add + ' if added else ''}RMSNorm [{rows}x{hidden}]"
    if name == "sample":
        rows, vocab = shape
        return rows * vocab * 4, 0.0, f"sampling [{rows}x{vocab}]"
    if name == "embedding":
        rows, hidden = shape
        return rows * hidden * (4 + dtype_bytes), 0.0, f"embedding [{rows}x{hidden}]"
    return 0, 0.0, name


def kernel_rooflines(model, raw: dict, batch: int, context: int, seed: int, dtype_bytes: int, hbm_gbs: float, burst_tflops: float,
                     top: int = 5) -> dict:
    """The kernels one decode step and one 2048-token prompt spend most time in, each launch alone between two CUDA
    events (no graph, no overlap with its neighbours: the isolated kernel), against the measured peaks: a launch's
    target time is the longer of bytes / copy bandwidth and flops / burst product peak."""
    import numpy as np
    import torch
    from cisr_b200 import StepEntry, Stepper
    from cisr_b200.ops import kernels

    out = {}
    peak_flops = burst_tflops * 1e12 if dtype_bytes == 2 else None
    rng = np.random.default_rng(seed + 3)
    for phase in ("decode", "prefill"):
        if phase == "decode":
            stepper = Stepper(model, n_pages=batch * (-(-context // PAGE_SIZE) + 1), page_size=PAGE_SIZE, max_slots=batch)
            keys = [f"k{i}" for i in range(batch)]
            last = fill_requests(stepper, keys, context - 4, model.spec.vocab_size, seed)
            entries = [StepEntry(k, [last[k]], [0]) for k in keys]
            stepper.step(entries)                                            # warm: libraries loaded, attributes set
            entries = [StepEntry(k, [last[k]], [0]) for k in keys]
            cache_tokens, causal = batch * (context - 2), 0
        else:
            stepper = Stepper(model, n_pages=-(-PREFILL_TOKENS // PAGE_SIZE) + 1, page_size=PAGE_SIZE, max_slots=1)
            ids = rng.integers(0, model.spec.vocab_size, size=PREFILL_TOKENS).tolist()
            stepper.create("p"); stepper.step([StepEntry("p", ids, [PREFILL_TOKENS - 1])]); stepper.release("p")
            stepper.create("p")
            entries = [StepEntry("p", ids, [PREFILL_TOKENS - 1])]
            cache_tokens, causal = 0, PREFILL_TOKENS
        torch.cuda.synchronize()
        # The device first idles for some tens of milliseconds, so that the host has queued the whole step before its
        # first kernel starts: the events then bracket kernels that run back to back, not the host's launch pace.
        torch.cuda._sleep(int(0.06 * 1.9e9))
        with kernels.timed_launches() as timed:
            logits = stepper.step(entries)
            if phase == "decode":
                from cisr_b200.sampling import sample_tokens
                sample_tokens(logits)
        summary = timed.summary()
        step_us = sum(v["us"] for v in summary.values())
        rows = []
        for (name, shape), v in summary.items():
            need_bytes, need_flops, label = kernel_need(name, shape, raw, dtype_bytes, cache_tokens, causal)
            us = v["us"] / v["launches"]
            target_us = need_bytes / (hbm_gbs * 1e9) * 1e6
            bound, achieved, unit = "hbm", need_bytes / us / 1e3, "GB/s"
            if peak_flops and need_flops / peak_flops * 1e6 > target_us:
                target_us, bound, achieved, unit = need_flops / peak_flops * 1e6, "tensor", need_flops / us / 1e6, "TFLOP/s"
            rows.append((v["us"], label, {"launches": v["launches"], "us": round(us, 2), "share_of_step": round(v["us"] / step_us, 3),
                                           "bound": bound, "achieved": round(achieved, 1), "unit": unit,
                                           "frac": round(target_us / us, 4) if us > 0 else None}))
        rows.sort(key=lambda r: -r[0])
        out[phase] = {label: entry for _, label, entry in rows[:top]}
        out[phase + "_sum_us"] = round(step_us, 1)
        del stepper
        torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------ the continuous-batching workload
def mixed_workload(model, raw: dict, layers: int, args, hbm_gbs: float, bf16_tflops: float) -> dict:
    """`--requests` requests with prompts uniform in [128, 2048] and `--new-tokens` generated tokens each, all queued at
    once, through the scheduler with graphs on: portions of prompts under a token budget beside decoding requests."""
    import numpy as np
    import torch
    from cisr_b200 import Engine, Request
    from cisr_b200.ops import kernels

    rng = np.random.default_rng(args.seed + 4)
    lengths = rng.integers(128, 2049, size=args.requests).tolist()
    page = PAGE_SIZE
    life = sum(-(-(n + args.new_tokens) // page) for n in lengths)
    engine = Engine.for_model(model, pages=life + 8, page_size=page, max_active=args.requests, token_budget=args.token_budget,
                              prefill_chunk=args.token_budget, policy="decode_first", graph=True)
    for i, n in enumerate(lengths):
        engine.submit(Request(f"m{i}", rng.integers(0, model.spec.vocab_size, size=n).tolist(), max_new_tokens=args.new_tokens))
    before = dict(kernels.LAUNCHES)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    while engine.tick():
        pass
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    done = list(engine.requests.values())
    assert all(r.status == "finished" and len(r.generated) == args.new_tokens for r in done)
    prompt_tokens, new_tokens = sum(lengths), sum(len(r.generated) for r in done)
    trace = engine.trace
    prefill_s = sum(t["step_s"] for t in trace if t["prefill_tokens"])
    decode_s = sum(t["step_s"] for t in trace if not t["prefill_tokens"])
    # launches: what ran outside graphs, plus every graph's launches once per replay
    graphs = engine.stepper.graphs
    captured = list(graphs.graphs.values()) + list(graphs.shapes.values())
    eager = {k: kernels.LAUNCHES[k] - before[k] - sum(g.launches[k] for g in captured if g.graph is not None) for k in before}
    replayed = {k: sum(g.launches[k] * g.replays for g in captured) for k in before}
    # the least time the run could take: per step every weight once and the live cache, or the products' flops
    per_layer, weight_bytes, kv_per_token = model_bytes_and_flops(raw, layers, 2)
    floor_s = 0.0
    for t in trace:
        need_bytes = weight_bytes + t["resident_pages"] * page * kv_per_token
        need_flops = 2.0 * t["processed_tokens"] * per_layer * layers
        floor_s += max(need_bytes / (hbm_gbs * 1e9), need_flops / (bf16_tflops * 1e12))
    report = graphs.report()
    return {
        "workload": "mixed", "metric": f"tokens/s, continuous batching ({args.preset} shape, {args.requests} requests, prompts 128-2048, "
                                        f"{args.new_tokens} new tokens each)",
        "value": round((prompt_tokens + new_tokens) / seconds, 1), "unit": "tokens/s", "n_gpus": 1, "seconds": round(seconds, 3),
        "steps": len(trace), "higher_is_better": True, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic token ids, seeded random weights",
        "prefill_tokens": prompt_tokens, "decode_tokens": new_tokens,
        "prefill_tok_s": round(prompt_tokens / prefill_s, 1) if prefill_s else None,      # ticks that held a prompt portion (decoding requests ride along)
        "decode_tok_s": round(sum(t["decode_tokens"] for t in trace if not t["prefill_tokens"]) / decode_s, 1) if decode_s else None,
        "ticks_with_prefill": sum(1 for t in trace if t["prefill_tokens"]), "ticks_decode_only": sum(1 for t in trace if not t["prefill_tokens"]),
        "gpu_launches": eager["own"] + replayed["own"], "library_gemm_launches": eager["library"] + replayed["library"],
        "graphs": {"decode_graphs": report["entries"], "shape_graphs": report["shape_entries"], "hits": report["hits"],
                   "misses": report["misses"], "evictions": report["evictions"]},
        "preemptions": sum(r.preemptions for r in done),
        "roofline": {"bound": "per step the longer of bytes / copy bandwidth and product flops / tensor peak",
                     "floor_s": round(floor_s, 4), "frac": round(floor_s / seconds, 4)},
        "config": {"model": args.preset, "requests": args.requests, "new_tokens": args.new_tokens, "token_budget": args.token_budget,
                   "layers": layers, "hidden_size": raw["hidden_size"], "intermediate_size": raw["intermediate_size"],
                   "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"], "head_dim": raw["head_dim"],
                   "vocab_size": raw["vocab_size"], "page_size": page, "policy": "decode_first", "graphs": "on"},
    }


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


REFERENCE_DIR = ROOT / "baseline" / "_ref"        # a plain copy of the reference's tree (it has no setup.py to install from)
REFERENCE_BUDGET_S = 75.0                         # the reference arm times as many of the asked steps as fit into this


def reference_arm(args) -> int:
    """Time the UNMODIFIED reference on the same workload: its stock NumPy path (runtime.backend.Backend() on the CPU,
    float32; its CUDA path needs CuPy, which is not installed), its own Model.step and the decode loop it benchmarks
    itself with (benchmarks/expansion.py:19-39: one token per sequence per step, argmax, fed back).  Nothing of this
    package runs on that path.  Its prefill is one token per step, so reaching the context through it would take tens of
    minutes; instead every layer's PagedCache is filled through its own create/append with seeded random keys and
    values, outside the timed region."""
    import numpy as np

    source = Path(os.environ.get("CISR_REFERENCE_DIR", REFERENCE_DIR))
    if not (source / "runtime" / "model.py").exists():
        print(json.dumps({"impl": "reference", "unavailable": f"no copy of the reference's tree under {source.relative_to(ROOT) if source.is_relative_to(ROOT) else source}"}))
        return 0
    raw = json.loads((ROOT / "cuda-inference-serving-runtime_b200" / "config" / "presets" / f"{args.preset}.json").read_text())
    full_layers = raw["num_hidden_layers"]
    layers = min(args.layers, full_layers) if args.layers else full_layers
    if raw["hidden_size"] // raw["num_attention_heads"] != raw["head_dim"]:
        print(json.dumps({"impl": "reference", "unavailable": "the reference fixes head_dim = hidden_size / heads (runtime/model.py:35)"}))
        return 0
    sys.path.insert(0, str(source))
    try:
        from runtime.backend import Backend
        from runtime.model import Config, Model, toy_weights
    except Exception as err:      # a missing dependency of the reference itself
        print(json.dumps({"impl": "reference", "unavailable": f"the reference does not import here: {err!r}"[:300]}))
        return 0
    config = Config(vocab_size=raw["vocab_size"], hidden_size=raw["hidden_size"], intermediate_size=raw["intermediate_size"],
                    num_hidden_layers=layers, num_attention_heads=raw["num_attention_heads"],
                    num_key_value_heads=raw["num_key_value_heads"], rms_norm_eps=raw["rms_norm_eps"], rope_theta=raw["rope_theta"],
                    max_position_embeddings=raw["max_position_embeddings"])
    backend = Backend()                                                    # device cpu, float32: its defaults
    weights = toy_weights(config, seed=args.seed)                          # the reference's own random weights
    if raw.get("tie_word_embeddings"):
        weights["lm_head.weight"] = weights["model.embed_tokens.weight"]   # as its checkpoint loader ties them (runtime/checkpoint.py:38-39)
    batch, page = args.batch, args.page_size
    model = Model(backend, config, weights, pages=batch * (-(-args.context // page) + 1), page_size=page)
    keys = [f"r{i}" for i in range(batch)]
    rng = np.random.default_rng(args.seed)
    warmup = max(args.warmup, 3)

    def fill(upto: int):
        hkv, dim = config.num_key_value_heads, config.dim
        for key in keys:
            have = model.caches[0].lengths[key]
            for cache in model.caches:
                k = rng.standard_normal((upto - have, hkv, dim), dtype=np.float32)
                v = rng.standard_normal((upto - have, hkv, dim), dtype=np.float32)
                for t in range(upto - have):
                    cache.append(key, k[t], v[t])

    def decode(steps: int, previous):
        for _ in range(steps):
            logits = model.step(previous, keys)                            # host token ids in
            previous = backend.numpy(model.xp.argmax(logits, axis=-1)).tolist()   # host token ids out
            backend.sync()
        return previous

    for key in keys:
        model.create(key)
    # one step at the full context first, to learn what a step costs and how many fit the budget
    probe_ctx = args.context - 2
    fill(probe_ctx - 1)
    previous = rng.integers(0, config.vocab_size, size=batch).tolist()
    t0 = time.perf_counter()
    previous = decode(1, previous)
    probe_s = time.perf_counter() - t0
    steps = max(1, min(args.steps, int(REFERENCE_BUDGET_S / probe_s) - warmup))
    # now the measurement proper, ending at the same context as the other arm: release, refill, warm up, time
    for key in keys:
        model.release(key); model.create(key)
    fill(args.context - steps - warmup - 1)
    previous = decode(warmup, previous)
    t0 = time.perf_counter()
    decode(steps, previous)
    seconds = time.perf_counter() - t0
    final_ctx = model.caches[0].lengths[keys[0]]
    value = batch * steps / seconds
    line = {
        "impl": "reference",
        "metric": "decode tok/s (SmolLM2-135M shape, batch 8, context 4096)" if args.preset == "smollm2-135m" else f"decode tok/s ({args.preset})",
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "steps_asked": args.steps, "warmup": warmup,
        "ms_per_step": round(seconds / steps * 1e3, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32", "device": "cpu", "data": "synthetic token ids, the reference's own seeded random weights (toy_weights)",
        "cache_fill": "PagedCache.append with seeded random keys and values, untimed",
        "config": {"model": args.preset, "global_batch": batch, "seq_len": args.context, "parallelism": "single-gpu",
                   "layers": layers, "layers_of_preset": full_layers, "hidden_size": raw["hidden_size"],
                   "intermediate_size": raw["intermediate_size"], "heads": raw["num_attention_heads"],
                   "kv_heads": raw["num_key_value_heads"], "head_dim": raw["head_dim"], "vocab_size": raw["vocab_size"],
                   "page_size": page, "final_context": final_ctx,
                   "decode": "Model.step + argmax per step (benchmarks/expansion.py:19-39), NumPy on the CPU",
                   "steps_timed": f"{steps} of {args.steps} asked: a step takes {probe_s:.2f} s and the arm keeps to {REFERENCE_BUDGET_S:.0f} s"},
        # the loop above is already end to end: token ids go in and come out as host lists every step, and on this path
        # nothing crosses to a device
        "e2e": {"value": round(value, 2), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "note": "CPU path: inputs and outputs never leave the host"},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
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
    parser.add_argument("--workload", choices=["decode", "mixed"], default="decode",
                        help="mixed: continuous batching through the scheduler (its default shape is smollm2-1.7b)")
    parser.add_argument("--requests", type=int, default=64, help="--workload mixed: number of requests")
    parser.add_argument("--new-tokens", type=int, default=256, help="--workload mixed: tokens generated per request")
    parser.add_argument("--token-budget", type=int, default=2048, help="--workload mixed: tokens per step")
    parser.add_argument("--no-kernels", action="store_true", help="skip the per-kernel figures")
    args = parser.parse_args()
    if args.workload == "mixed" and "--preset" not in " ".join(sys.argv):
        args.preset = "smollm2-1.7b"

    if args.impl == "reference":
        if args.gpus != 1:
            print(json.dumps({"impl": "reference", "unavailable": "the reference runs on one device"}))
            return 0
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine is single-GPU by design (--gpus {args.gpus} is not run)")
        return 2
    args.warmup = max(args.warmup, 3)
    global PAGE_SIZE
    PAGE_SIZE = args.page_size

    import torch

    hbm_gbs, bf16_tflops, bf16_burst, peak_source = peaks()
    model, raw, full_layers = make_model(args)
    layers = raw["num_hidden_layers"]
    dtype_bytes = 2 if args.dtype == "bfloat16" else 4

    if args.timeline:
        return decode_timeline(model, args.batch, args.context, args.seed, args.timeline)
    if args.workload == "mixed":
        sampler = ClockSampler().start()
        line = mixed_workload(model, raw, layers, args, hbm_gbs, bf16_tflops)
        line["clocks"] = sampler.stop()
        line["config"]["peaks"] = peak_source
        print(json.dumps(line))
        return 0
    if args.only == "prefill":
        ms = prefill_run(model, PREFILL_TOKENS, args.seed, reps=2, profile=True)
        print(json.dumps({"only": "prefill", "tokens": PREFILL_TOKENS, "ms": round(ms, 3)}))
        return 0
    if args.only == "decode":
        d = device_decode(model, args.batch, args.context, args.steps, args.warmup, args.seed, min_seconds=0.0)
        print(json.dumps({"only": "decode", "value": round(d["value"], 1), "ms_per_step": round(d["ms_per_step"], 4),
                          "launches_per_step": d["launches"]}))
        return 0
    sampler = ClockSampler().start()
    d = device_decode(model, args.batch, args.context, args.steps, args.warmup, args.seed)
    clocks = sampler.stop()
    value, ms_per_step, launches = d["value"], d["ms_per_step"], d["launches"]
    e2e, h2d, d2h = entry_point_decode(model, args.batch, args.context, min(args.steps, 128), args.warmup, args.seed)
    prefill_ms = prefill_run(model, PREFILL_TOKENS, args.seed)
    points = {}
    if not args.no_points:
        for b in (1, 64):
            point = device_decode(model, b, args.context, min(args.steps, 128), args.warmup, args.seed)
            points[f"decode_b{b}"] = round(point["value"], 1)
            points[f"decode_b{b}_ms_per_step"] = round(point["ms_per_step"], 4)
            points[f"decode_b{b}_own_launches_per_step"] = point["launches"]["own"]
            points[f"decode_b{b}_library_gemm_launches_per_step"] = point["launches"]["library"]

    _, weight_bytes, kv_per_token = model_bytes_and_flops(raw, layers, dtype_bytes)
    step_bytes = weight_bytes + args.batch * d["mean_ctx"] * kv_per_token
    achieved_gbs = step_bytes / (ms_per_step / 1e3) / 1e9
    flops = prefill_flops(raw, layers, PREFILL_TOKENS)
    if args.dtype == "bfloat16":
        peak_flops, fp32_peak = bf16_tflops * 1e12, None
    else:
        fp32_peak = measure_fp32_peak()
        peak_flops = fp32_peak * 1e12
    shape = args.preset.replace("smollm2", "SmolLM2").replace("llama", "Llama").replace("135m", "135M").replace("1.7b", "1.7B").replace("8b", "8B")
    line = {
        "metric": f"decode tok/s ({shape} shape, batch {args.batch}, context {args.context})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4), "ms_per_step_spread": [round(x, 4) for x in d["spread"]], "windows": d["windows"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic token ids, seeded random weights",
        "config": {"model": args.preset, "global_batch": args.batch, "seq_len": args.context, "parallelism": "single-gpu",
                   "layers": layers, "layers_of_preset": full_layers, "hidden_size": raw["hidden_size"],
                   "intermediate_size": raw["intermediate_size"], "heads": raw["num_attention_heads"],
                   "kv_heads": raw["num_key_value_heads"], "head_dim": raw["head_dim"], "vocab_size": raw["vocab_size"],
                   "page_size": PAGE_SIZE, "decode": "cuda graph, tokens fed back on device", "peaks": peak_source,
                   "l2": "inputs larger than L2 (weights + cache per step), no flush",
                   "timing": f"median of {d['windows']} windows of {args.steps} steps (at least {MIN_TIMED_SECONDS} s timed), CUDA events",
                   "mean_context_timed": round(d["mean_ctx"], 1)},
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
    if fp32_peak is not None:
        line["config"]["fp32_peak_tflops"] = round(fp32_peak, 1)
    if not args.no_kernels:
        line["kernels"] = kernel_rooflines(model, raw, args.batch, args.context, args.seed, dtype_bytes, hbm_gbs, bf16_burst)
    if "decode_b1" in points:
        line["decode_b1_vs_published"] = round(points["decode_b1"] / PUBLISHED_DECODE_B1_TOKS, 1)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
