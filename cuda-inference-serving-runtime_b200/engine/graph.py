"""Decode steps replayed from captured CUDA graphs.

A step in which every request brings exactly one token and wants its logits has a
fixed shape once the batch is padded to a bucket size, so the whole step (table
updates, embedding, every layer, final norm, head, sampling, and the feed-back of the
sampled tokens) is captured once per (batch bucket, context bucket) and replayed with
new contents in fixed buffers.

Parity: runtime/execution.py:1-6,24-61,102-129 (`ModelProgram`: one program per batch
size, inputs rebound by content into stable buffers, replay instead of recapture, an
LRU of programs).  Differences: padding rows point at a null slot whose block table is
empty, so warm-up and padding never touch a live page (the reference saves and restores
KV slot 0 around its warm-up, runtime/execution.py:49-59); sampling is inside the graph;
after a replay the graph's own buffers already hold the next step's inputs, so several
steps can run back to back without the host (`run_ahead`).
"""
from __future__ import annotations

import collections
import contextlib
import gc
import os
from collections import OrderedDict
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..ops import kernels
from ..sampling import sample_tokens
from .batch import HostBatch, PlanViews, StepContext, StepEntry

MIN_CONTEXT_BUCKET = 256
RING_SLOTS = 4


@contextlib.contextmanager
def capturing(graph: "torch.cuda.CUDAGraph", pool=None):
    """Capture what runs inside into `graph`, on a stream of its own.  `pool`: the memory pool its buffers come from; the
    graphs of one stepper share one (they replay one after the other on one stream, and each keeps what it returns
    referenced), so a later capture reuses the intermediate buffers of the earlier ones instead of asking the driver
    for its own.

    No automatic garbage collection inside: destroying an older CUDA graph (a captured step of a stepper that is no
    longer referenced, found by a collection that an allocation happens to trigger) is not permitted while a stream is
    capturing and would invalidate the capture.  And none of torch.cuda.graph's housekeeping before it (a full
    collection and an emptied allocator cache per capture: about a tenth of a second with a large cache pool resident,
    which a server pays whenever a new batch or context bucket appears in the middle of its work)."""
    was_enabled = gc.isenabled()
    gc.disable()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    try:
        with torch.cuda.stream(stream):
            graph.capture_begin(pool=pool)
            try:
                yield
            finally:
                graph.capture_end()
        torch.cuda.current_stream().wait_stream(stream)
    finally:
        if was_enabled:
            gc.enable()


def bucket_of(n: int, minimum: int = 1) -> int:
    b = minimum
    while b < n:
        b *= 2
    return b


def context_bucket_of(n: int) -> int:
    """The context bound a decode graph is captured for: powers of two up to 1024, then quarter steps between them
    (1280, 1536, 1792, 2048, 2560, ...), so that at most a fifth of a step's key ranges lie beyond the context."""
    b = bucket_of(n, MIN_CONTEXT_BUCKET)
    if b <= 1024:
        return b
    quarter = b // 8                      # b / 2 < n <= b: steps of a quarter of b / 2
    return b // 2 + -(-(n - b // 2) // quarter) * quarter


def _align(n: int) -> int:
    return (n + 3) & ~3


class DecodeGraph:
    """One captured decode step for `rows` padded rows and contexts up to `ctx_bucket`."""

    def __init__(self, stepper, rows: int, ctx_bucket: int):
        self.stepper, self.rows, self.ctx_bucket = stepper, rows, ctx_bucket
        cache = stepper.cache
        device = stepper.model.device
        self.n_updates = 2 * rows
        names = ["token_ids", "positions", "token_req", "req_slot", "q_start", "q_len", "ctx_len", "logit_rows",
                 "temperature", "counter", "live"]
        sizes = {n: rows for n in names}
        sizes["seed"] = 2 * rows
        names.append("seed")
        # the parts' launch plans for `rows` single tokens with contexts up to the bucket: fixed for the graph's life
        self.plan_host = HostBatch([None] * rows, [cache.null_slot] * rows, list(range(rows)), [1] * rows, [ctx_bucket] * rows,
                                   rows, list(range(rows)), ctx_bound=ctx_bucket)
        self.plans = [(part.plan_key(), i, part.step_plan(self.plan_host)) for i, part in enumerate(stepper.planners)]
        for _, i, plan in self.plans:
            for name, arr in plan.arrays.items():
                sizes[f"plan{i}.{name}"] = max(1, int(np.asarray(arr).size))
                names.append(f"plan{i}.{name}")
        for g in cache.page_groups:
            for kind in ("upd_idx", "upd_val"):
                sizes[f"{kind}{g.index}"] = self.n_updates
                names.append(f"{kind}{g.index}")
        self.offsets: Dict[str, Tuple[int, int]] = {}
        total = 0
        for n in names:
            self.offsets[n] = (total, sizes[n])
            total += _align(sizes[n])
        self.host = torch.zeros(total, dtype=torch.int32, pin_memory=True)
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(total, dtype=torch.int32, device=device)
        arange = np.arange(rows, dtype=np.int32)
        for n in ("token_req", "q_start", "logit_rows"):
            self.h(n)[:] = arange
        self.h("q_len")[:] = 1
        for _, i, plan in self.plans:
            for name, arr in plan.arrays.items():
                self.h(f"plan{i}.{name}")[:np.asarray(arr).size] = np.asarray(arr, dtype=np.int32).reshape(-1)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.pool = None                  # the memory pool to capture into (the owner of the graphs shares one among them)
        self.logits: Optional[torch.Tensor] = None
        self.tokens = torch.zeros(rows, dtype=torch.int32, device=device)
        # every replay also leaves its tokens, and the kernels' error flag, in the next slot of a small ring, so the host
        # can copy step k out while steps k + 1 .. k + RING_SLOTS - 1 run
        self.ring = torch.zeros((RING_SLOTS, rows + 1), dtype=torch.int32, device=device)
        self.step_index = torch.zeros(1, dtype=torch.int32, device=device)
        self.slot_copies = collections.deque()      # (replay number, event) of copies out of ring slots still to be confirmed
        # the update lists are the tail of the buffer; two pinned copies of that tail, used in turn, let a step's lists be
        # written while the copy of the step before may still be on its way
        self.upd_start = min((self.offsets[f"upd_idx{g.index}"][0] for g in cache.page_groups), default=total)
        self.upd_host = [torch.full((total - self.upd_start,), -1, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.upd_sent: List[Optional[torch.cuda.Event]] = [None, None]
        self.upd_turn = 0
        self.sent: Optional[torch.cuda.Event] = None      # the last copy out of `host`
        self.replays = 0
        self.launches = {"own": 0, "library": 0}

    def h(self, name: str) -> np.ndarray:
        start, size = self.offsets[name]
        return self.host_np[start:start + size]

    def d(self, name: str) -> torch.Tensor:
        start, size = self.offsets[name]
        return self.dev[start:start + size]

    def fill(self, slots, tokens, positions, temperature, seed, counter, updates) -> None:
        """Write one step's contents into the pinned buffer (rows beyond the live ones become padding)."""
        n, rows = len(slots), self.rows
        null = self.stepper.cache.null_slot
        if self.sent is not None:
            self.sent.synchronize()      # the copy of the step before must have left the pinned buffer
        self.h("token_ids")[:n] = tokens; self.h("token_ids")[n:] = 0
        self.h("positions")[:n] = positions; self.h("positions")[n:] = 0
        self.h("req_slot")[:n] = slots; self.h("req_slot")[n:] = null
        self.h("ctx_len")[:n] = np.asarray(positions) + 1; self.h("ctx_len")[n:] = 0
        self.h("live")[:n] = 1; self.h("live")[n:] = 0
        self.h("temperature").view(np.float32)[:n] = temperature; self.h("temperature")[n:] = 0
        self.h("seed").view(np.int64)[:n] = seed
        self.h("counter")[:n] = counter; self.h("counter")[n:] = 0
        for g, (idx, val) in zip(self.stepper.cache.page_groups, updates):
            hi, hv = self.h(f"upd_idx{g.index}"), self.h(f"upd_val{g.index}")
            hi[:] = -1
            hi[:idx.size] = idx
            hv[:idx.size] = val

    def upload(self) -> None:
        self.dev.copy_(self.host, non_blocking=True)
        if self.sent is None:
            self.sent = torch.cuda.Event()
        self.sent.record()

    def upload_updates(self, updates) -> None:
        """Send this step's block-table update lists (the rest of the buffer holds what the device fed back to itself)."""
        if self.upd_start >= self.dev.numel():
            return
        self.upd_turn ^= 1
        staging = self.upd_host[self.upd_turn]
        if self.upd_sent[self.upd_turn] is not None:
            self.upd_sent[self.upd_turn].synchronize()     # two copies ago: long done unless the host ran far ahead
        flat = staging.numpy()
        for g, (idx, val) in zip(self.stepper.cache.page_groups, updates):
            a, size = self.offsets[f"upd_idx{g.index}"]
            b, _ = self.offsets[f"upd_val{g.index}"]
            flat[a - self.upd_start:a - self.upd_start + size] = -1
            flat[a - self.upd_start:a - self.upd_start + idx.size] = idx
            flat[b - self.upd_start:b - self.upd_start + idx.size] = val
        self.dev[self.upd_start:].copy_(staging, non_blocking=True)
        if self.upd_sent[self.upd_turn] is None:
            self.upd_sent[self.upd_turn] = torch.cuda.Event()
        self.upd_sent[self.upd_turn].record()

    def _run(self, advance: bool) -> None:
        stepper = self.stepper
        cache, model = stepper.cache, stepper.model
        for g in cache.page_groups:
            kernels.table_update(g.device_table, self.d(f"upd_idx{g.index}"), self.d(f"upd_val{g.index}"))
        ctx = StepContext(model.device, self.plan_host)
        ctx.token_ids, ctx.positions, ctx.token_req = self.d("token_ids"), self.d("positions"), self.d("token_req")
        ctx.req_slot, ctx.q_start, ctx.q_len, ctx.ctx_len = self.d("req_slot"), self.d("q_start"), self.d("q_len"), self.d("ctx_len")
        ctx.logit_rows = self.d("logit_rows")
        for key, i, plan in self.plans:
            ctx.plans[key] = PlanViews({name: self.d(f"plan{i}.{name}")[:np.asarray(arr).size] for name, arr in plan.arrays.items()},
                                       dict(plan.info))
        self.logits = model.forward(ctx, cache)
        sample_tokens(self.logits, self.d("temperature").view(torch.float32), self.d("seed").view(torch.int64),
                      self.d("counter"), out=self.tokens)
        if advance:
            kernels.decode_advance(self.d("token_ids"), self.d("positions"), self.d("ctx_len"), self.d("counter"),
                                   self.tokens, self.d("live"), ring=self.ring, step_index=self.step_index)

    def capture(self, warm_up: bool = True) -> None:
        """Warm up once outside the graph (library set-up, kernel attributes), then capture.  `warm_up=False`: a graph
        for the same number of rows was captured before, so the same kernels have run already."""
        if warm_up:
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                self._run(advance=False)
            torch.cuda.current_stream().wait_stream(stream)
            torch.cuda.synchronize()
        before = dict(kernels.LAUNCHES)
        self.graph = torch.cuda.CUDAGraph()
        pdl = os.environ.get("CISR_PDL", "1") != "0"
        kernels.set_pdl(pdl)        # inside the graph a kernel may fetch its weights while the one before it still runs
        try:
            with capturing(self.graph, self.pool):
                self._run(advance=True)
        finally:
            kernels.set_pdl(False)
        self.launches = {k: kernels.LAUNCHES[k] - before[k] for k in before}   # kernels one replay launches

    def replay(self) -> None:
        self.graph.replay()
        self.replays += 1

    def last_slot(self) -> torch.Tensor:
        """The ring slot the last replay wrote: its tokens, then the kernels' error flag."""
        return self.ring[(self.replays - 1) % RING_SLOTS]


class ShapeGraph:
    """One captured step of a fixed shape: the same portion lengths per request, in the same order, and the same number
    of wanted logit rows.  Portions of prompts repeat their shape whenever prompts are cut by a fixed budget."""

    def __init__(self, stepper, q_lens: Tuple[int, ...], n_rows: int, ctx_bucket: int):
        from .batch import StaticMeta
        cache = stepper.cache
        tokens = sum(q_lens)
        self.stepper = stepper
        capacity = tokens // max(1, cache.page_size) + 2 * len(q_lens) + 8
        # room for the parts' launch plans: their sizes depend on the shape only, so one trial run measures them
        starts = [sum(q_lens[:i]) for i in range(len(q_lens))]
        trial = HostBatch([None] * len(q_lens), [0] * len(q_lens), starts, list(q_lens), [max(ctx_bucket, n) for n in q_lens], tokens,
                          [], ctx_bound=ctx_bucket)
        plan_ints = sum(_align(int(np.asarray(a).size)) for part in stepper.planners for a in part.step_plan(trial).arrays.values())
        ints = 4 * tokens + 8 * len(q_lens) + plan_ints + n_rows * 8 + 2 * capacity * max(1, len(cache.page_groups)) + 256
        self.static = StaticMeta(stepper.model.device, ints, capacity, ctx_bucket)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.pool = None
        self.logits: Optional[torch.Tensor] = None
        self.replays = 0
        self.launches = {"own": 0, "library": 0}

    def _run(self, ctx, update_views) -> None:
        cache, model = self.stepper.cache, self.stepper.model
        ctx.shared.clear()      # what parts share within a step (rotary tables) is computed inside every run, so also inside the graph
        for g, (idx, val) in zip(cache.page_groups, update_views):
            kernels.table_update(g.device_table, idx, val)
        self.logits = model.forward(ctx, cache)

    def run(self, ctx, update_views) -> torch.Tensor:
        """`ctx` and `update_views` view this shape's static buffers, already filled and sent for this step."""
        if self.graph is None:
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                self._run(ctx, update_views)        # warm-up outside the graph; writes the same cache entries the replay will
            torch.cuda.current_stream().wait_stream(stream)
            torch.cuda.synchronize()
            before = dict(kernels.LAUNCHES)
            self.graph = torch.cuda.CUDAGraph()
            kernels.set_pdl(os.environ.get("CISR_PDL", "1") != "0")
            try:
                with capturing(self.graph, self.pool):
                    self._run(ctx, update_views)
            finally:
                kernels.set_pdl(False)
            self.launches = {k: kernels.LAUNCHES[k] - before[k] for k in before}
        self.graph.replay()
        self.replays += 1
        return self.logits


class DecodeGraphs:
    """The graphs of one stepper, kept by (batch bucket, context bucket), least recently used evicted first."""

    def __init__(self, stepper, capacity: int = 8):
        self.stepper, self.capacity = stepper, capacity
        self.graphs: "OrderedDict[Tuple[int, int], DecodeGraph]" = OrderedDict()
        self.shapes: "OrderedDict[tuple, ShapeGraph]" = OrderedDict()
        self.seen: Dict[tuple, int] = {}
        self.hits = self.misses = self.evictions = 0
        self.pool = torch.cuda.graph_pool_handle() if torch.cuda.is_available() else None
        self.warmed_rows: set = set()

    def get(self, n_rows: int, max_ctx: int) -> Tuple[DecodeGraph, bool]:
        key = (bucket_of(n_rows), context_bucket_of(max_ctx))
        graph = self.graphs.get(key)
        if graph is not None:
            self.graphs.move_to_end(key)
            self.hits += 1
            return graph, False
        self.misses += 1
        graph = DecodeGraph(self.stepper, *key)
        graph.pool = self.pool
        self.graphs[key] = graph
        while len(self.graphs) > self.capacity:
            self.graphs.popitem(last=False)
            self.evictions += 1
        return graph, True

    def first_of_its_rows(self, graph: DecodeGraph) -> bool:
        """Whether no graph of this many rows was captured here before (then its kernels have not all run yet, and the
        capture is preceded by a plain run).  Asked once per graph, right before its capture."""
        first = graph.rows not in self.warmed_rows
        self.warmed_rows.add(graph.rows)
        return first

    def shape(self, q_lens: Tuple[int, ...], n_rows: int, max_decode_ctx: int) -> Optional[ShapeGraph]:
        """The graph of a step shape, from the second time the shape is seen (a shape seen once is not worth a capture)."""
        key = (q_lens, n_rows, context_bucket_of(max_decode_ctx) if max_decode_ctx else 0)
        graph = self.shapes.get(key)
        if graph is not None:
            self.shapes.move_to_end(key)
            self.hits += 1
            return graph
        self.seen[key] = self.seen.get(key, 0) + 1
        if self.seen[key] < 2:
            return None
        if len(self.seen) > 4096:
            self.seen.clear()
        self.misses += 1
        graph = ShapeGraph(self.stepper, q_lens, n_rows, key[2])
        graph.pool = self.pool
        self.shapes[key] = graph
        while len(self.shapes) > self.capacity:
            self.shapes.popitem(last=False)
            self.evictions += 1
        return graph

    def report(self) -> dict:
        return {"entries": len(self.graphs), "shape_entries": len(self.shapes), "hits": self.hits, "misses": self.misses, "evictions": self.evictions,
                "replays": {f"{k[0]}x{k[1]}": g.replays for k, g in self.graphs.items()}}
