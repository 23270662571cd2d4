"""The step function: one batch of (request, its next tokens) through the model.

`Stepper.step` runs only the tokens it is given, as one batch, against the cache that
earlier steps left, and returns float logits at the wanted places.  Portions of
prompts and single decoded tokens may be mixed freely; a prompt may be cut anywhere.

Parity: runtime/model.py:86-120 (`Model.step`: validate, preflight the pages, run,
return logits) and runtime/execution.py:102-129 (lengths advance only after the work
is enqueued).  The reference takes exactly one token per sequence per step and returns
logits for every row; here a request brings any number of tokens and names the rows.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager
from ..ops import kernels
from .batch import HostBatch, PinnedRing, StepContext, StepEntry, build_context
from .model import Model


def validate_entries(cache: CacheManager, entries: Sequence[StepEntry], vocab_size: int) -> None:
    if not entries:
        raise ValueError("a step needs at least one entry")
    keys = [e.key for e in entries]
    if len(set(keys)) != len(keys):
        raise ValueError("a request may appear once in a step")
    for e in entries:
        if e.key not in cache.requests:
            raise KeyError(f"unknown sequence {e.key!r}")
        if len(e.tokens) == 0:
            raise ValueError(f"entry of {e.key!r} brings no tokens")
        if any(t < 0 or t >= vocab_size for t in e.tokens):
            raise ValueError(f"token out of range in entry of {e.key!r}")
        if any(w < 0 or w >= len(e.tokens) for w in e.want):
            raise ValueError(f"wanted place outside the tokens of entry {e.key!r}")


def run_page_copies(cache: CacheManager, device) -> None:
    """Copy-on-write of shared, partly filled pages queued by `reserve`, for every entry of a group at once."""
    for g in cache.page_groups:
        copies = cache.drain_copies(g.index)
        if copies:
            pairs = torch.tensor(copies, dtype=torch.int32, device=device)
            page_bytes = g.page_bytes()
            kernels.page_copy(g.storage, pairs, g.storage.shape[0] * 2, g.pool.n_pages * page_bytes, page_bytes)


def prepare_step(cache: CacheManager, ring: PinnedRing, device, entries: Sequence[StepEntry], vocab_size: int,
                 extra: Optional[Dict[str, np.ndarray]] = None, shape_graphs=None, planners: Sequence = ()):
    """Validate a batch, reserve its pages (all or nothing), send its metadata and bring the device's block
    tables up to date.  Returns (context, device views of `extra`, graph or None).  Lengths advance in `commit_step`.

    With `shape_graphs`, a step whose shape has a captured graph gets its metadata into that graph's buffers and
    leaves the table updates to the graph.  `planners`: the parts whose launch plans are packed into the same copy."""
    validate_entries(cache, entries, vocab_size)
    keys = [e.key for e in entries]
    cache.reserve([(e.key, len(e.tokens)) for e in entries])   # raises before any change

    slots, q_start, q_len, ctx_len, logit_rows = [], [], [], [], []
    token_ids, positions, token_req = [], [], []
    total = 0
    for r, e in enumerate(entries):
        n = len(e.tokens)
        start = cache.length(e.key)
        slots.append(cache.slot(e.key)); q_start.append(total); q_len.append(n); ctx_len.append(start + n)
        token_ids.extend(int(t) for t in e.tokens)
        positions.extend(range(start, start + n))
        token_req.extend([r] * n)
        logit_rows.extend(total + int(w) for w in e.want)
        total += n
    host = HostBatch(keys, slots, q_start, q_len, ctx_len, total, logit_rows)
    graph = None
    if shape_graphs is not None:
        decode_ctx = max((c for n, c in zip(q_len, ctx_len) if n == 1), default=0)
        graph = shape_graphs.shape(tuple(q_len), len(logit_rows), decode_ctx)
    updates = []
    for g in cache.page_groups:
        idx, val = cache.drain_table_updates(g.index)
        if graph is not None and idx.size > graph.static.update_capacity:      # more than the graph's list holds: apply now
            kernels.table_update(g.device_table, torch.from_numpy(idx).to(device), torch.from_numpy(val).to(device))
            idx, val = idx[:0], val[:0]
        updates.append((idx, val))
    ctx, update_views, extras = build_context(
        device, ring, host, np.asarray(token_ids, dtype=np.int32), np.asarray(positions, dtype=np.int32),
        np.asarray(token_req, dtype=np.int32), updates, extra, static=graph.static if graph is not None else None,
        planners=planners)
    if graph is None:
        for g, (idx, val) in zip(cache.page_groups, update_views):
            if idx.numel():
                kernels.table_update(g.device_table, idx, val)
    run_page_copies(cache, device)
    ctx.update_views = update_views
    return ctx, extras, graph


def commit_step(cache: CacheManager, entries: Sequence[StepEntry]) -> None:
    for e in entries:
        cache.commit(e.key, len(e.tokens))


class StagedTokens:
    """Sampled tokens on their way to pinned host memory; read() waits for that copy only."""

    def __init__(self, pinned: torch.Tensor, event: "torch.cuda.Event", n: int, status_at: int):
        self.pinned, self.event, self.n, self.status_at = pinned, event, n, status_at

    def read(self) -> List[int]:
        self.event.synchronize()
        kernels.raise_for_code(int(self.pinned[self.status_at]))
        return self.pinned[:self.n].tolist()


class Stepper:
    """`graph=True` replays steps made only of single new tokens from captured CUDA graphs (see engine/graph.py);
    it is ignored when a mixer of the model reads the step through host values."""

    def __init__(self, model: Model, n_pages: int, page_size: int = 16, max_slots: int = 64, graph: bool = False):
        if not model.loaded:
            raise RuntimeError("the model has no weights yet")
        self.model = model
        self.max_slots = max_slots
        self.cache: CacheManager = model.make_cache(n_pages, page_size, max_slots)
        self.ring = PinnedRing()
        self.planners = model.planners()
        self.last_context: Optional[StepContext] = None
        self.last_extras: Dict[str, torch.Tensor] = {}
        self.last_tokens: Optional[torch.Tensor] = None     # tokens a graph step sampled itself
        self._last_graph = None                             # the graph whose buffer `last_tokens` views, if it does
        self._stage_slots = None                            # pinned buffers and events for stage_last_tokens
        self._copy_stream = None                            # where staged copies run
        self._stage_next = 0
        self.graphs = None
        if graph and all(layer.mixer.graph_safe for layer in model.layers):
            from .graph import DecodeGraphs
            self.graphs = DecodeGraphs(self)
        self._ahead = None

    # requests -------------------------------------------------------------
    def create(self, key) -> None:
        self.cache.create(key)

    def release(self, key) -> None:
        self.cache.release(key)

    def fork(self, source, target) -> None:
        self.cache.fork(source, target)

    @staticmethod
    def check_kernels() -> None:
        """Raise if a kernel reported that it gave up on a bounded wait (reads a device flag: synchronises)."""
        kernels.raise_if_kernel_gave_up()

    # the step ---------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], extra: Optional[Dict[str, np.ndarray]] = None) -> torch.Tensor:
        """Float logits [number of wanted places, vocab], in the order of the entries and of their `want`."""
        self._ahead = None
        if self.graphs is not None and entries and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
            return self._graph_step(entries, extra)
        ctx, extras, graph = prepare_step(self.cache, self.ring, self.model.device, entries, self.model.spec.vocab_size,
                                          extra, shape_graphs=self.graphs, planners=self.planners)
        if graph is not None:
            logits = graph.run(ctx, ctx.update_views)
        else:
            logits = self.model.forward(ctx, self.cache)
        commit_step(self.cache, entries)
        self.last_context, self.last_extras, self.last_tokens = ctx, extras, None
        return logits

    def _flush_tables(self, limit: int):
        """Pending block-table changes per group; those beyond `limit` entries are applied at once."""
        device = self.model.device
        out = []
        for g in self.cache.page_groups:
            idx, val = self.cache.drain_table_updates(g.index)
            if idx.size > limit:
                kernels.table_update(g.device_table, torch.from_numpy(idx).to(device), torch.from_numpy(val).to(device))
                idx, val = idx[:0], val[:0]
            out.append((idx, val))
        run_page_copies(self.cache, device)
        return out

    def _graph_step(self, entries: Sequence[StepEntry], extra) -> torch.Tensor:
        cache = self.cache
        validate_entries(cache, entries, self.model.spec.vocab_size)
        cache.reserve([(e.key, 1) for e in entries])
        n = len(entries)
        slots = [cache.slot(e.key) for e in entries]
        positions = [cache.length(e.key) for e in entries]
        graph, fresh = self.graphs.get(n, max(positions) + 1)
        updates = self._flush_tables(graph.n_updates)
        extra = extra or {}
        graph.fill(slots, [int(e.tokens[0]) for e in entries], positions, extra.get("temperature", 0.0),
                   extra.get("seed", 0), extra.get("counter", 0), updates)
        graph.upload()
        if fresh:
            graph.capture(warm_up=self.graphs.first_of_its_rows(graph))
        self._before_replay(graph)
        graph.replay()
        commit_step(cache, entries)
        self.last_context, self.last_extras = None, {}
        self.last_tokens = graph.tokens[:n].clone()       # a later replay overwrites the graph's own buffer
        self._last_graph = None
        self._ahead = (graph, [e.key for e in entries])
        return graph.logits[:n]

    def decode_ahead(self, steps: int, history: bool = True) -> Optional[torch.Tensor]:
        """Run up to `steps` more decode steps of the batch of the last step without the host in between.

        Each step feeds every request the token the step before sampled for it (on the device).  Valid only
        right after a step that ran from a graph; stops early at the graph's context limit.  Pages for all
        the steps are reserved first, all or nothing.  Returns the sampled tokens, int32 [steps run, requests];
        with history=False nothing is kept but the last step's tokens (`last_tokens`, a view of the graph's own
        buffer that the next replay overwrites: stage or copy it before), and the return value is the number of steps.
        """
        if self._ahead is None:
            raise RuntimeError("decode_ahead follows a step of single tokens that ran from a CUDA graph")
        graph, keys = self._ahead
        cache = self.cache
        longest = max(cache.length(k) for k in keys)
        steps = min(steps, graph.ctx_bucket - longest, self.model.spec.max_positions - longest)
        device = self.model.device
        if steps <= 0:
            return torch.empty((0, len(keys)), dtype=torch.int32, device=device) if history else 0
        cache.reserve([(k, steps) for k in keys])
        # new pages reach the device through the graph's own update lists (a pinned copy that does not wait for the step
        # in flight); applying the same list again in the later replays of this call changes nothing
        graph.upload_updates(self._flush_tables(graph.n_updates))
        kept = torch.empty((steps, graph.rows), dtype=torch.int32, device=device) if history else None
        for i in range(steps):
            self._before_replay(graph)
            graph.replay()
            if kept is not None:
                kept[i].copy_(graph.tokens, non_blocking=True)
        for k in keys:
            cache.commit(k, steps)
        if kept is None:
            self.last_tokens = graph.tokens[:len(keys)]
            self._last_graph = graph
            return steps
        self.last_tokens = kept[steps - 1, :len(keys)]
        self._last_graph = None
        return kept[:, :len(keys)]

    def can_run_ahead(self) -> bool:
        return self._ahead is not None

    def _before_replay(self, graph) -> None:
        """The coming replay writes the ring slot that the replay RING_SLOTS before it wrote: a staged copy out of that
        slot must have run.  It has, steps ago, unless the host ran that far ahead of its own reads."""
        from .graph import RING_SLOTS
        copies = graph.slot_copies
        while copies and graph.replays - copies[0][0] >= RING_SLOTS:
            number, event = copies.popleft()
            if not event.query():
                torch.cuda.current_stream().wait_event(event)

    def stage_last_tokens(self) -> "StagedTokens":
        """Queue the copy of the last step's sampled tokens to pinned host memory right behind that step.

        Reading the returned handle waits for that copy alone, not for steps queued after it, so the host can look at
        step k's tokens while step k + 1 runs."""
        if self.last_tokens is None:
            raise RuntimeError("the last step did not sample its tokens on the device")
        if self._stage_slots is None:
            self._stage_slots = [(torch.zeros(2 * self.max_slots + 2, dtype=torch.int32, pin_memory=True), torch.cuda.Event())
                                 for _ in range(4)]
        pinned, event = self._stage_slots[self._stage_next]
        self._stage_next = (self._stage_next + 1) % len(self._stage_slots)
        n = self.last_tokens.numel()
        graph = self._last_graph
        # The copy runs on a stream of its own, behind an event that marks the end of the step: the next step on the
        # main stream then starts without waiting for the copy engine.
        main = torch.cuda.current_stream()
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream()
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(self._copy_stream):
            self._copy_stream.wait_event(done)
            if graph is not None:
                # the ring slot that step wrote: its tokens, then the kernels' error flag as of that step.  Later
                # replays write other slots, so nothing on the main stream has to wait for this copy.
                pinned[:graph.rows + 1].copy_(graph.last_slot(), non_blocking=True)
                status_at = graph.rows
                graph.slot_copies.append((graph.replays - 1, event))
            else:
                pinned[:n].copy_(self.last_tokens, non_blocking=True)
                flag = kernels.error_flag_tensor()      # the kernels' "gave up on a wait" flag travels with the tokens
                if flag is not None:
                    pinned[n:n + 1].copy_(flag, non_blocking=True)
                else:
                    pinned[n] = 0
                status_at = n
            event.record(self._copy_stream)
        return StagedTokens(pinned, event, n, status_at)
