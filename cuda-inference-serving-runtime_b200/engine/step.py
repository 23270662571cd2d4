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

from typing import Dict, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager
from ..ops import kernels
from .batch import HostBatch, PinnedRing, StepContext, StepEntry, build_context
from .model import Model


def prepare_step(cache: CacheManager, ring: PinnedRing, device, entries: Sequence[StepEntry], vocab_size: int,
                 extra: Optional[Dict[str, np.ndarray]] = None):
    """Validate a batch, reserve its pages (all or nothing), send its metadata and bring the device's block
    tables up to date.  Returns (context, device views of `extra`).  Lengths advance in `commit_step`."""
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
    updates = [cache.drain_table_updates(g.index) for g in cache.page_groups]
    ctx, update_views, extras = build_context(
        device, ring, host, np.asarray(token_ids, dtype=np.int32), np.asarray(positions, dtype=np.int32),
        np.asarray(token_req, dtype=np.int32), updates, extra)
    for g, (idx, val) in zip(cache.page_groups, update_views):
        if idx.numel():
            kernels.table_update(g.device_table, idx, val)
        copies = cache.drain_copies(g.index)
        if copies:   # copy-on-write of shared, partly filled pages, for every entry of the group at once
            pairs = torch.tensor(copies, dtype=torch.int32, device=device)
            page_bytes = g.page_bytes()
            kernels.page_copy(g.storage, pairs, g.storage.shape[0] * 2, g.pool.n_pages * page_bytes, page_bytes)
    return ctx, extras


def commit_step(cache: CacheManager, entries: Sequence[StepEntry]) -> None:
    for e in entries:
        cache.commit(e.key, len(e.tokens))


class Stepper:
    def __init__(self, model: Model, n_pages: int, page_size: int = 16, max_slots: int = 64):
        if not model.loaded:
            raise RuntimeError("the model has no weights yet")
        self.model = model
        self.cache: CacheManager = model.make_cache(n_pages, page_size, max_slots)
        self.ring = PinnedRing()
        self.last_context: Optional[StepContext] = None
        self.last_extras: Dict[str, torch.Tensor] = {}

    # requests -------------------------------------------------------------
    def create(self, key) -> None:
        self.cache.create(key)

    def release(self, key) -> None:
        self.cache.release(key)

    def fork(self, source, target) -> None:
        self.cache.fork(source, target)

    # the step ---------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], extra: Optional[Dict[str, np.ndarray]] = None) -> torch.Tensor:
        """Float logits [number of wanted places, vocab], in the order of the entries and of their `want`."""
        ctx, extras = prepare_step(self.cache, self.ring, self.model.device, entries, self.model.spec.vocab_size, extra)
        logits = self.model.forward(ctx, self.cache)
        commit_step(self.cache, entries)
        self.last_context, self.last_extras = ctx, extras
        return logits
