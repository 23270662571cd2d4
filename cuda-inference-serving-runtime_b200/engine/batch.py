"""One step's batch: what the host knows and what the kernels read.

A step is a list of entries (request, its next tokens, the places whose logits are
wanted).  Portions of prompts and single decoded tokens sit side by side in one flat
token batch.  All integer metadata of the step is packed into one pinned host buffer
and reaches the device in one copy; `StepContext` holds views into the device copy.

Parity: the reference builds five arrays per step (tokens, positions, lengths, tables,
slots; runtime/execution.py:106-117) for one token per sequence.  Here a request brings
any number of tokens, tables stay on the device, and only changed table entries travel.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..ops import kernels

CTA_TARGET = 444           # three CTAs per SM on a 148-SM part: what the decode split aims to fill
SPLIT_QUANTUM = 64         # key ranges of the split are multiples of this
SPLIT_MIN = 256            # a CTA's four warps each take tiles of up to 64 keys: a shorter range leaves warps idle
CLUSTER_MAX = 16           # key ranges of one request and head that one thread-block cluster can merge


@dataclass
class StepEntry:
    key: object
    tokens: Sequence[int]
    want: Sequence[int] = ()          # indices into `tokens` whose logits are returned


@dataclass
class HostBatch:
    """The step as plain Python numbers, for bookkeeping and for parts written in torch."""
    keys: List[object]
    slots: List[int]
    q_start: List[int]
    q_len: List[int]
    ctx_len: List[int]                # length of each request after this step
    n_tokens: int
    logit_rows: List[int]


class StepContext:
    """Device-side view of one step, handed to every part."""

    def __init__(self, device, host: HostBatch):
        self.device = device
        self.host = host
        self.n_tokens = host.n_tokens
        self.n_requests = len(host.keys)
        self.shared: Dict[object, object] = {}   # values parts share within a step (rotary tables, ...)
        self.token_ids = self.positions = self.token_req = None
        self.req_slot = self.q_start = self.q_len = self.ctx_len = None
        self.tile_req = self.tile_q0 = self.dec_req = None
        self.wide_req = self.wide_q0 = None      # the same portions cut into tiles of kernels.WIDE_TILE queries
        self.n_tiles = self.n_wide = self.n_decode = 0
        self.logit_rows = None
        self.max_decode_ctx = 0
        self.fixed_splits: Optional[Tuple[int, int]] = None

    def decode_splits(self, kv_heads: int) -> Tuple[int, int]:
        """(keys per range, number of ranges) for the split decode attention of this step.

        Ranges start at multiples of the range size in absolute positions, so which keys
        fall together does not depend on the batch; the range size is chosen to give the
        device about three CTAs per SM, and up to 16 ranges are merged inside one thread-block cluster.
        """
        if self.fixed_splits is not None:
            return self.fixed_splits
        return plan_decode_splits(self.n_decode, kv_heads, self.max_decode_ctx)


def plan_decode_splits(n_decode: int, kv_heads: int, max_ctx: int) -> Tuple[int, int]:
    ctas = max(1, n_decode * kv_heads)
    wanted = max(1, CTA_TARGET // ctas)          # rounded down: one wave of CTAs, not a wave and a bit
    size = -(-max(1, max_ctx) // wanted)
    size = max(SPLIT_MIN, -(-size // SPLIT_QUANTUM) * SPLIT_QUANTUM)
    n_splits = max(1, -(-max_ctx // size))
    if n_splits > CLUSTER_MAX:       # whole clusters: the ranges beyond the context are empty
        n_splits = -(-n_splits // CLUSTER_MAX) * CLUSTER_MAX
    return size, n_splits


class PinnedRing:
    """A few pinned host buffers used in turn; a buffer is reused only after its copy has finished."""

    def __init__(self, count: int = 4, ints: int = 1 << 16):
        self.buffers = [torch.empty(ints, dtype=torch.int32, pin_memory=True) for _ in range(count)]
        self.events: List[Optional[torch.cuda.Event]] = [None] * count
        self.next = 0

    def take(self, ints: int) -> Tuple[torch.Tensor, int]:
        i = self.next
        self.next = (self.next + 1) % len(self.buffers)
        if self.events[i] is not None:
            self.events[i].synchronize()
        if self.buffers[i].numel() < ints:
            self.buffers[i] = torch.empty(max(ints, 2 * self.buffers[i].numel()), dtype=torch.int32, pin_memory=True)
        return self.buffers[i], i

    def sent(self, i: int) -> None:
        event = torch.cuda.Event()
        event.record()
        self.events[i] = event


def _align(n: int) -> int:
    return (n + 3) & ~3


class StaticMeta:
    """Fixed host and device buffers for the metadata of steps of one shape (the inputs of a captured graph).

    Block-table updates are padded to `update_capacity` entries per group (index -1: no change), so a step of the
    same shape always has the same layout; the caller applies what does not fit before packing.
    """

    def __init__(self, device, ints: int, update_capacity: int, max_decode_ctx: int):
        self.pinned = torch.zeros(ints, dtype=torch.int32, pin_memory=True)
        self.dev = torch.zeros(ints, dtype=torch.int32, device=device)
        self.update_capacity = update_capacity
        self.max_decode_ctx = max_decode_ctx        # an upper bound (the bucket), so the decode split plan is fixed


def build_context(device, ring: PinnedRing, host: HostBatch, token_ids: np.ndarray, positions: np.ndarray,
                  token_req: np.ndarray, table_updates: Sequence[Tuple[np.ndarray, np.ndarray]],
                  extra: Optional[Dict[str, np.ndarray]] = None, static: Optional[StaticMeta] = None):
    """Pack the step's metadata, send it in one copy, and return (context, update views, extra views).

    With `static`, the metadata goes into that shape's fixed buffers instead of fresh ones."""
    q_len = np.asarray(host.q_len, dtype=np.int32)
    tile = kernels.PREFILL_TILE
    tile_req: List[int] = []
    tile_q0: List[int] = []
    wide_req: List[int] = []
    wide_q0: List[int] = []
    dec_req: List[int] = []
    max_decode_ctx = 0
    for r, n in enumerate(host.q_len):
        if n == 1:
            dec_req.append(r)
            max_decode_ctx = max(max_decode_ctx, host.ctx_len[r])
        else:
            for q0 in reversed(range(0, n, tile)):     # a portion's last tile has the longest key loop: launch it first
                tile_req.append(r)
                tile_q0.append(q0)
            for q0 in reversed(range(0, n, kernels.WIDE_TILE)):
                wide_req.append(r)
                wide_q0.append(q0)
    segments: List[Tuple[str, np.ndarray]] = [
        ("token_ids", token_ids), ("positions", positions), ("token_req", token_req),
        ("req_slot", np.asarray(host.slots, dtype=np.int32)), ("q_start", np.asarray(host.q_start, dtype=np.int32)),
        ("q_len", q_len), ("ctx_len", np.asarray(host.ctx_len, dtype=np.int32)),
        ("tile_req", np.asarray(tile_req, dtype=np.int32)), ("tile_q0", np.asarray(tile_q0, dtype=np.int32)),
        ("wide_req", np.asarray(wide_req, dtype=np.int32)), ("wide_q0", np.asarray(wide_q0, dtype=np.int32)),
        ("dec_req", np.asarray(dec_req, dtype=np.int32)), ("logit_rows", np.asarray(host.logit_rows, dtype=np.int32)),
    ]
    for g, (idx, val) in enumerate(table_updates):
        if static is not None:
            padded_idx = np.full(static.update_capacity, -1, dtype=np.int32)
            padded_val = np.zeros(static.update_capacity, dtype=np.int32)
            padded_idx[:idx.size] = idx
            padded_val[:val.size] = val
            idx, val = padded_idx, padded_val
        segments.append((f"upd_idx{g}", idx))
        segments.append((f"upd_val{g}", val))
    for name, arr in (extra or {}).items():
        segments.append((name, np.ascontiguousarray(arr).view(np.int32).reshape(-1)))
    offsets = {}
    total = 0
    for name, arr in segments:
        offsets[name] = (total, arr.size)
        total += _align(arr.size)
    total = max(total, 4)
    if static is not None:
        if total > static.pinned.numel():
            raise ValueError("the step's metadata does not fit the buffers of its shape")
        pinned, dev = static.pinned, static.dev
    else:
        pinned, ring_index = ring.take(total)
        dev = torch.empty(total, dtype=torch.int32, device=device)
    flat = pinned.numpy()
    for name, arr in segments:
        start, size = offsets[name]
        flat[start:start + size] = arr
    dev[:total].copy_(pinned[:total], non_blocking=True)
    if static is None:
        ring.sent(ring_index)

    def view(name: str) -> torch.Tensor:
        start, size = offsets[name]
        return dev[start:start + size]

    ctx = StepContext(device, host)
    ctx.token_ids, ctx.positions, ctx.token_req = view("token_ids"), view("positions"), view("token_req")
    ctx.req_slot, ctx.q_start, ctx.q_len, ctx.ctx_len = view("req_slot"), view("q_start"), view("q_len"), view("ctx_len")
    ctx.tile_req, ctx.tile_q0, ctx.dec_req = view("tile_req"), view("tile_q0"), view("dec_req")
    ctx.wide_req, ctx.wide_q0 = view("wide_req"), view("wide_q0")
    ctx.n_tiles, ctx.n_wide, ctx.n_decode = len(tile_req), len(wide_req), len(dec_req)
    ctx.logit_rows = view("logit_rows")
    ctx.max_decode_ctx = max_decode_ctx if static is None else max(static.max_decode_ctx, max_decode_ctx)
    updates = [(view(f"upd_idx{g}"), view(f"upd_val{g}")) for g in range(len(table_updates))]
    extras = {name: view(name) for name in (extra or {})}
    return ctx, updates, extras
