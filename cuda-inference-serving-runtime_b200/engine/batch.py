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
    # When set: a bound on the ctx_len of every request that brings a single token, which also holds for later steps
    # run with this step's launch plans (a captured graph is replayed with other lengths, up to its context bucket).
    # None or 0: the plans serve this step alone and may use the lengths themselves.
    ctx_bound: Optional[int] = None


@dataclass
class StepPlan:
    """What a part derives on the host from a step's shape before the step runs: int32 lists its kernels read on the
    device (tile lists and the like) and plain numbers for its launches (grid sizes).  A plan may depend on the
    portion lengths `q_len` and their order, and on the lengths of single-token requests only through an upper bound
    (`ctx_bound` when set, else their largest `ctx_len`); never on token values or on the lengths of longer portions,
    so that steps of the same shape share it and a captured step stays right when replayed."""
    arrays: Dict[str, np.ndarray] = field(default_factory=dict)
    info: Dict[str, int] = field(default_factory=dict)


class PlanViews:
    """A `StepPlan` once its lists are on the device: `views[name]` are int32 device tensors, `info` the numbers."""

    def __init__(self, views: Dict[str, torch.Tensor], info: Dict[str, int]):
        self.views, self.info = views, info

    def __getitem__(self, name: str) -> torch.Tensor:
        return self.views[name]


class StepContext:
    """Device-side view of one step, handed to every part.

    It holds only what every mixer needs: the tokens, their positions and requests, per request its slot, first row,
    portion length and length after the step, and the rows whose logits are wanted.  Launch plans of single parts
    (`plan_for`) and values parts share within a step (`shared`: rotary tables) hang beside it under the parts' keys.
    """

    def __init__(self, device, host: HostBatch):
        self.device = device
        self.host = host
        self.n_tokens = host.n_tokens
        self.n_requests = len(host.keys)
        self.shared: Dict[object, object] = {}   # values parts share within a step (rotary tables, ...)
        self.plans: Dict[object, PlanViews] = {}  # launch plans by the parts' plan keys
        self.token_ids = self.positions = self.token_req = None
        self.req_slot = self.q_start = self.q_len = self.ctx_len = None
        self.logit_rows = None

    def plan_for(self, part) -> PlanViews:
        """The launch plan of `part` for this step.  The engine packs the plans of a model's parts into the step's one
        metadata copy; a part run outside that (a test of one part) gets its plan made and sent here."""
        key = part.plan_key()
        views = self.plans.get(key)
        if views is None:
            plan = part.step_plan(self.host)
            views = PlanViews({name: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(self.device)
                               for name, a in plan.arrays.items()}, dict(plan.info))
            self.plans[key] = views
        return views


def unique_planners(parts) -> list:
    """The parts that make launch plans, one per plan key (thirty attention layers of one geometry share one plan)."""
    seen, out = set(), []
    for part in parts:
        key = part.plan_key() if hasattr(part, "plan_key") else None
        if key is not None and key not in seen:
            seen.add(key)
            out.append(part)
    return out


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

    def __init__(self, device, ints: int, update_capacity: int, ctx_bound: int):
        self.pinned = torch.zeros(ints, dtype=torch.int32, pin_memory=True)
        self.dev = torch.zeros(ints, dtype=torch.int32, device=device)
        self.update_capacity = update_capacity
        self.ctx_bound = ctx_bound                  # the context bucket: launch plans made for it stay right at replay
        self.sent: Optional[torch.cuda.Event] = None   # the last copy out of `pinned`

    def wait_until_sent(self) -> None:
        """The pinned buffer is about to be rewritten: the copy of the step before must have left it."""
        if self.sent is not None:
            self.sent.synchronize()

    def mark_sent(self) -> None:
        if self.sent is None:
            self.sent = torch.cuda.Event()
        self.sent.record()


def build_context(device, ring: PinnedRing, host: HostBatch, token_ids: np.ndarray, positions: np.ndarray,
                  token_req: np.ndarray, table_updates: Sequence[Tuple[np.ndarray, np.ndarray]],
                  extra: Optional[Dict[str, np.ndarray]] = None, static: Optional[StaticMeta] = None,
                  planners: Sequence = ()):
    """Pack the step's metadata, send it in one copy, and return (context, update views, extra views).

    `planners`: parts whose launch plans (`part.step_plan(host)`) travel in the same copy.
    With `static`, the metadata goes into that shape's fixed buffers instead of fresh ones."""
    if static is not None:
        host.ctx_bound = static.ctx_bound
    segments: List[Tuple[str, np.ndarray]] = [
        ("token_ids", token_ids), ("positions", positions), ("token_req", token_req),
        ("req_slot", np.asarray(host.slots, dtype=np.int32)), ("q_start", np.asarray(host.q_start, dtype=np.int32)),
        ("q_len", np.asarray(host.q_len, dtype=np.int32)), ("ctx_len", np.asarray(host.ctx_len, dtype=np.int32)),
        ("logit_rows", np.asarray(host.logit_rows, dtype=np.int32)),
    ]
    plans = []
    for i, part in enumerate(planners):
        plan = part.step_plan(host)
        plans.append((part.plan_key(), i, plan))
        for name, arr in plan.arrays.items():
            segments.append((f"plan{i}.{name}", np.ascontiguousarray(arr, dtype=np.int32).reshape(-1)))
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
        static.wait_until_sent()
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
    else:
        static.mark_sent()

    def view(name: str) -> torch.Tensor:
        start, size = offsets[name]
        return dev[start:start + size]

    ctx = StepContext(device, host)
    ctx.token_ids, ctx.positions, ctx.token_req = view("token_ids"), view("positions"), view("token_req")
    ctx.req_slot, ctx.q_start, ctx.q_len, ctx.ctx_len = view("req_slot"), view("q_start"), view("q_len"), view("ctx_len")
    ctx.logit_rows = view("logit_rows")
    for key, i, plan in plans:
        ctx.plans[key] = PlanViews({name: view(f"plan{i}.{name}") for name in plan.arrays}, dict(plan.info))
    updates = [(view(f"upd_idx{g}"), view(f"upd_val{g}")) for g in range(len(table_updates))]
    extras = {name: view(name) for name in (extra or {})}
    return ctx, updates, extras
