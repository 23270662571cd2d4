"""The cache manager: paged keys and values with a block table per request, and
fixed-size per-request state slots.

Run entries of the model are sorted into groups by what their mixer needs
(`CacheUse.group_key()`): all entries that keep every key with the same geometry share
one page pool and one block table per request; entries that keep a window of keys form
another group with pages of their own, and give a page back as soon as the window has
passed it; entries with fixed-size state get a tensor [slots, ...] each.  A page id
means the same page in every entry of its group, so one allocation serves all of them.

Every live request holds one slot.  The slot indexes the request's row in each
group's block table on the device and its row in every state tensor.  Block tables
live on the device as [slots, width] int32 and are kept up to date by sending only
the entries that changed (`drain_table_updates`).

Parity: runtime/cache.py:9-118 (create, fork, copy-on-write of a shared partial page,
atomic failure, release, invariants, report).  Unlike the reference (one allocator per
layer, runtime/model.py:66-67) there is one allocator per group, and lengths are
committed by the caller after the step is enqueued (runtime/execution.py:125-126).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..config.spec import CacheUse
from .pages import OutOfPages, PagePool


@dataclass
class PagedBinding:
    """What a paged mixer sees of the cache for one run entry."""
    k: torch.Tensor              # [pages, kv_heads, page_size, head_dim]
    v: torch.Tensor
    block_table: torch.Tensor    # [slots, width] int32 on the device
    page_size: int
    write: bool                  # False: the entry reads another entry's pages
    window: Optional[int]


@dataclass
class StateBinding:
    """What a stateful mixer sees: its tensor [slots, ...]; rows are picked by the step's request slots."""
    state: torch.Tensor


@dataclass
class _Request:
    slot: int
    length: int = 0
    tables: Dict[int, List[int]] = field(default_factory=dict)   # group index -> logical page -> physical page or -1
    first_live: Dict[int, int] = field(default_factory=dict)     # group index -> first logical page still held


class PageGroup:
    def __init__(self, index: int, use: CacheUse, entries: List[int], n_pages: int, page_size: int, max_slots: int,
                 width: int, dtype: torch.dtype, device):
        self.index, self.use, self.entries = index, use, entries
        self.page_size, self.width = page_size, width
        self.pool = PagePool(n_pages)
        self.entry_slot = {e: i for i, e in enumerate(entries)}
        self.storage = None
        self.device_table = None
        if device is not None:
            # [entries, key|value, pages, kv_heads, page_size, head_dim]
            self.storage = torch.zeros((len(entries), 2, n_pages, use.kv_heads, page_size, use.head_dim), dtype=dtype,
                                       device=device)
            self.device_table = torch.full((max_slots + 1, width), -1, dtype=torch.int32, device=device)   # last row: the null slot
        self.host_table = np.full((max_slots, width), -1, dtype=np.int32)
        self.updates: List[Tuple[int, int]] = []   # (flat index into the table, page id)
        self.copies: List[Tuple[int, int]] = []    # (source page, destination page) to run before the next step

    def set_entry(self, slot: int, logical: int, page: int) -> None:
        self.host_table[slot, logical] = page
        self.updates.append((slot * self.width + logical, page))

    def page_bytes(self) -> int:
        return self.use.kv_heads * self.page_size * self.use.head_dim * self.storage.element_size()


class StateGroup:
    def __init__(self, index: int, use: CacheUse, entries: List[int], max_slots: int, device):
        self.index, self.use, self.entries = index, use, entries
        self.entry_slot = {e: i for i, e in enumerate(entries)}
        self.storage = None
        if device is not None:
            self.storage = torch.zeros((len(entries), max_slots + 1) + tuple(use.state_shape),
                                       dtype=getattr(torch, use.state_dtype), device=device)


class CacheManager:
    """Owns every page pool, block table and state slot of one model instance.

    `uses[i]` is the `CacheUse` of run entry i, or the index of the earlier entry whose
    cache entry i reads.  `n_pages` pages of `page_size` tokens are given to each page
    group.  With `device=None` only the host bookkeeping exists (tests of the allocator).
    """

    def __init__(self, uses: Sequence, n_pages: int, page_size: int, max_slots: int, max_positions: int,
                 dtype: torch.dtype = torch.float32, device=None):
        if n_pages <= 0 or page_size <= 0 or max_slots <= 0:
            raise ValueError("cache dimensions must be positive")
        self.page_size, self.max_slots, self.max_positions = page_size, max_slots, max_positions
        self.width = -(-max_positions // page_size)
        self.device, self.dtype = device, dtype
        self.page_groups: List[PageGroup] = []
        self.state_groups: List[StateGroup] = []
        self.entry_group: Dict[int, Tuple[str, int]] = {}   # run entry -> ("pages"|"state", group index)
        self.entry_source: Dict[int, int] = {}              # run entry -> entry whose storage it uses
        by_key: Dict[tuple, List[int]] = {}
        for entry, use in enumerate(uses):
            if isinstance(use, int):
                self.entry_source[entry] = use
                continue
            self.entry_source[entry] = entry
            if use.kind != "none":
                by_key.setdefault(use.group_key(), []).append(entry)
        for key, entries in by_key.items():
            use = uses[entries[0]]
            if use.kind == "pages":
                group = PageGroup(len(self.page_groups), use, entries, n_pages, page_size, max_slots, self.width, dtype, device)
                self.page_groups.append(group)
                for e in entries:
                    self.entry_group[e] = ("pages", group.index)
            elif use.kind == "state":
                group = StateGroup(len(self.state_groups), use, entries, max_slots, device)
                self.state_groups.append(group)
                for e in entries:
                    self.entry_group[e] = ("state", group.index)
            else:
                raise ValueError(f"unknown cache use {use.kind!r}")
        self.requests: Dict[object, _Request] = {}
        self.free_slots: List[int] = list(reversed(range(max_slots)))

    @property
    def null_slot(self) -> int:
        """A slot no request ever holds: its block table row stays empty.  Padding rows of a fixed-size batch point here."""
        return self.max_slots

    # ---------------------------------------------------------------- requests
    def create(self, key) -> int:
        if key in self.requests:
            raise ValueError(f"duplicate sequence {key!r}")
        if not self.free_slots:
            raise OutOfPages(f"all {self.max_slots} request slots are in use")
        slot = self.free_slots.pop()
        req = _Request(slot)
        for g in self.page_groups:
            req.tables[g.index] = []
            req.first_live[g.index] = 0
        for g in self.state_groups:
            if g.storage is not None:
                g.storage[:, slot].zero_()
        self.requests[key] = req
        return slot

    def fork(self, source, target) -> int:
        """`target` starts as a copy of `source`, sharing its pages (copied only when written)."""
        if target in self.requests:
            raise ValueError(f"duplicate sequence {target!r}")
        src = self.requests[source]
        if not self.free_slots:
            raise OutOfPages(f"all {self.max_slots} request slots are in use")
        slot = self.free_slots.pop()
        req = _Request(slot, src.length)
        for g in self.page_groups:
            table = list(src.tables[g.index])
            req.tables[g.index] = table
            req.first_live[g.index] = src.first_live[g.index]
            for logical, page in enumerate(table):
                if page >= 0:
                    g.pool.retain(page)
                    g.set_entry(slot, logical, page)
        for g in self.state_groups:
            if g.storage is not None:
                g.storage[:, slot].copy_(g.storage[:, src.slot])
        self.requests[target] = req
        return slot

    def length(self, key) -> int:
        return self.requests[key].length

    def slot(self, key) -> int:
        return self.requests[key].slot

    def pages_needed(self, key, n_tokens: int) -> int:
        """Pages `reserve` would take from each full-attention group for n_tokens more tokens (worst group)."""
        req = self.requests[key]
        need = 0
        for g in self.page_groups:
            need = max(need, self._plan(req, g, n_tokens)[0])
        return need

    def _plan(self, req: _Request, g: PageGroup, n_tokens: int) -> Tuple[int, bool]:
        table = req.tables[g.index]
        new_pages = max(0, -(-(req.length + n_tokens) // g.page_size) - len(table))
        cow = False
        if n_tokens > 0 and req.length % g.page_size and table and table[-1] >= 0 and g.pool.refs[table[-1]] > 1:
            cow = True   # the partly filled last page is shared: it is copied before it is written
        return new_pages + (1 if cow else 0), cow

    def reserve(self, portions: Sequence[Tuple[object, int]]) -> None:
        """Make room for `n_tokens` more tokens of each request, all or nothing.

        New pages go into the block tables (and onto the update list for the device);
        a shared, partly filled last page is replaced by a private copy (the copy is
        queued in `group.copies`).  Lengths are not changed: call `commit` once the
        step is enqueued.
        """
        for key, n_tokens in portions:
            req = self.requests[key]
            if n_tokens < 0 or req.length + n_tokens > self.max_positions:
                raise ValueError(f"sequence {key!r} would exceed the context limit of {self.max_positions}")
        for g in self.page_groups:
            need = sum(self._plan(self.requests[key], g, n)[0] for key, n in portions)
            if need > g.pool.n_free:
                raise OutOfPages(f"insufficient KV pages for step: {need} wanted, {g.pool.n_free} free "
                                 f"of {g.pool.n_pages} (group {g.index})")
        for g in self.page_groups:
            for key, n_tokens in portions:
                req = self.requests[key]
                count, cow = self._plan(req, g, n_tokens)
                pages = g.pool.allocate(count)
                table = req.tables[g.index]
                if cow:
                    fresh = pages.pop()
                    old = table[-1]
                    g.copies.append((old, fresh))
                    g.pool.release(old)
                    table[-1] = fresh
                    g.set_entry(req.slot, len(table) - 1, fresh)
                for page in pages:
                    table.append(page)
                    g.set_entry(req.slot, len(table) - 1, page)

    def commit(self, key, n_tokens: int) -> None:
        """The step that wrote `n_tokens` more tokens is enqueued: advance the length, give back passed pages."""
        req = self.requests[key]
        req.length += n_tokens
        for g in self.page_groups:
            if g.use.window is None:
                continue
            # the next query sits at position `length` and sees keys > length - window
            dead = max(0, (req.length - g.use.window + 1) // g.page_size)
            table = req.tables[g.index]
            for logical in range(req.first_live[g.index], min(dead, len(table))):
                if table[logical] >= 0:
                    g.pool.release(table[logical])
                    table[logical] = -1
                    g.set_entry(req.slot, logical, -1)
            req.first_live[g.index] = max(req.first_live[g.index], min(dead, len(table)))

    def release(self, key) -> None:
        """The request is over: every page it holds goes back (to be used again), its slot too.

        No device synchronisation is needed: later steps run on the same stream, after
        the kernels that read these pages.
        """
        req = self.requests.pop(key)
        for g in self.page_groups:
            for logical, page in enumerate(req.tables[g.index]):
                if page >= 0:
                    g.pool.release(page)
                    g.set_entry(req.slot, logical, -1)
        self.free_slots.append(req.slot)

    # ---------------------------------------------------------------- device side
    def drain_table_updates(self, group_index: int) -> Tuple[np.ndarray, np.ndarray]:
        g = self.page_groups[group_index]
        if not g.updates:
            return np.zeros(0, np.int32), np.zeros(0, np.int32)
        last = dict(g.updates)   # one value per table entry: the scatter on the device runs in no fixed order
        idx = np.fromiter(last.keys(), dtype=np.int32, count=len(last))
        val = np.fromiter(last.values(), dtype=np.int32, count=len(last))
        g.updates.clear()
        return idx, val

    def drain_copies(self, group_index: int) -> List[Tuple[int, int]]:
        g = self.page_groups[group_index]
        copies, g.copies = g.copies, []
        return copies

    def binding(self, entry: int, reads_from: Optional[int] = None):
        """The cache view of run entry `entry` (or of the entry it reads from)."""
        source = entry if reads_from is None else reads_from
        kind_group = self.entry_group.get(source)
        if kind_group is None:
            return None
        kind, gi = kind_group
        if kind == "pages":
            g = self.page_groups[gi]
            e = g.entry_slot[source]
            return PagedBinding(g.storage[e, 0], g.storage[e, 1], g.device_table, g.page_size,
                                write=reads_from is None, window=g.use.window)
        g = self.state_groups[gi]
        return StateBinding(g.storage[g.entry_slot[source]])

    # ---------------------------------------------------------------- checks and reports
    def check(self) -> None:
        """No page lost, held twice or freed twice; host tables and lengths are consistent."""
        for g in self.page_groups:
            g.pool.check(req.tables[g.index] for req in self.requests.values())
            for key, req in self.requests.items():
                table = req.tables[g.index]
                if len(table) < -(-req.length // g.page_size):
                    raise AssertionError(f"sequence {key!r} holds fewer pages than its length needs")
                row = g.host_table[req.slot]
                if list(row[: len(table)]) != table or (row[len(table):] != -1).any():
                    raise AssertionError(f"block table row of {key!r} disagrees with its page list")
                for logical, page in enumerate(table):
                    live = g.use.window is None or (logical + 1) * g.page_size > req.length - g.use.window + 1
                    if live and logical * g.page_size < req.length and page < 0:
                        raise AssertionError(f"sequence {key!r} lost page {logical} that it still needs")
        slots = [req.slot for req in self.requests.values()]
        if len(slots) != len(set(slots)) or set(slots) & set(self.free_slots):
            raise AssertionError("a request slot is held twice")
        if len(slots) + len(self.free_slots) != self.max_slots or len(set(self.free_slots)) != len(self.free_slots):
            raise AssertionError("a request slot was lost or freed twice")
        live_slots = set(slots)
        for g in self.page_groups:
            for slot in range(self.max_slots):
                if slot not in live_slots and (g.host_table[slot] != -1).any():
                    raise AssertionError(f"slot {slot} is free but its block table row is not empty")

    def report(self) -> dict:
        out = {"sequences": len(self.requests), "free_slots": len(self.free_slots), "groups": []}
        for g in self.page_groups:
            out["groups"].append({
                "kind": "pages", "window": g.use.window, "entries": len(g.entries), "pages": g.pool.n_pages,
                "resident_pages": g.pool.n_used, "free_pages": g.pool.n_free, "peak_pages": g.pool.peak,
                "shared_pages": int(np.count_nonzero(g.pool.refs > 1)),
                "pool_bytes": 0 if g.storage is None else g.storage.numel() * g.storage.element_size()})
        for g in self.state_groups:
            out["groups"].append({"kind": "state", "entries": len(g.entries), "shape": tuple(g.use.state_shape),
                                  "bytes": 0 if g.storage is None else g.storage.numel() * g.storage.element_size()})
        return out
