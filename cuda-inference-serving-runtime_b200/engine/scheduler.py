"""Continuous batching: admission, prompt portions under a token budget, decoding,
finishing and freeing.

Parity: runtime/engine.py:13-122 (`Request`, `Engine.submit/cancel/tick/run`, the
policies serial / chunked / decode_first, rotation for fairness, admission by full
page reservation, greedy choice, the per-tick trace).  Differences: a prompt portion
is one multi-token forward pass instead of `prefill_chunk` one-token steps; one tick
is one step of the model; logits are computed only where a token is chosen; sampling
may use a temperature; and a second reservation mode ("lazy") is offered.

What happens when pages run out
-------------------------------
reserve="full" (default, the reference's rule): a request is admitted only when the
pages of its whole life (prompt + max_new_tokens - 1 tokens) fit beside what earlier
admissions reserved, so a running request can never lack a page; requests that do not
fit yet wait, later smaller ones may pass them; a request that could never fit is
refused at `submit`.
reserve="lazy": a request is admitted when its prompt fits into the pages free now.
If a step then finds too few pages, the most recently admitted running request is
preempted: its pages are freed, it returns to the head of the queue, and when it
runs again it recomputes its prompt and the tokens it had generated (which it keeps).
The step is retried without it.  A single running request always fits (checked at
`submit`), so this terminates.
"""
from __future__ import annotations

import math
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple, Union

from ..cache import OutOfPages
from .batch import StepEntry

POLICIES = ("serial", "chunked", "decode_first")
RESERVE_MODES = ("full", "lazy")


@dataclass
class Request:
    key: str
    prompt: list
    max_new_tokens: int = 16
    eos_token_id: Union[int, Sequence[int], None] = None
    arrival_s: float = 0.0
    temperature: float = 0.0
    seed: int = 0
    generated: list = field(default_factory=list)
    cursor: int = 0                      # tokens of prompt + generated that are in the cache
    status: str = "waiting"              # waiting | prefill | decode | finished | cancelled
    submitted_at: float = 0.0
    first_token_at: Optional[float] = None
    token_times: list = field(default_factory=list)
    finished_at: Optional[float] = None
    preemptions: int = 0

    def tokens(self) -> list:
        return self.prompt + self.generated

    def eos_ids(self) -> tuple:
        if self.eos_token_id is None:
            return ()
        if isinstance(self.eos_token_id, int):
            return (self.eos_token_id,)
        return tuple(self.eos_token_id)


class Engine:
    """Scheduler above a step function.

    `stepper` gives `.cache` (the cache manager), `.create/.release` and `.step(entries, extra)`;
    `choose(logits, requests)` returns one token per logits row.  `Engine.for_model` wires the
    real ones; tests of the decisions pass host-only stand-ins.
    """

    def __init__(self, stepper, choose: Callable, vocab_size: int, max_positions: int, max_active: int = 8,
                 token_budget: int = 32, prefill_chunk: int = 8, policy: str = "chunked", reserve: str = "full",
                 lookahead: bool = False):
        if min(max_active, token_budget, prefill_chunk) <= 0:
            raise ValueError("invalid scheduler limits")
        if policy not in POLICIES:
            raise ValueError(f"invalid policy {policy!r}; choose from {POLICIES}")
        if reserve not in RESERVE_MODES:
            raise ValueError(f"invalid reserve mode {reserve!r}; choose from {RESERVE_MODES}")
        self.stepper, self.choose = stepper, choose
        self.vocab_size, self.max_positions = vocab_size, max_positions
        self.max_active = 1 if policy == "serial" else max_active
        self.token_budget, self.prefill_chunk, self.policy, self.reserve = token_budget, prefill_chunk, policy, reserve
        self.lookahead = lookahead
        self.waiting: deque = deque()
        self.active: List[Request] = []
        self.requests = {}
        self.reserved = {}
        self.trace: List[dict] = []
        self.start = time.perf_counter()
        self.rotation = 0
        self._deferred = None      # (requests, device tokens, began): a decode step whose chosen tokens are not read yet

    @classmethod
    def for_model(cls, model, pages: int = 128, page_size: int = 16, max_active: int = 8, token_budget: int = 32,
                  prefill_chunk: int = 8, policy: str = "chunked", reserve: str = "full", graph: bool = False) -> "Engine":
        from ..sampling import DeviceSampler
        from .step import Stepper

        stepper = Stepper(model, n_pages=pages, page_size=page_size, max_slots=max(max_active, 1), graph=graph)
        sampler = DeviceSampler(stepper)
        return cls(stepper, sampler, model.spec.vocab_size, model.spec.max_positions, max_active, token_budget,
                   prefill_chunk, policy, reserve, lookahead=graph)

    # ---------------------------------------------------------------- page arithmetic
    @property
    def _page_size(self) -> int:
        return self.stepper.cache.page_size

    def _pool_pages(self) -> int:
        groups = self.stepper.cache.page_groups
        return min(g.pool.n_pages for g in groups) if groups else 1 << 30

    def _free_pages(self) -> int:
        groups = self.stepper.cache.page_groups
        return min(g.pool.n_free for g in groups) if groups else 1 << 30

    def _resident_pages(self) -> int:
        groups = self.stepper.cache.page_groups
        return max(g.pool.n_used for g in groups) if groups else 0

    def _life_pages(self, r: Request) -> int:
        # the last token chosen is never fed back, so it needs no place in the cache
        return math.ceil((len(r.prompt) + max(0, r.max_new_tokens - 1)) / self._page_size)

    # ---------------------------------------------------------------- requests
    def submit(self, request: Request) -> None:
        r = request
        if r.key in self.requests:
            raise ValueError("duplicate request ID")
        if not r.prompt or r.max_new_tokens < 0 or r.arrival_s < 0:
            raise ValueError("invalid request")
        if r.status != "waiting" or r.cursor or r.generated:
            raise ValueError("request already used")
        if any(t < 0 or t >= self.vocab_size for t in r.prompt):
            raise ValueError("invalid prompt token")
        if r.temperature < 0:
            raise ValueError("temperature must not be negative")
        if len(r.prompt) + max(0, r.max_new_tokens - 1) > self.max_positions:
            raise ValueError("request exceeds context limit")
        if self._life_pages(r) > self._pool_pages():
            raise ValueError("request cannot fit in page pool")
        r.submitted_at = self.start + r.arrival_s
        self.requests[r.key] = r
        self.waiting.append(r)

    def _finish(self, r: Request, status: str = "finished") -> None:
        if r in self.active:
            self.stepper.release(r.key)   # pages go back at once; later steps follow on the same stream
            self.reserved.pop(r.key, None)
            self.active.remove(r)
        r.status = status
        r.finished_at = time.perf_counter()

    def cancel(self, key) -> None:
        r = self.requests[key]
        if r.status in ("finished", "cancelled"):
            return
        if r in self.waiting:
            self.waiting.remove(r)
        self._finish(r, "cancelled")

    def _admit(self) -> None:
        if self.reserve == "full":
            available = self._pool_pages() - sum(self.reserved.values())
        else:
            available = self._free_pages()
        # scan the whole queue: a large request does not block smaller ones behind it
        for r in list(self.waiting):
            if len(self.active) >= self.max_active:
                break
            if time.perf_counter() < r.submitted_at:
                continue
            if self.reserve == "full":
                pages = self._life_pages(r)
            else:
                pages = math.ceil(len(r.tokens()) / self._page_size)
            if pages > available:
                continue
            self.waiting.remove(r)
            if r.max_new_tokens == 0:
                self._finish(r)
                continue
            self.stepper.create(r.key)
            self.reserved[r.key] = pages
            available -= pages
            r.status = "prefill"
            self.active.append(r)

    def _preempt(self, r: Request) -> None:
        self.stepper.release(r.key)
        self.reserved.pop(r.key, None)
        self.active.remove(r)
        r.cursor = 0
        r.status = "waiting"
        r.preemptions += 1
        self.waiting.appendleft(r)

    # ---------------------------------------------------------------- one step
    def _plan(self) -> List[Tuple[Request, int]]:
        """(request, number of its next tokens) for this step, within the token budget."""
        order = self.active[self.rotation:] + self.active[:self.rotation]
        self.rotation = (self.rotation + 1) % max(1, len(self.active))
        if self.policy == "decode_first":
            order.sort(key=lambda r: r.status != "decode")
        remaining = self.token_budget
        plan = []
        for r in order:
            if remaining <= 0:
                break
            pending = len(r.prompt) + len(r.generated) - r.cursor
            n = 1 if r.status == "decode" else min(pending, self.prefill_chunk, remaining)
            plan.append((r, n))
            remaining -= n
        return plan

    def _staged(self, tokens):
        """The last step's tokens as a handle whose read does not wait for later steps, where the stepper offers one."""
        stage = getattr(self.stepper, "stage_last_tokens", None)
        return stage() if stage is not None else tokens

    def _tick_deferred(self) -> bool:
        """Finish a decode step whose tokens were left on the device, launching the step after it first when nothing
        about the batch can change in between: the device feeds its own tokens back, so the host's read of step k
        overlaps step k + 1.  A request that ends at step k (EOS) has then run one step too many, whose token is dropped."""
        reqs, tokens_dev, began = self._deferred
        self._deferred = None
        ahead = None
        stable = (not self.waiting and len(reqs) == len(self.active) and all(r in self.active for r in reqs)
                  and all(len(r.generated) + 2 <= r.max_new_tokens for r in reqs))
        if stable and self.stepper.can_run_ahead():
            try:
                if getattr(self.stepper, "stage_last_tokens", None) is not None:
                    ahead = self._staged(None) if self.stepper.decode_ahead(1, history=False) == 1 else None
                else:
                    ran = self.stepper.decode_ahead(1)
                    ahead = ran[0] if ran.shape[0] == 1 else None
            except OutOfPages:
                ahead = None
        # waits for step k only: its copy to the host was queued before step k + 1
        if hasattr(tokens_dev, "read"):
            chosen = tokens_dev.read()                 # checks the kernels' error flag as of that step, too
        else:
            chosen = tokens_dev.to("cpu").tolist()
            self.stepper.check_kernels()
        completed = time.perf_counter()
        decoded = 0
        for r, token in zip(reqs, chosen):
            if r not in self.active or r.status != "decode":
                continue                               # ended or cancelled since the step was launched
            r.cursor += 1
            decoded += 1
            r.generated.append(int(token))
            r.token_times.append(completed)
            if len(r.generated) >= r.max_new_tokens or int(token) in r.eos_ids():
                self._finish(r)
        self.trace.append({"elapsed_s": time.perf_counter() - self.start, "step_s": time.perf_counter() - began,
                           "processed_tokens": decoded, "prefill_tokens": 0, "decode_tokens": decoded,
                           "active": len(self.active), "resident_pages": self._resident_pages()})
        if ahead is not None:
            self._deferred = (reqs, ahead, completed)
        return bool(self.active or self.waiting or self._deferred)

    def tick(self) -> bool:
        if self._deferred is not None:
            return self._tick_deferred()
        self._admit()
        if not self.active:
            return bool(self.waiting)
        began = time.perf_counter()
        while True:
            plan = self._plan()
            entries = []
            for r, n in plan:
                tokens = r.tokens()
                last = r.cursor + n == len(tokens)
                entries.append(StepEntry(r.key, tokens[r.cursor:r.cursor + n], [n - 1] if last else []))
            choosing = [r for (r, n), e in zip(plan, entries) if e.want]
            try:
                logits = self.stepper.step(entries, extra=self._sampling_arrays(choosing))
                break
            except OutOfPages:
                if self.reserve != "lazy" or len(self.active) <= 1:
                    raise
                self._preempt(self.active[-1])
        can_ahead = getattr(self.stepper, "can_run_ahead", None)
        if (self.lookahead and can_ahead is not None and can_ahead() and len(choosing) == len(plan)
                and all(r.status == "decode" for r in choosing)):
            # a pure decode step from a graph: leave its tokens on the device until the next tick
            self._deferred = (list(choosing), self._staged(self.stepper.last_tokens), began)
            return True
        chosen = self.choose(logits, choosing) if choosing else []
        check = getattr(self.stepper, "check_kernels", None)
        if check is not None:
            check()        # after the read of the chosen tokens synchronised the device
        completed = time.perf_counter()
        prefilled = decoded = 0
        for (r, n), e in zip(plan, entries):
            r.cursor += n
            if r.status == "decode":
                decoded += n
            else:
                prefilled += n
        for r, token in zip(choosing, chosen):
            r.status = "decode"
            r.generated.append(int(token))
            r.token_times.append(completed)
            if r.first_token_at is None:
                r.first_token_at = completed
            if len(r.generated) >= r.max_new_tokens or int(token) in r.eos_ids():
                self._finish(r)
        self.trace.append({"elapsed_s": time.perf_counter() - self.start, "step_s": time.perf_counter() - began,
                           "processed_tokens": prefilled + decoded, "prefill_tokens": prefilled,
                           "decode_tokens": decoded, "active": len(self.active),
                           "resident_pages": self._resident_pages()})
        return bool(self.active or self.waiting)

    @staticmethod
    def _sampling_arrays(choosing: List[Request]):
        import numpy as np

        if not choosing or all(r.temperature <= 0 for r in choosing):
            return None
        return {"temperature": np.asarray([r.temperature for r in choosing], dtype=np.float32),
                "seed": np.asarray([r.seed for r in choosing], dtype=np.int64),
                "counter": np.asarray([len(r.generated) for r in choosing], dtype=np.int32)}

    def run(self) -> List[Request]:
        while self.tick():
            if not self.active and self.waiting:
                delay = min(r.submitted_at for r in self.waiting) - time.perf_counter()
                if delay > 0:
                    time.sleep(min(delay, 0.01))
        return list(self.requests.values())
