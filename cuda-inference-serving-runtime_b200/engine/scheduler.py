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
ENDED = ("finished", "cancelled")


@dataclass(eq=False)                     # a request is itself, not its fields: membership tests and removals go by identity
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

    def life_tokens(self) -> int:
        """Tokens the request holds in the cache at most: its prompt and all it generates but the last token."""
        return len(self.prompt) + max(0, self.max_new_tokens - 1)

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

    def _pools(self):
        return [g.pool for g in self.stepper.cache.page_groups]

    def _pool_pages(self) -> int:
        return min((pool.n_pages for pool in self._pools()), default=1 << 30)

    def _free_pages(self) -> int:
        return min((pool.n_free for pool in self._pools()), default=1 << 30)

    def _resident_pages(self) -> int:
        return max((pool.n_used for pool in self._pools()), default=0)

    def _pages_for(self, tokens: int) -> int:
        return math.ceil(tokens / self._page_size)

    def _life_pages(self, r: Request) -> int:
        """Pages of a request's whole life.  The last token chosen is never fed back, so it needs no place in the cache
        (runtime/engine.py:46-47)."""
        return self._pages_for(r.life_tokens())

    # ---------------------------------------------------------------- requests
    def _problems(self, r: Request) -> List[str]:
        """Everything that is wrong with a request, all at once (the checks of runtime/engine.py:40-48, one more for
        the temperature)."""
        found = []
        if r.key in self.requests:
            found.append(f"duplicate request ID {r.key!r}")
        if not r.prompt or r.max_new_tokens < 0 or r.arrival_s < 0:
            found.append("invalid request (it needs a prompt, max_new_tokens >= 0 and arrival_s >= 0)")
        if r.status != "waiting" or r.cursor or r.generated:
            found.append("request already used")
        bad = [t for t in r.prompt if not 0 <= t < self.vocab_size]
        if bad:
            found.append(f"invalid prompt token {bad[0]} (vocabulary of {self.vocab_size})")
        if r.temperature < 0:
            found.append("temperature must not be negative")
        if r.life_tokens() > self.max_positions:
            found.append(f"request exceeds context limit of {self.max_positions}")
        elif self._life_pages(r) > self._pool_pages():
            found.append(f"request cannot fit in page pool ({self._life_pages(r)} pages wanted, {self._pool_pages()} exist)")
        return found

    def submit(self, request: Request) -> None:
        problems = self._problems(request)
        if problems:
            raise ValueError("; ".join(problems))
        request.submitted_at = self.start + request.arrival_s
        self.requests[request.key] = request
        self.waiting.append(request)

    def _retire(self, r: Request, status: str) -> None:
        """The request is over.  Its pages go back at once: later steps follow on the same stream, behind any step of
        its own that is still in flight (the reference synchronises the device first, runtime/model.py:78-80)."""
        if r.key in self.reserved:
            self.stepper.release(r.key)
            del self.reserved[r.key]
            self.active.remove(r)
        r.status = status
        r.finished_at = time.perf_counter()

    def _finish(self, r: Request) -> None:
        self._retire(r, "finished")

    def cancel(self, key) -> None:
        """Stop a request wherever it is: in the queue, running, or with a step of its own still in flight (whose token
        is then dropped when it is read)."""
        r = self.requests[key]
        if r.status in ENDED:
            return
        if r.status == "waiting":
            self.waiting.remove(r)
        self._retire(r, "cancelled")

    def _entry_price(self, r: Request) -> int:
        """Pages a request must find to be admitted: its whole life under "full" (then it can never lack one later,
        runtime/engine.py:65-76), what it holds tokens for now under "lazy"."""
        return self._life_pages(r) if self.reserve == "full" else self._pages_for(len(r.tokens()))

    def _admit(self) -> None:
        budget = self._pool_pages() - sum(self.reserved.values()) if self.reserve == "full" else self._free_pages()
        now = time.perf_counter()
        # every waiting request is looked at, so a large one does not hold up smaller ones behind it
        for r in [w for w in self.waiting if w.submitted_at <= now]:
            if len(self.active) >= self.max_active:
                return
            price = self._entry_price(r)
            if price > budget:
                continue
            self.waiting.remove(r)
            if r.max_new_tokens == 0:
                self._finish(r)           # nothing to generate: it never touches the cache
                continue
            self.stepper.create(r.key)
            self.reserved[r.key] = price
            budget -= price
            r.status = "prefill"
            self.active.append(r)

    def _preempt(self, r: Request) -> None:
        self.stepper.release(r.key)
        del self.reserved[r.key]
        self.active.remove(r)
        r.cursor = 0
        r.status = "waiting"
        r.preemptions += 1
        self.waiting.appendleft(r)

    # ---------------------------------------------------------------- one step
    def _turn_order(self) -> List[Request]:
        """Who is served first this step: the running requests, starting one further along each step so that none
        starves when the budget is smaller than the batch; under decode_first the decoding ones move to the front,
        otherwise keeping that order (runtime/engine.py:83-85)."""
        first = self.rotation % max(1, len(self.active))
        self.rotation = (first + 1) % max(1, len(self.active))
        order = self.active[first:] + self.active[:first]
        if self.policy == "decode_first":
            order = [r for r in order if r.status == "decode"] + [r for r in order if r.status != "decode"]
        return order

    def _plan(self) -> List[Tuple[Request, int]]:
        """(request, number of its next tokens) for this step, within the token budget: one token for a decoding
        request, for the others as much of the prompt as the chunk limit and the rest of the budget allow."""
        left = self.token_budget
        plan = []
        for r in self._turn_order():
            if left <= 0:
                break
            n = 1 if r.status == "decode" else min(len(r.tokens()) - r.cursor, self.prefill_chunk, left)
            plan.append((r, n))
            left -= n
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

    def _sleep_until_an_arrival(self) -> None:
        """Nothing runs and everything queued is still to arrive: wait a little (at most 10 ms, so a new submit is seen)."""
        if self.active or not self.waiting:
            return
        wait = min(r.submitted_at for r in self.waiting) - time.perf_counter()
        if wait > 0:
            time.sleep(min(wait, 0.01))

    def run(self) -> List[Request]:
        """Tick until every request has ended; the requests in the order they were submitted."""
        while self.tick():
            self._sleep_until_an_arrival()
        return list(self.requests.values())
