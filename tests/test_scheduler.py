"""The scheduler's decisions with a host-only step function (no GPU).

The stand-in uses the real cache manager (host bookkeeping only) and produces logits
that depend only on a request's own token history, so any two runs that feed every
request its tokens in order, whatever the batching, must choose identical tokens.
"""
import hashlib

import numpy as np
import pytest

from cisr_b200.cache import CacheManager, OutOfPages
from cisr_b200.config.spec import CacheUse
from cisr_b200.engine.scheduler import Engine, Request

VOCAB = 50


class HostStepper:
    def __init__(self, pages=16, page_size=2, max_slots=8, max_positions=64):
        self.cache = CacheManager([CacheUse("pages", kv_heads=1, head_dim=16)] * 2, pages, page_size, max_slots, max_positions)
        self.history = {}
        self.steps = []
        self.last_extras = {}

    def create(self, key):
        self.cache.create(key); self.history[key] = []

    def release(self, key):
        self.cache.release(key); del self.history[key]

    def step(self, entries, extra=None):
        self.cache.reserve([(e.key, len(e.tokens)) for e in entries])
        rows = []
        for e in entries:
            assert self.cache.length(e.key) == len(self.history[e.key])
            for i, t in enumerate(e.tokens):
                self.history[e.key].append(int(t))
                if i in e.want:
                    digest = hashlib.sha256(repr(self.history[e.key]).encode()).digest()
                    row = np.zeros(VOCAB, np.float32); row[digest[0] % VOCAB] = 1.0
                    rows.append(row)
            self.cache.commit(e.key, len(e.tokens))
        self.steps.append([(e.key, len(e.tokens), list(e.want)) for e in entries])
        self.cache.check()
        return np.stack(rows) if rows else np.zeros((0, VOCAB), np.float32)


def choose(logits, requests):
    return np.argmax(logits, axis=-1).tolist()


def engine(stepper=None, **kw):
    stepper = stepper or HostStepper()
    return Engine(stepper, choose, VOCAB, stepper.cache.max_positions, **kw), stepper


def expected_tokens(prompt, n):
    seq, out = list(prompt), []
    for _ in range(n):
        token = hashlib.sha256(repr(seq).encode()).digest()[0] % VOCAB
        out.append(token); seq.append(token)
    return out


def test_policies_and_budgets_choose_identical_tokens_and_return_all_pages():
    prompts = [[1], list(range(7)), [3, 4, 5]]
    results = []
    for kw in (dict(policy="serial"), dict(policy="chunked", token_budget=3, prefill_chunk=2),
               dict(policy="decode_first", token_budget=3, prefill_chunk=2), dict(policy="chunked", token_budget=64, prefill_chunk=64),
               dict(policy="decode_first", token_budget=2, prefill_chunk=5, reserve="lazy")):
        e, s = engine(**kw)
        for i, p in enumerate(prompts):
            e.submit(Request(str(i), p, 5))
        done = e.run()
        results.append([r.generated for r in done])
        assert all(r.status == "finished" for r in done)
        assert s.cache.page_groups[0].pool.n_free == 16 and not e.reserved and not s.cache.requests
    assert all(r == results[0] for r in results)
    assert results[0] == [expected_tokens(p, 5) for p in prompts]


def test_a_step_stays_within_the_token_budget_and_cuts_prompts_into_portions():
    e, s = engine(token_budget=5, prefill_chunk=3, policy="chunked")
    e.submit(Request("a", list(range(10)), 2)); e.submit(Request("b", list(range(4)), 2))
    e.run()
    for step in s.steps:
        assert sum(n for _, n, _ in step) <= 5
        assert all(n <= 3 for _, n, _ in step)
    portions_a = [n for step in s.steps for k, n, _ in step if k == "a"]
    assert portions_a[:4] == [3, 3, 3, 1] or sum(portions_a[:4]) >= 9
    wants = [(k, n, w) for step in s.steps for k, n, w in step if w]
    assert all(w == [n - 1] for _, n, w in wants)       # logits only at the last token of a finishing portion or a decode token
    assert [t["processed_tokens"] for t in e.trace] == [sum(n for _, n, _ in step) for step in s.steps]


def test_decode_first_puts_decoding_requests_before_prompt_portions():
    e, s = engine(token_budget=3, prefill_chunk=2, policy="decode_first")
    e.submit(Request("short", [1], 6)); e.submit(Request("long", list(range(12)), 2))
    e.run()
    mixed = [step for step in s.steps if len(step) == 2]
    assert mixed and all(step[0][0] == "short" and step[0][1] == 1 for step in mixed[1:])


def test_rotation_lets_every_request_progress_when_the_budget_is_smaller_than_the_batch():
    e, s = engine(token_budget=1, prefill_chunk=1, policy="chunked")
    for k in "abc":
        e.submit(Request(k, [1, 2, 3], 2))
    for _ in range(3):
        e.tick()
    assert sorted(step[0][0] for step in s.steps[:3]) == ["a", "b", "c"]


def test_full_reservation_makes_requests_wait_for_pages_and_lets_smaller_ones_pass():
    stepper = HostStepper(pages=6, page_size=2)
    e, s = engine(stepper, token_budget=8, prefill_chunk=8)
    e.submit(Request("big", list(range(8)), 3))          # 10 tokens -> 5 pages
    e.submit(Request("big2", list(range(8)), 3))         # must wait: 5 + 5 > 6
    e.submit(Request("small", [1], 2))                   # 2 tokens -> 1 page: passes big2
    e.tick()
    assert [r.key for r in e.active] == ["big", "small"] and [r.key for r in e.waiting] == ["big2"]
    done = {r.key: r for r in e.run()}
    assert all(r.status == "finished" for r in done.values())
    assert done["big2"].generated == expected_tokens(range(8), 3)
    assert done["big2"].first_token_at > done["big"].finished_at   # it ran only after big's pages came back
    assert stepper.cache.page_groups[0].pool.n_free == 6 and stepper.cache.page_groups[0].pool.peak <= 6


def test_lazy_reservation_preempts_the_youngest_request_and_recomputes_it():
    stepper = HostStepper(pages=7, page_size=2)
    e, s = engine(stepper, token_budget=16, prefill_chunk=16, reserve="lazy", policy="chunked")
    e.submit(Request("a", list(range(6)), 8))            # life: 13 tokens -> 7 pages (fits alone)
    e.submit(Request("b", list(range(10, 14)), 8))       # prompts fit together (3 + 2 pages), their lives do not
    done = {r.key: r for r in e.run()}
    assert done["b"].preemptions >= 1 and done["a"].preemptions == 0
    assert done["a"].generated == expected_tokens(range(6), 8)
    assert done["b"].generated == expected_tokens(range(10, 14), 8)    # kept and recomputed, not lost
    assert stepper.cache.page_groups[0].pool.n_free == 7
    e2, _ = engine(HostStepper(pages=7, page_size=2), reserve="full", token_budget=16, prefill_chunk=16)
    e2.submit(Request("a", list(range(6)), 8)); e2.submit(Request("b", list(range(10, 14)), 8))
    assert all(r.preemptions == 0 for r in e2.run())


def test_submit_checks_and_cancel():
    e, s = engine(HostStepper(pages=4, page_size=2, max_positions=16))
    e.submit(Request("a", [1, 2], 2))
    for bad, word in ((Request("a", [1], 1), "duplicate"), (Request("b", [], 1), "invalid request"),
                      (Request("c", [1], -1), "invalid request"), (Request("d", [VOCAB], 1), "invalid prompt token"),
                      (Request("e", [1] * 16, 2), "context limit"), (Request("f", [1] * 9, 1), "page pool"),
                      (Request("g", [1], 1, temperature=-1.0), "temperature")):
        with pytest.raises(ValueError, match=word):
            e.submit(bad)
    e.submit(Request("zero", [1], 0)); e.submit(Request("w", [1, 2, 3], 3))
    e.cancel("w")
    e.tick()
    e.cancel("a")
    assert e.requests["a"].status == "cancelled" and e.requests["w"].status == "cancelled"
    assert e.requests["zero"].status == "finished" and e.requests["zero"].generated == []
    assert not e.tick() and s.cache.page_groups[0].pool.n_free == 4
    used = Request("h", [1], 1); used.cursor = 1
    with pytest.raises(ValueError, match="already used"):
        e.submit(used)


def test_eos_ends_a_request_and_serial_runs_one_at_a_time():
    first = expected_tokens([7, 8], 1)[0]
    e, s = engine(policy="serial")
    e.submit(Request("a", [7, 8], 9, eos_token_id=first)); e.submit(Request("b", [7, 8], 3, eos_token_id=[49, 48]))
    done = {r.key: r for r in e.run()}
    assert done["a"].generated == [first] and len(done["b"].generated) <= 3
    assert all(len({k for k, _, _ in step}) == 1 for step in s.steps)


def test_invalid_limits_are_refused():
    for kw in (dict(max_active=0), dict(token_budget=0), dict(prefill_chunk=0), dict(policy="fifo"), dict(reserve="none")):
        with pytest.raises(ValueError):
            engine(**kw)


class AheadStepper(HostStepper):
    """A stand-in whose decode steps can run one step ahead of the host, as the graph path does: the tokens a step chose
    stay "on the device" (a tensor) and the next step feeds them back by itself."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self._batch = None
        self.last_tokens = None
        self.ahead_calls = 0

    def _choose(self, key):
        return hashlib.sha256(repr(self.history[key]).encode()).digest()[0] % VOCAB

    def step(self, entries, extra=None):
        import torch
        logits = super().step(entries, extra)
        self._batch = None
        if all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
            self._batch = [e.key for e in entries]
            self.last_tokens = torch.tensor(np.argmax(logits, axis=-1))
        return logits

    def can_run_ahead(self):
        return self._batch is not None

    def check_kernels(self):
        pass

    def decode_ahead(self, steps):
        import torch
        assert steps == 1
        self.ahead_calls += 1
        self.cache.reserve([(k, 1) for k in self._batch])
        out = []
        for k in self._batch:
            self.history[k].append(self._pending_token(k))
            self.cache.commit(k, 1)
            out.append(self._choose(k))
        self.last_tokens = torch.tensor(out)
        return torch.tensor([out])

    def _pending_token(self, key):
        # the token the step before chose for this request: the hash of its history as that step saw it
        return hashlib.sha256(repr(self.history[key]).encode()).digest()[0] % VOCAB


def test_lookahead_runs_the_next_decode_step_before_reading_the_last_and_drops_what_an_eos_made_useless():
    prompts = {"a": [1, 2, 3], "b": [9], "c": list(range(5))}
    plain, _ = engine(token_budget=16, prefill_chunk=16)
    for k, p in prompts.items():
        plain.submit(Request(k, p, 9))
    want = {r.key: r.generated for r in plain.run()}
    eos = want["b"][4]
    cut = {k: (v[:v.index(eos) + 1] if eos in v else v) for k, v in want.items()}

    stepper = AheadStepper()
    e = Engine(stepper, choose, VOCAB, stepper.cache.max_positions, token_budget=16, prefill_chunk=16, lookahead=True)
    for k, p in prompts.items():
        e.submit(Request(k, p, 9))
    assert {r.key: r.generated for r in e.run()} == want and stepper.ahead_calls >= 5

    stepper = AheadStepper()
    e = Engine(stepper, choose, VOCAB, stepper.cache.max_positions, token_budget=16, prefill_chunk=16, lookahead=True)
    for k, p in prompts.items():
        e.submit(Request(k, p, 9, eos_token_id=eos))
    done = {r.key: r for r in e.run()}
    assert {k: r.generated for k, r in done.items()} == cut
    assert all(r.status == "finished" for r in done.values())
    assert stepper.cache.page_groups[0].pool.n_free == 16 and not stepper.cache.requests
