"""Schedules in which pages change hands while a step may still be in flight, on the GPU with graphs on.

Each case is an ordinary run: float32 greedy tokens must equal the plain implementation's, the cache manager's
invariants hold after every tick, and every page is back at the end.  Parity: the reference's
tests/test_execution.py:42-64 (changing batch composition against a CPU model) and tests/test_engine.py:23-39
(identical tokens under every policy, nothing leaked).
"""
import numpy as np
import pytest
import torch

import plain_llama as pl
import replay
import tiny_models as tm

pytestmark = pytest.mark.gpu

CASES = {"tiny_b": (tm.TINY_B, 52, 0.08, 8), "tiny_d": (tm.TINY_D, 54, 0.05, 16)}    # config, seed, weight scale, page size


@pytest.fixture(scope="module", params=list(CASES))
def setup(request, tmp_path_factory):
    from cisr_b200 import Model

    cfg, seed, scale, page = CASES[request.param]
    weights = tm.make_weights(cfg, seed, scale=scale, bf16_exact=True)
    path = tm.write_model_dir(tmp_path_factory.mktemp("sched_" + request.param), cfg, weights)
    return cfg, weights, Model.from_pretrained(path, dtype="float32"), page


def plain(cfg, weights, prompt, n, eos=None):
    return pl.generate_greedy(cfg, tm.torch_weights(weights), prompt, n, eos=eos)


def run_checked(engine, between=None, limit=2000):
    """Tick to the end; after every tick the allocator's invariants hold.  `between(engine, tick)` may act between ticks."""
    ticks = 0
    while engine.tick():
        engine.stepper.cache.check()
        if between is not None:
            between(engine, ticks)
        ticks += 1
        assert ticks < limit, "the engine does not come to an end"
    engine.stepper.cache.check()
    pool = engine.stepper.cache.page_groups[0].pool
    assert pool.n_free == pool.n_pages and not engine.stepper.cache.requests, "pages or slots were not given back"
    return {r.key: r for r in engine.requests.values()}


def test_eos_while_the_next_step_is_in_flight_and_admission_into_the_freed_pages(setup):
    """Three requests decode from a graph, one step ahead of the host; one of them meets its EOS, so the step already
    launched was one too many for it.  Its pages go back, and a fourth request, which did not fit before, is admitted
    into them on the next tick."""
    from cisr_b200 import Engine, Request

    cfg, weights, model, page = setup
    new = 12
    prompts = {"a": tm.random_tokens(cfg, 19, 1), "b": tm.random_tokens(cfg, 7, 2), "c": tm.random_tokens(cfg, 26, 3),
               "d": tm.random_tokens(cfg, 11, 4)}
    free_run = {k: plain(cfg, weights, p, new) for k, p in prompts.items()}
    eos = free_run["b"][4]                                   # "b" ends at its fifth token (or earlier, if it met this token before)
    expected = {k: plain(cfg, weights, p, new, eos=eos) for k, p in prompts.items()}
    assert len(expected["b"]) <= 5
    life = lambda k: -(-(len(prompts[k]) + new - 1) // page)
    pages = life("a") + life("b") + life("c") + max(0, life("d") - life("b"))      # "d" fits only once "b" is gone
    engine = Engine.for_model(model, pages=pages, page_size=page, max_active=4, token_budget=64, prefill_chunk=32,
                              policy="decode_first", graph=True)
    assert engine.lookahead
    for k, p in prompts.items():
        engine.submit(Request(k, p, max_new_tokens=new, eos_token_id=eos))
    seen = {"deferred": 0, "d_waited": False}

    def watch(e, tick):
        seen["deferred"] += e._deferred is not None
        if e.requests["b"].status == "decode" and e.requests["d"].status == "waiting":
            seen["d_waited"] = True

    done = run_checked(engine, watch)
    assert seen["deferred"] >= 3, "decode steps did not run ahead of the host"
    assert seen["d_waited"], "the fourth request was to wait for the pages of the one that ends"
    assert {k: r.generated for k, r in done.items()} == expected
    assert all(r.status == "finished" for r in done.values())


def test_lazy_reservation_preempts_and_recomputes_under_graphs(setup):
    from cisr_b200 import Engine, Request

    cfg, weights, model, page = setup
    new = 20
    prompts = {f"r{i}": tm.random_tokens(cfg, n, 10 + i) for i, n in enumerate((5, 9, 14))}
    expected = {k: plain(cfg, weights, p, new) for k, p in prompts.items()}
    whole_life = sum(-(-(len(p) + new - 1) // page) for p in prompts.values())
    biggest = max(-(-(len(p) + new - 1) // page) for p in prompts.values())
    pages = max(biggest, whole_life - 2)                    # all three start, not all three can finish side by side
    engine = Engine.for_model(model, pages=pages, page_size=page, max_active=3, token_budget=32, prefill_chunk=16,
                              policy="decode_first", reserve="lazy", graph=True)
    for k, p in prompts.items():
        engine.submit(Request(k, p, max_new_tokens=new))
    done = run_checked(engine)
    assert sum(r.preemptions for r in done.values()) >= 1, "the pool was to run out"
    assert {k: r.generated for k, r in done.items()} == expected


def test_cancel_between_a_step_in_flight_and_its_read(setup):
    from cisr_b200 import Engine, Request

    cfg, weights, model, page = setup
    new = 10
    prompts = {"keep": tm.random_tokens(cfg, 13, 21), "drop": tm.random_tokens(cfg, 6, 22), "late": tm.random_tokens(cfg, 9, 23)}
    expected = {k: plain(cfg, weights, p, new) for k, p in prompts.items()}
    life = lambda k: -(-(len(prompts[k]) + new - 1) // page)
    engine = Engine.for_model(model, pages=life("keep") + max(life("drop"), life("late")), page_size=page, max_active=3,
                              token_budget=64, prefill_chunk=32, policy="decode_first", graph=True)
    for k, p in prompts.items():
        engine.submit(Request(k, p, max_new_tokens=new))
    state = {"cancelled_at": None}

    def cancel_once(e, tick):
        # a decode step of "keep" and "drop" is in flight, its tokens not read yet: cancel one of its requests now
        if state["cancelled_at"] is None and e._deferred is not None and len(e.requests["drop"].generated) >= 3:
            state["cancelled_at"] = len(e.requests["drop"].generated)
            e.cancel("drop")

    done = run_checked(engine, cancel_once)
    assert state["cancelled_at"] is not None
    assert done["drop"].status == "cancelled"
    assert done["drop"].generated == expected["drop"][:state["cancelled_at"]]        # the token in flight was dropped
    assert done["keep"].generated == expected["keep"] and done["late"].generated == expected["late"]   # "late" took the freed pages


def test_fork_of_a_request_that_decodes_from_a_graph(setup):
    """A request decodes a few tokens from a graph, is forked in the middle of a page, and both go on with tokens of
    their own: the shared, partly filled page is copied before the first write, inside the graph step."""
    from cisr_b200 import StepEntry, Stepper

    cfg, weights, model, page = setup
    prefix = tm.random_tokens(cfg, page + 5, 31)
    tails = {"x": tm.random_tokens(cfg, 9, 32), "y": tm.random_tokens(cfg, 9, 33)}
    stepper = Stepper(model, n_pages=8, page_size=page, max_slots=3, graph=True)
    stepper.create("x")
    stepper.step([StepEntry("x", prefix[:-3], [])])
    got = {}
    for i in range(3):                                                       # single tokens: from the graph
        at = len(prefix) - 3 + i
        got[("x", at)] = stepper.step([StepEntry("x", [prefix[at]], [0])]).cpu().numpy()[0].copy()
    assert stepper.graphs.report()["entries"] >= 1
    stepper.fork("x", "y")
    stepper.cache.check()
    for j in range(9):
        logits = stepper.step([StepEntry("x", [tails["x"][j]], [0]), StepEntry("y", [tails["y"][j]], [0])]).cpu().numpy()
        got[("x", len(prefix) + j)], got[("y", len(prefix) + j)] = logits[0].copy(), logits[1].copy()
        stepper.cache.check()
    tx, ty = stepper.cache.requests["x"].tables[0], stepper.cache.requests["y"].tables[0]
    assert tx[0] == ty[0] and tx[1] != ty[1]                                 # the full page stays shared, the partly filled one was copied
    reference = {k: replay.plain_logits(cfg, weights, prefix + tails[k]) for k in tails}
    replay.compare(got, None, reference, "float32")
    stepper.release("x"); stepper.release("y")
    assert stepper.cache.page_groups[0].pool.n_free == 8
