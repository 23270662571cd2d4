"""The cache manager's host bookkeeping (no GPU): no page lost, held twice or freed twice."""
import numpy as np
import pytest

from cisr_b200.cache import CacheManager, OutOfPages, PagePool
from cisr_b200.config.spec import CacheUse

FULL = CacheUse("pages", kv_heads=2, head_dim=16)
WINDOW = CacheUse("pages", kv_heads=2, head_dim=16, window=10)
STATE = CacheUse("state", state_shape=(4,), state_dtype="float32")


def manager(uses=(FULL, FULL), n_pages=8, page_size=4, max_slots=4, max_positions=64):
    return CacheManager(list(uses), n_pages, page_size, max_slots, max_positions)


def step(m, key, n):
    m.reserve([(key, n)])
    m.commit(key, n)


def test_pool_allocates_all_or_nothing_and_detects_double_free():
    pool = PagePool(3)
    a = pool.allocate(2)
    with pytest.raises(OutOfPages):
        pool.allocate(2)
    assert pool.n_free == 1
    pool.release(a[0])
    with pytest.raises(AssertionError, match="freed twice"):
        pool.release(a[0])
    pool.check([[a[1]]])
    with pytest.raises(AssertionError):
        pool.check([[a[1]], [a[1]]])          # a page named twice but held once


def test_layers_with_equal_needs_share_one_group_and_windows_get_their_own():
    m = manager(uses=(FULL, WINDOW, FULL, 1, STATE, CacheUse("none")))
    assert [len(g.entries) for g in m.page_groups] == [2, 1]
    assert m.page_groups[0].entries == [0, 2] and m.page_groups[1].entries == [1]
    assert len(m.state_groups) == 1 and m.entry_group[4] == ("state", 0)
    assert m.entry_source[3] == 1 and 5 not in m.entry_group


def test_pages_follow_the_length_and_come_back_on_release():
    m = manager()
    m.create("a")
    step(m, "a", 5)
    assert m.length("a") == 5 and m.page_groups[0].pool.n_used == 2
    step(m, "a", 3)
    assert m.page_groups[0].pool.n_used == 2           # 8 tokens fill two pages of 4 exactly
    step(m, "a", 1)
    assert m.page_groups[0].pool.n_used == 3
    m.check()
    m.release("a")
    assert m.page_groups[0].pool.n_free == 8 and len(m.free_slots) == 4
    m.check()
    with pytest.raises(ValueError, match="duplicate"):
        m.create("b"); m.create("b")


def test_reserve_is_atomic_when_pages_run_out():
    m = manager(n_pages=3)
    m.create("a"); m.create("b")
    step(m, "a", 4)
    before = (m.page_groups[0].pool.n_free, list(m.requests["a"].tables[0]), list(m.requests["b"].tables[0]))
    with pytest.raises(OutOfPages, match="insufficient KV pages"):
        m.reserve([("a", 4), ("b", 5)])               # needs 1 + 2 pages, 2 are free
    assert (m.page_groups[0].pool.n_free, m.requests["a"].tables[0], m.requests["b"].tables[0]) == before
    assert m.length("a") == 4 and m.length("b") == 0
    m.check()
    with pytest.raises(ValueError, match="context limit"):
        m.reserve([("a", 100)])


def test_reserved_pages_reach_the_device_table_as_updates():
    m = manager()
    slot = m.create("a")
    m.reserve([("a", 6)])
    idx, val = m.drain_table_updates(0)
    width = m.width
    assert idx.tolist() == [slot * width, slot * width + 1] and val.tolist() == m.requests["a"].tables[0]
    assert m.drain_table_updates(0)[0].size == 0
    m.commit("a", 6)
    m.release("a")
    idx, val = m.drain_table_updates(0)
    assert sorted(idx.tolist()) == [slot * width, slot * width + 1] and set(val.tolist()) == {-1}
    # a slot freed and taken again within one batch of updates: one value per entry, the latest
    m.create("b"); m.reserve([("b", 1)]); m.commit("b", 1); m.release("b"); m.create("c"); m.reserve([("c", 1)])
    idx, val = m.drain_table_updates(0)
    assert len(set(idx.tolist())) == len(idx) and val[idx.tolist().index(m.slot("c") * width)] == m.requests["c"].tables[0][0]


def test_fork_shares_pages_and_copies_a_shared_partial_page_before_writing():
    m = manager()
    m.create("a")
    step(m, "a", 6)                                    # pages [p0, p1], p1 half full
    m.fork("a", "b")
    pool = m.page_groups[0].pool
    p0, p1 = m.requests["a"].tables[0]
    assert pool.refs[p0] == 2 and pool.refs[p1] == 2 and pool.n_used == 2
    m.reserve([("b", 1)])                              # b writes into the shared partial page: gets its own copy
    assert m.requests["b"].tables[0][0] == p0 and m.requests["b"].tables[0][1] != p1
    assert m.drain_copies(0) == [(p1, m.requests["b"].tables[0][1])]
    assert pool.refs[p1] == 1 and pool.refs[p0] == 2
    m.commit("b", 1)
    m.reserve([("a", 1)])                              # a now owns p1 alone: no copy
    assert m.drain_copies(0) == [] and m.requests["a"].tables[0] == [p0, p1]
    m.commit("a", 1)
    m.check()
    m.release("a")
    assert pool.refs[p0] == 1
    m.release("b")
    assert pool.n_free == 8
    m.check()


def test_fork_fails_cleanly_when_the_copy_cannot_be_allocated():
    m = manager(n_pages=2)
    m.create("a"); step(m, "a", 6)
    m.fork("a", "b")
    with pytest.raises(OutOfPages):
        m.reserve([("b", 1)])
    assert m.requests["b"].tables[0] == m.requests["a"].tables[0]
    m.check()


def test_a_window_group_gives_pages_back_once_the_window_has_passed_them():
    m = manager(uses=(FULL, WINDOW), n_pages=20, page_size=4, max_positions=200)
    m.create("a")
    used = []
    for _ in range(40):
        step(m, "a", 1)
        m.check()
        used.append((m.page_groups[0].pool.n_used, m.page_groups[1].pool.n_used))
    assert used[-1][0] == 10                           # every key kept: 40 tokens, 10 pages
    assert max(u[1] for u in used) <= 4                # a window of 10 keys spans at most 4 pages of 4
    table = m.requests["a"].tables[1]
    # the next query (position 40) sees keys 31..39: pages 0..6 are gone, 7..9 live
    assert [p >= 0 for p in table] == [False] * 7 + [True] * 3
    step(m, "a", 30)                                   # a long portion needs all its pages during the step...
    assert m.page_groups[1].pool.n_used <= 4           # ...and gives the passed ones back right after
    m.release("a")
    assert m.page_groups[1].pool.n_free == 20 and m.page_groups[0].pool.n_free == 20
    m.check()


def test_slots_are_handed_out_once_and_run_out():
    m = manager(max_slots=2)
    a, b = m.create("a"), m.create("b")
    assert a != b
    with pytest.raises(OutOfPages, match="slots"):
        m.create("c")
    m.release("a")
    assert m.create("c") == a
    m.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests_never_lose_or_double_a_page(seed):
    rng = np.random.default_rng(seed)
    m = manager(uses=(FULL, WINDOW, FULL), n_pages=24, page_size=4, max_slots=5, max_positions=120)
    live, counter = [], 0
    for _ in range(400):
        action = rng.integers(0, 10)
        try:
            if action < 2 and len(live) < 5:
                key = f"r{counter}"; counter += 1
                m.create(key); live.append(key)
            elif action == 2 and live and len(live) < 5:
                key = f"r{counter}"; counter += 1
                m.fork(live[int(rng.integers(len(live)))], key); live.append(key)
            elif action < 8 and live:
                batch = [(k, int(rng.integers(1, 9))) for k in live if rng.random() < 0.6]
                batch = [(k, n) for k, n in batch if m.length(k) + n <= 120]
                if batch:
                    m.reserve(batch)
                    for k, n in batch:
                        m.commit(k, n)
            elif live:
                m.release(live.pop(int(rng.integers(len(live)))))
        except OutOfPages:
            pass                                        # refused atomically; the check below proves nothing moved
        m.check()
    for key in live:
        m.release(key)
    m.check()
    assert all(g.pool.n_free == 24 for g in m.page_groups) and len(m.free_slots) == 5
