"""The cache manager's bookkeeping (CPU): no page lost, held twice or freed twice, under
random orders of requests; window release; reservations that fail change nothing."""
import random

import pytest

from llm_rs_b200.cache import CacheError, CacheManager, GroupSpec, NoFreeSlot, OutOfPages, PagePool, RELEASED
from llm_rs_b200.parts import CacheNeed, RunStep


def test_pool_contract():
    pool = PagePool(3)
    a, b, c = pool.allocate(), pool.allocate(), pool.allocate()
    assert (a, b, c) == (0, 1, 2) and pool.free_pages() == 0
    with pytest.raises(OutOfPages):
        pool.allocate()
    pool.increment_ref(b)
    assert pool.free(b) is False and pool.free(b) is True
    with pytest.raises(CacheError, match="double free"):
        pool.free(b)
    with pytest.raises(CacheError, match="invalid page"):
        pool.free(7)
    with pytest.raises(CacheError, match="not allocated"):
        pool.increment_ref(b)
    assert pool.allocate() == b        # a freed page is used again
    with pytest.raises(OutOfPages):
        pool.allocate_many(2)


def _manager(n_pages=8, page=4, slots=3, window=0):
    groups = [GroupSpec(CacheNeed("full", 2, 16), [0, 1], n_pages)]
    if window:
        groups.append(GroupSpec(CacheNeed("window", 2, 16, window), [2], n_pages))
    return CacheManager(groups, page, slots)


def test_reserve_commit_release():
    m = _manager()
    m.admit("a")
    m.reserve("a", 6)                      # 2 pages of 4
    assert m.table("a", 0) == [0, 1] and m.free_pages() == 6
    with pytest.raises(CacheError, match="uncommitted"):
        m.reserve("a", 1)
    m.commit("a", 6)
    m.reserve("a", 2)                      # positions 6, 7 fit the second page
    assert m.table("a", 0) == [0, 1]
    m.commit("a", 2)
    m.reserve("a", 1)
    assert m.table("a", 0) == [0, 1, 2]
    m.cancel("a")                          # the step did not run
    assert m.table("a", 0) == [0, 1] and m.record("a").cached_len == 8
    m.check_invariants()
    m.release("a")
    assert m.free_pages() == 8 and not m.requests
    with pytest.raises(CacheError, match="not live"):
        m.release("a")


def test_failed_reservation_changes_nothing():
    m = _manager(n_pages=3)
    m.admit("a")
    m.reserve("a", 8)
    m.commit("a", 8)
    m.admit("b")
    with pytest.raises(OutOfPages):
        m.reserve("b", 5)                  # needs 2, 1 free
    assert m.table("b", 0) == [] and m.free_pages() == 1
    assert m.can_reserve("b", 4) and not m.can_reserve("b", 5)
    assert m.pages_needed(None, 9, 0) == [3]
    m.check_invariants()


def test_slots():
    m = _manager(slots=2)
    s = {m.admit("a").slot, m.admit("b").slot}
    assert s == {0, 1}
    with pytest.raises(NoFreeSlot):
        m.admit("c")
    with pytest.raises(CacheError, match="already live"):
        m.admit("a")
    m.release("a")
    assert m.admit("c").slot in s
    m.check_invariants()


def test_window_group_gives_pages_back():
    m = _manager(n_pages=6, page=4, window=6)
    m.admit("a")
    for step in range(10):                 # 3 tokens a step
        m.reserve("a", 3)
        m.commit("a", 3)
        m.check_invariants()
        c = m.record("a").cached_len
        first_needed = max(0, c - 6 + 1) // 4
        table = m.table("a", 1)
        assert all(p == RELEASED for p in table[:first_needed])
        assert all(p != RELEASED for p in table[first_needed:])
        if step < 7:                       # the full group holds everything (6 pages = 24 tokens)
            assert RELEASED not in m.table("a", 0)
        if c + 3 > 24:
            break
    # The window group never held more than ceil((6 + 3) / 4) + 1 pages.
    assert m.pools[1].used_pages() <= 4
    m.release("a")
    assert m.free_pages(0) == 6 and m.free_pages(1) == 6


def test_window_group_long_first_portion():
    """A first portion longer than the window still gets every page it writes to."""
    m = _manager(n_pages=10, page=4, window=5)
    m.admit("a")
    m.reserve("a", 30)
    assert RELEASED not in m.table("a", 1)       # queries at 0.. read from page 0 on
    m.commit("a", 30)
    assert m.table("a", 1)[:6] == [RELEASED] * 6  # next query at 30 reads keys 26.. -> page 6
    assert m.pages_needed("a", 1) == [0, 0]
    m.check_invariants()


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    m = _manager(n_pages=24, page=4, slots=4, window=7)
    live, counter = {}, 0
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and len(live) < 4:
            counter += 1
            rid = f"r{counter}"
            m.admit(rid)
            live[rid] = 0
        elif action < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 3, 5, 9])
            try:
                m.reserve(rid, n)
            except OutOfPages:
                before = [p.free_pages() for p in m.pools]
                m.check_invariants()
                assert before == [p.free_pages() for p in m.pools]
                victim = rng.choice(list(live))
                m.release(victim)
                del live[victim]
                continue
            if rng.random() < 0.1:
                m.cancel(rid)
            else:
                m.commit(rid, n)
                live[rid] += n
                assert m.record(rid).cached_len == live[rid]
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check_invariants()
        # A page is never in two tables.
        for g in range(2):
            held = [p for r in live for p in m.table(r, g) if p != RELEASED]
            assert len(held) == len(set(held))
    for rid in list(live):
        m.release(rid)
    assert [p.free_pages() for p in m.pools] == [24, 24]


def test_groups_are_planned_from_needs():
    from llm_rs_b200.cache.storage import plan_groups
    full, win = CacheNeed("full", 2, 16), CacheNeed("window", 2, 16, 8)
    order = [RunStep(0), RunStep(1), RunStep(0), RunStep(2, cache_of=1), RunStep(3)]
    needs = [(full, None), (win, None), (full, None), (None, None), (None, None)]
    groups, eg, ei = plan_groups(needs, order, 10)
    assert [g.need for g in groups] == [full, win]
    assert groups[0].entries == [0, 2] and groups[1].entries == [1]
    assert eg == [0, 1, 0, 1, None] and ei == [0, 0, 1, 0, None]
