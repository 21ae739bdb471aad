"""The cache manager on the host: pages are never lost, held twice or freed twice, under random
orders of requests; windows give pages back; state slots are counted."""
import random

import pytest

from tinyinfer_b200.cache import CacheExhausted, CacheManager, PagePool, group_cache_needs
from tinyinfer_b200.parts import CacheNeed, StateNeed

FULL = CacheNeed(2, 16, None)
WIN = CacheNeed(2, 16, 10)
NEEDS = [(FULL, None), (WIN, None), (FULL, None), (None, StateNeed((4,)))]


def test_groups_by_need():
    groups = group_cache_needs(NEEDS)
    assert [(n.window, e) for n, e in groups] == [(None, [0, 2]), (10, [1])]


def test_pool_refuses_double_free_and_foreign_free():
    pool = PagePool(3)
    a = pool.take("x")
    pool.give_back(a, "x")
    with pytest.raises(RuntimeError, match="twice"):
        pool.give_back(a, "x")
    b = pool.take("x")
    with pytest.raises(RuntimeError, match="belongs"):
        pool.give_back(b, "y")
    pool.take("x"), pool.take("x")
    with pytest.raises(CacheExhausted):
        pool.take("x")


def test_extend_commit_release_and_window():
    m = CacheManager(NEEDS, page_size=4, num_pages=8, max_requests=2)
    m.admit("a")
    m.extend("a", 9)                       # 3 pages in both groups
    assert [len(t) for t in m.get("a").tables] == [3, 3]
    m.commit("a", 9)
    m.check_consistency()
    m.extend("a", 26)
    m.commit("a", 26)                      # window 10: next query at 26 reads keys >= 17 -> pages 0..3 go
    full, win = m.get("a").tables
    assert all(p >= 0 for p in full) and win[:4] == [-1] * 4 and all(p >= 0 for p in win[4:])
    assert m.groups[1].pool.num_free == 8 - 3
    m.check_consistency()
    assert not m.can_extend("a", 40)       # the full group is out of pages
    with pytest.raises(CacheExhausted):
        m.extend("a", 40)
    assert [len(t) for t in m.get("a").tables] == [7, 7]      # nothing was taken by the failed call
    m.admit("b")
    with pytest.raises(CacheExhausted):
        m.admit("c")
    with pytest.raises(RuntimeError):
        m.admit("b")
    m.release("a")
    m.release("b")
    assert all(g.pool.num_free == 8 for g in m.groups)
    m.check_consistency()
    with pytest.raises(KeyError):
        m.release("a")


def test_freed_pages_are_reused_oldest_first_and_tail_first():
    m = CacheManager([(FULL, None)], page_size=2, num_pages=4, max_requests=2)
    m.admit("a")
    m.extend("a", 6)                       # pages 0, 1, 2
    m.release("a")                         # back as 2, 1, 0 behind page 3
    m.admit("b")
    m.extend("b", 8)
    assert m.get("b").tables[0] == [3, 2, 1, 0]


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_invariant(seed):
    rng = random.Random(seed)
    m = CacheManager(NEEDS, page_size=4, num_pages=24, max_requests=5)
    live = {}
    next_id = 0
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and m.can_admit():
            m.admit(next_id)
            live[next_id] = 0
            next_id += 1
        elif action < 0.85 and live:
            rid = rng.choice(list(live))
            new = live[rid] + rng.choice([1, 1, 1, 2, 5, 17])
            if m.can_extend(rid, new):
                m.extend(rid, new)
                m.commit(rid, new)
                live[rid] = new
            else:
                with pytest.raises(CacheExhausted):
                    m.extend(rid, new)
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check_consistency()
        for rid, n in live.items():
            rc = m.get(rid)
            assert rc.length == n
            full, win = rc.tables
            assert len(full) == len(win) == (n + 3) // 4 or len(full) >= (n + 3) // 4
            lo = max(0, n - 10 + 1) // 4   # first page the next query may read in the window group
            assert all(p >= 0 for p in win[lo:]) and all(p == -1 for p in win[:lo])
    for rid in list(live):
        m.release(rid)
    assert all(g.pool.num_free == 24 for g in m.groups)
    assert m.stats()["free_state_slots"] == 5
