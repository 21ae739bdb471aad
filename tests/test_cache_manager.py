"""The cache manager on the host: pages are never lost, held twice or freed twice, under random
orders of requests; windows give pages back; state slots are counted."""
import random

import pytest

from tinyinfer_b200.cache import (CacheExhausted, CacheManager, PagePool, group_cache_needs,
                                  prefix_caching_possible)
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


# ---------------------------------------------------------------------------- prefix cache
ONLY_FULL = [(FULL, None), (FULL, None)]


def run_request(m, rid, tokens, upto=None):
    """Admits with its tokens, stores keys for all (or ``upto``) of them, files the full pages."""
    rc = m.admit(rid, tokens)
    cached = rc.length
    n = len(tokens) if upto is None else upto
    m.extend(rid, n)
    m.commit(rid, n)
    m.note_tokens(rid, tokens)
    return cached


def test_prefix_cache_is_refused_where_pages_do_not_tell_the_whole_story():
    assert prefix_caching_possible(ONLY_FULL)
    assert not prefix_caching_possible(NEEDS)                                   # a window, a state
    assert not prefix_caching_possible([(FULL, StateNeed((4,)))])
    with pytest.raises(ValueError, match="prefix cache"):
        CacheManager(NEEDS, 4, 8, 2, prefix_caching=True)


def test_prefix_hit_after_release_and_one_token_is_always_left():
    m = CacheManager(ONLY_FULL, page_size=4, num_pages=8, max_requests=4, prefix_caching=True)
    toks = list(range(50, 62))                                                 # 12 tokens: 3 full pages
    assert run_request(m, "a", toks) == 0
    pages_a = list(m.get("a").tables[0])
    m.release("a")
    m.check_consistency()
    assert m.groups[0].pool.num_free == 8                                      # kept pages count as free
    # the same prompt again: its last page must be computed again, so that one token runs
    assert run_request(m, "b", toks) == 8
    assert m.get("b").tables[0][:2] == pages_a[:2]
    # a prompt that is longer takes all three; one that differs inside page 1 takes only page 0
    assert run_request(m, "c", toks + [1, 2]) == 12
    assert run_request(m, "d", toks[:5] + [0] + toks[6:]) == 4
    m.check_consistency()
    assert m.groups[0].pool.holders_of(pages_a[0]) == {"b", "c", "d"}
    for rid in "bcd":
        m.release(rid)
    m.check_consistency()
    assert m.stats()["prefix_hit_tokens"] == 8 + 12 + 4


def test_shared_page_stays_until_its_last_holder_goes_and_reuse_forgets_it():
    m = CacheManager(ONLY_FULL, page_size=2, num_pages=4, max_requests=4, prefix_caching=True)
    toks = [7, 8, 9, 10, 11]
    run_request(m, "a", toks)                                                  # pages 0,1 full, 2 half
    assert run_request(m, "b", toks) == 4
    shared = m.get("a").tables[0][:2]
    m.release("a")
    assert all(m.groups[0].pool.holders_of(p) == {"b"} for p in shared)
    m.check_consistency()
    m.release("b")
    assert m.stats()["kept_pages"] == 2
    # a stranger needs every page: the kept ones are handed out and forgotten, tail of the prefix first
    run_request(m, "x", [1, 2, 3, 4, 5, 6, 7, 8][:7])
    assert m.stats()["kept_pages"] == 3                                        # x's own full pages
    m.release("x")
    assert run_request(m, "c", toks) == 0
    m.check_consistency()


def test_a_page_is_filed_only_when_full_of_stored_keys():
    m = CacheManager(ONLY_FULL, page_size=4, num_pages=8, max_requests=4, prefix_caching=True)
    toks = list(range(20, 30))
    run_request(m, "a", toks, upto=7)                                          # a portion: one full page
    assert m.stats()["kept_pages"] == 1
    m.extend("a", 10), m.commit("a", 10), m.note_tokens("a", toks)
    assert m.stats()["kept_pages"] == 2
    with pytest.raises(ValueError, match="fewer tokens"):
        m.extend("a", 12), m.commit("a", 12), m.note_tokens("a", toks)
    m.release("a")


@pytest.mark.parametrize("seed", range(4))
def test_prefix_cache_random_traffic_keeps_every_invariant(seed):
    rng = random.Random(100 + seed)
    m = CacheManager(ONLY_FULL, page_size=4, num_pages=24, max_requests=5, prefix_caching=True)
    stems = [[rng.randrange(50) for _ in range(rng.randrange(4, 30))] for _ in range(4)]
    live = {}
    hits = 0
    for step in range(600):
        if live and (rng.random() < 0.35 or not m.can_admit()):
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        elif m.can_admit():
            toks = list(rng.choice(stems)) + [rng.randrange(50) for _ in range(rng.randrange(1, 9))]
            rid = f"r{step}"
            rc = m.admit(rid, toks)
            hits += rc.length
            assert rc.length % 4 == 0 and rc.length < len(toks)
            # what was taken over really is this prompt's beginning
            for i, page in enumerate(rc.tables[0]):
                assert m._page_key[page][2] == tuple(toks[4 * i:4 * i + 4])
            if not m.can_extend(rid, len(toks)):
                m.release(rid)
            else:
                m.extend(rid, len(toks)), m.commit(rid, len(toks)), m.note_tokens(rid, toks)
                live[rid] = toks
        m.check_consistency()
    assert hits > 0
    for rid in list(live):
        m.release(rid)
    m.check_consistency()
    assert m.groups[0].pool.num_free == 24
