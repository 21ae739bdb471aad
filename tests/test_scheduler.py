"""The scheduler's decisions (CPU): budgets, the decode reserve, round-robin, portions, stopping,
and what happens when pages run out."""
import random

import pytest

from tinyinfer_b200.cache import CacheManager
from tinyinfer_b200.config import EngineConfig
from tinyinfer_b200.engine.scheduler import Scheduler
from tinyinfer_b200.engine.sequence import Sequence, SequenceStatus
from tinyinfer_b200.parts import CacheNeed
from tinyinfer_b200.sampling import SamplingParams


def make(num_pages=64, page=4, **kw):
    cfg = EngineConfig(**{**dict(max_num_batched_tokens=16, max_num_seqs=4, max_model_len=64,
                                 kvcache_block_size=page, num_kvcache_blocks=num_pages), **kw})
    manager = CacheManager([(CacheNeed(2, 16, None), None)], page, num_pages, cfg.live_requests)
    return Scheduler(cfg, manager, eos_token_id=9), manager


def seq(i, n, **kw):
    return Sequence(i, list(range(100, 100 + n)), SamplingParams(**{**dict(greedy=True, max_tokens=4), **kw}))


def run_step(s, token=1):
    items = s.schedule()
    s.postprocess(items, {it.seq.seq_id: token for it in items if it.sample_after})
    s.manager.check_consistency()
    return [(it.seq.seq_id, it.start_pos, it.num_tokens, it.is_prefill, it.sample_after) for it in items]


def test_portions_under_the_budget_and_no_token_before_the_prompt_ends():
    s, _ = make()
    a = seq(0, 37)
    s.add(a)
    assert run_step(s) == [(0, 0, 16, True, False)]
    assert a.num_completion_tokens == 0 and a.status is SequenceStatus.WAITING
    assert run_step(s) == [(0, 16, 16, True, False)]
    assert run_step(s) == [(0, 32, 5, True, True)]
    assert a.num_completion_tokens == 1 and a.status is SequenceStatus.RUNNING
    assert run_step(s) == [(0, 37, 1, False, True)]        # the sampled token is the next input


def test_prefill_chunk_caps_one_request():
    s, _ = make(prefill_chunk=6)
    s.add(seq(0, 20)), s.add(seq(1, 5))
    assert run_step(s) == [(0, 0, 6, True, False), (1, 0, 5, True, True)]
    assert run_step(s) == [(1, 5, 1, False, True), (0, 6, 6, True, False)]


def test_decode_first_round_robin_and_reserve_for_waiting():
    s, _ = make(max_num_batched_tokens=10, max_num_seqs=3)
    for i in range(3):
        s.add(seq(i, 2, max_tokens=50))
    run_step(s)                                             # all three prompts fit one step
    assert [q.seq_id for q in s.running] == [0, 1, 2]
    s.add(seq(3, 30, max_tokens=50))
    # one waiting: decoding may use max_num_seqs - 1 requests and int(0.8 * 10) tokens
    assert run_step(s) == [(0, 2, 1, False, True), (1, 2, 1, False, True), (3, 0, 8, True, False)]
    assert run_step(s) == [(2, 2, 1, False, True), (0, 3, 1, False, True), (3, 8, 8, True, False)]


def test_stop_conditions():
    s, m = make()
    a, b, c = seq(0, 3, max_tokens=2), seq(1, 3, max_tokens=9), seq(2, 3, max_tokens=9, ignore_eos=True)
    for q in (a, b, c):
        s.add(q)
    run_step(s, token=5)
    run_step(s, token=9)                                    # 9 is the end-of-sequence token
    assert a.finish_reason == "max_tokens" and b.finish_reason == "eos" and c.finish_reason is None
    assert b.token_ids[-1] == 9                             # it stays in the output
    assert m.live_requests == [2]
    s2, _ = make(max_model_len=8)
    d = seq(0, 6, max_tokens=50)
    s2.add(d)
    run_step(s2), run_step(s2)
    assert d.finish_reason == "max_model_len" and d.num_tokens == 8
    with pytest.raises(ValueError, match="max_model_len"):
        s2.add(seq(1, 8))


def test_prompt_waits_for_pages_and_decode_sits_out():
    s, m = make(num_pages=6, page=4)                        # 24 tokens of cache
    a, b = seq(0, 15, max_tokens=20), seq(1, 12, max_tokens=20)
    s.add(a), s.add(b)
    assert run_step(s) == [(0, 0, 15, True, True)]          # b needs 3 pages, 2 are free: it waits
    assert not b.admitted and b in s.waiting
    with pytest.raises(ValueError, match="pages"):
        s.add(seq(2, 40))                                   # can never fit
    for _ in range(9):
        run_step(s)
    assert a.num_tokens == 25 and a.num_computed_tokens == 24 and a.status is SequenceStatus.RUNNING
    # a holds all six pages and wants a seventh; b still waits. Nothing can run: a is alone
    # among the admitted, so it ends, and b gets its turn.
    items = run_step(s)
    assert a.finish_reason == "cache_exhausted" and items == [(1, 0, 12, True, True)]
    assert s.finished_early == [a]


def test_preemption_recomputes_the_youngest():
    s, m = make(num_pages=4, page=4, max_num_batched_tokens=32)     # 16 tokens of cache
    a, b = seq(0, 6, max_tokens=20), seq(1, 6, max_tokens=20)
    s.add(a), s.add(b)
    assert run_step(s) == [(0, 0, 6, True, True), (1, 0, 6, True, True)]
    run_step(s), run_step(s)                                # both at 8 computed, 9 tokens: pages full
    assert m.groups[0].pool.num_free == 0
    items = run_step(s)                                     # neither can grow: b (admitted last) yields
    assert s.num_preemptions == 1 and b.num_preemptions == 1
    assert items == [(0, 8, 1, False, True)]
    assert b.status is SequenceStatus.WAITING and s.waiting[0] is b and b.num_computed_tokens == 0
    assert b.num_tokens == 9 and b.num_prefill_tokens == 9 and b.num_prompt_tokens == 6
    # b comes back when pages allow, recomputes all its nine tokens in one portion (which
    # samples its next token), and goes on decoding
    seen = []
    while not s.is_finished():
        seen += run_step(s)
    assert (1, 0, 9, True, True) in seen and (1, 9, 1, False, True) in seen
    assert a.is_finished and b.is_finished and b.token_ids[:9] == list(range(100, 106)) + [1, 1, 1]
    assert m.groups[0].pool.num_free == 4


@pytest.mark.parametrize("seed", range(5))
def test_random_traffic_always_finishes(seed):
    rng = random.Random(seed)
    s, m = make(num_pages=12, page=4, max_num_batched_tokens=12, max_num_seqs=3, prefill_chunk=7)
    seqs = [seq(i, rng.randint(1, 30), max_tokens=rng.randint(1, 25)) for i in range(12)]
    pending = list(seqs)
    for _ in range(3000):
        if pending and rng.random() < 0.3:
            s.add(pending.pop(0))
        if s.is_finished():
            if not pending:
                break
            continue
        items = s.schedule()
        assert items, "no progress while requests remain"
        assert sum(it.num_tokens for it in items) <= 12 and len(items) <= 3
        assert len({it.seq.seq_id for it in items}) == len(items)
        s.postprocess(items, {it.seq.seq_id: rng.randrange(20) for it in items if it.sample_after})
        m.check_consistency()
    assert s.is_finished() and not pending
    assert all(q.is_finished for q in seqs)
    assert m.groups[0].pool.num_free == 12 and not m.live_requests


# ---------------------------------------------------------------------------- prefix cache
def make_prefix(num_pages=16, page=4, **kw):
    cfg = EngineConfig(**{**dict(max_num_batched_tokens=16, max_num_seqs=4, max_model_len=64,
                                 kvcache_block_size=page, num_kvcache_blocks=num_pages), **kw})
    manager = CacheManager([(CacheNeed(2, 16, None), None)], page, num_pages, cfg.live_requests,
                           prefix_caching=True)
    return Scheduler(cfg, manager, eos_token_id=9), manager


def run_step_stored(s, token=1):
    """As run_step, and records the keys as stored, which the step function does in the engine."""
    items = s.schedule()
    for it in items:
        s.manager.commit(it.seq.seq_id, it.start_pos + it.num_tokens)
    s.postprocess(items, {it.seq.seq_id: token for it in items if it.sample_after})
    s.manager.check_consistency()
    return [(it.seq.seq_id, it.start_pos, it.num_tokens, it.is_prefill, it.sample_after) for it in items]


def test_a_later_prompt_starts_after_the_pages_it_shares():
    s, m = make_prefix()
    a = seq(0, 14, max_tokens=3)
    s.add(a)
    assert run_step_stored(s) == [(0, 0, 14, True, True)]
    b = seq(1, 14, max_tokens=2)                          # the same 14 tokens while a still decodes
    s.add(b)
    assert run_step_stored(s) == [(0, 14, 1, False, True), (1, 12, 2, True, True)]
    assert (a.num_cached_tokens, b.num_cached_tokens) == (0, 12)
    assert m.get(0).tables[0][:3] == m.get(1).tables[0][:3]
    while not s.is_finished():
        run_step_stored(s)
    assert m.groups[0].pool.num_free == 16
    # after both are gone their pages still serve a prompt that is one page longer
    c = Sequence(2, list(range(100, 114)) + [1, 1, 5, 6], SamplingParams(greedy=True, max_tokens=1))
    s.add(c)
    assert run_step_stored(s) == [(2, 16, 2, True, True)]  # a's decoded tokens 1, 1 filled page 3
    assert c.num_cached_tokens == 16


def test_a_preempted_request_finds_its_own_pages_again():
    s, m = make_prefix(num_pages=6, max_num_seqs=2)
    a, b = seq(0, 9, max_tokens=12), seq(1, 9, max_tokens=12)
    a.token_ids[0] = 55                                    # nothing in common
    s.add(a), s.add(b)
    for _ in range(40):
        if s.is_finished():
            break
        run_step_stored(s)
    assert s.is_finished() and s.num_preemptions >= 1
    assert b.num_preemptions >= 1 and b.num_cached_tokens >= 4   # the head of its pages outlived a's growth
    assert a.num_completion_tokens == 12 and b.num_completion_tokens == 12
    assert m.groups[0].pool.num_free == 6


def test_begun_prompts_are_finished_before_new_ones_are_begun():
    """More waiting prompts than the pool has pages for: those that hold pages are continued first, so
    they get to decode and to end. Taken in turn instead, every prompt would be begun, the pool would be
    shared out among prompts none of which can go on, and preemption would move pages around for ever."""
    s, m = make(num_pages=48, page=4, max_num_batched_tokens=16, max_num_seqs=4)
    seqs = [seq(i, 30, max_tokens=6) for i in range(12)]
    for q in seqs:
        s.add(q)
    begun = []
    for _ in range(400):
        if s.is_finished():
            break
        for item in run_step_stored(s):
            if item[3] and item[1] == 0:
                begun.append(item[0])
            # a prompt is never begun while an older one that holds pages still waits for its turn
        held_waiting = [q.seq_id for q in s.waiting if q.admitted]
        assert len(held_waiting) <= 2, held_waiting
    assert s.is_finished() and all(q.num_completion_tokens == 6 for q in seqs)
    assert begun == sorted(begun) and s.num_preemptions <= 2
    assert m.groups[0].pool.num_free == 48
