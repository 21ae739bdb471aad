"""The engine's logic (cache, batching, step function, replay) on the CPU, with the CUDA kernels
replaced by their plain PyTorch statements (tests/torch_ops.py). What is under test is the
host side: block tables, page reuse, positions, the order of appends and reads; the kernels
themselves are tested on the GPU."""
import numpy as np
import pytest
import torch

import helpers
import torch_ops


@pytest.fixture
def cpu_ops(monkeypatch):
    from tinyinfer_b200 import ops
    for name in torch_ops.ALL:
        monkeypatch.setattr(ops, name, getattr(torch_ops, name))
    return ops


def session_for(folder, max_tokens, page_size, poison=True):
    from tinyinfer_b200.config import load_config
    from tinyinfer_b200.engine.replay import TraceSession
    from tinyinfer_b200.weights import load_weights
    arch, config = load_config(folder)
    model = arch.model_factory(config, torch.float32, torch.device("cpu"))
    load_weights(model, folder)
    return TraceSession(None, "float32", max_tokens, page_size=page_size, model=model, poison_cache=poison)


@pytest.mark.parametrize("name,page", [("A", 4), ("B", 8), ("Bw", 8)])
def test_every_cut_matches_plain_on_cpu(tmp_path, cpu_ops, name, page):
    cfg = helpers.TINY[name]
    folder = helpers.make_model_folder(tmp_path / name, cfg, seed=3)
    requests = helpers.random_requests(cfg, [1, 7, 33, 90, 61, 47, 2, 70, 18, 120, 64, 65], seed=5)
    want = helpers.plain_logits(folder, requests)
    traces = {
        "whole": helpers.trace_whole(requests),
        "tail": helpers.trace_decode_tail(requests, tail=32),
        "chunked": helpers.trace_chunked(requests, seed=1),
        "mixed": helpers.trace_mixed(requests, seed=2),
    }
    for tag, steps in traces.items():
        session = session_for(folder, helpers.peak_tokens(steps), page)
        got = helpers.collect(session, steps)
        assert {r: len(v) for r, v in got.items()} == {r: len(t) for r, t in requests.items()}, tag
        bad = helpers.first_bad(got, want, 2e-5)
        assert bad is None, (tag, bad)
        session.runner.manager.check_consistency()
        assert not session.runner.manager.live_requests
        if tag == "mixed":
            stats = session.runner.manager.stats()["groups"]
            assert all(g["pages_taken"] > g["pages"] for g in stats), "pages were not used again"


def test_a_step_takes_pages_for_all_its_entries_or_for_none(tmp_path, cpu_ops):
    """A step whose second entry cannot get its pages leaves the cache as it was: the first entry's
    pages are not kept, and a request that the step itself would have admitted is not live."""
    from tinyinfer_b200.cache import CacheExhausted
    from tinyinfer_b200.engine.batch import StepEntry
    cfg = helpers.TINY_A
    folder = helpers.make_model_folder(tmp_path / "m", cfg, seed=3)
    session = session_for(folder, max_tokens=64, page_size=4)          # 16 pages
    runner = session.runner
    runner.step([StepEntry("old", list(range(20)), [19])])             # 5 pages held
    before = runner.manager.stats()
    with pytest.raises(CacheExhausted):
        # 'old' could grow by 12 tokens (3 pages) alone, and 'new' could get 36 tokens (9 pages) alone: not both
        runner.step([StepEntry("old", list(range(12)), [11]), StepEntry("new", list(range(36)), [35])])
    assert runner.manager.stats() == before
    assert "new" not in runner.manager and runner.manager.get("old").length == 20
    runner.manager.check_consistency()
    with pytest.raises(ValueError):                                    # a bad token is seen before anybody is admitted
        runner.step([StepEntry("late", [1, 2, cfg["vocab_size"]], [2])])
    assert "late" not in runner.manager and runner.manager.stats() == before
    logits = runner.step([StepEntry("old", list(range(12)), [11])])    # the step that fits still runs
    assert logits.shape == (1, cfg["vocab_size"])


def test_patching_the_last_decode_step_needs_the_same_admissions():
    """The staged arrays of a decode step are patched for the next one only if the requests are the
    same admissions: an id that ended and came back holds other pages and another state slot."""
    from tinyinfer_b200.engine.batch import BatchBuffers, StepEntry
    buffers = BatchBuffers("cpu", max_tokens=8, max_seqs=4, max_blocks=4, num_groups=1)
    entries = [StepEntry("a", [5], [0]), StepEntry("b", [6], [0])]
    ctx = buffers.build(entries, [3, 9], [0, 1], [[[7], [2, 4, 8]]], fixed_layout=True, admissions=[1, 2])
    assert ctx.block_tables[0].tolist() == [[7, -1, -1, -1], [2, 4, 8, -1]]
    same = buffers.advance_decode([1, 2], 0, [11, 12], [4, 10], [[[7, 3], [2, 4, 8]]])
    assert same is ctx and ctx.block_tables[0].tolist() == [[7, 3, -1, -1], [2, 4, 8, -1]]
    assert ctx.positions.tolist() == [4, 10] and ctx.token_ids.tolist() == [11, 12]
    # 'a' ended and a new 'a' (admission 3) brings one token: tables of equal length, other pages
    assert buffers.advance_decode([3, 2], 0, [1, 13], [0, 11], [[[5], [2, 4, 8]]]) is None
    # without admission numbers nothing is remembered to patch
    buffers.build(entries, [3, 9], [0, 1], [[[7], [2, 4, 8]]], fixed_layout=True)
    assert buffers.advance_decode([1, 2], 0, [11, 12], [4, 10], [[[7, 3], [2, 4, 8]]]) is None


def test_rows_that_fill_a_batch_up_hold_a_page_and_a_state_slot_of_their_own():
    """A decode batch is filled up to the size of its captured graph with rows of a request that is
    none: its one page and its state slot are ones that no request holds, so a part that writes keys
    or state for every row of the step alike spoils nothing."""
    from tinyinfer_b200.engine.batch import BatchBuffers, StepEntry
    buffers = BatchBuffers("cpu", max_tokens=8, max_seqs=4, max_blocks=4, num_groups=1)
    entries = [StepEntry("a", [5], [0]), StepEntry("b", [6], [0]), StepEntry("c", [7], [0])]
    ctx = buffers.build(entries, [3, 9, 1], [2, 0, 1], [[[7], [2, 4, 8], [6]]], fixed_layout=True, pad_to=4,
                        pad_pages=[99], pad_slot=3)
    assert ctx.num_seqs == 4 and ctx.num_real_seqs == 3
    assert ctx.state_slots.tolist() == [2, 0, 1, 3]
    assert ctx.block_tables[0][3].tolist() == [99, -1, -1, -1] and ctx.positions.tolist() == [3, 9, 1, 0]


def test_the_cache_keeps_a_state_slot_for_the_rows_that_fill_up():
    from tinyinfer_b200.cache import CacheManager, CacheStorage
    from tinyinfer_b200.parts import StateNeed
    needs = [(None, StateNeed((5,), torch.float32))]
    manager = CacheManager(needs, 8, 4, 3)
    storage = CacheStorage(needs, manager, torch.float32, "cpu")
    slots = []
    for rid in "abc":
        manager.admit(rid)
        slots.append(manager.get(rid).state_slot)
    assert sorted(slots) == [0, 1, 2] and CacheStorage.dump_slot(manager) == 3
    assert storage.state[0].shape == (4, 5)


def test_an_id_that_comes_back_is_another_admission(tmp_path, cpu_ops):
    from tinyinfer_b200.engine.batch import StepEntry
    folder = helpers.make_model_folder(tmp_path / "m", helpers.TINY_A, seed=3)
    runner = session_for(folder, max_tokens=64, page_size=4).runner
    runner.step([StepEntry("a", [1, 2, 3], [])])
    first = runner.manager.get("a").serial
    runner.release("a")
    runner.step([StepEntry("a", [4], [])])
    assert runner.manager.get("a").serial != first
