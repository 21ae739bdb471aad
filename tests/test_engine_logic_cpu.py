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


@pytest.mark.parametrize("name,page", [("A", 4), ("B", 8)])
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
