"""Many requests of random lengths through the entry point, far more than are served at once: with a
pool that holds them comfortably and with one so small that requests wait and are preempted, with and
without CUDA graphs and the prefix cache. Every request must end with the tokens it asked for, every
generated token is checked by teacher forcing against the plain implementation, and nothing is left
in the cache manager. (With more waiting prompts than pages an earlier scheduler began every prompt
and finished none.)"""
import random

import numpy as np
import pytest
import torch

import helpers
import plain_qwen3 as plain
from tinyinfer_b200.sampling import SamplingParams


def requests_for(cfg, n, seed):
    rng = random.Random(seed)
    heads = [[rng.randrange(cfg["vocab_size"]) for _ in range(rng.choice([17, 40, 64, 100]))] for _ in range(4)]
    prompts, params = [], []
    for _ in range(n):
        tail = [rng.randrange(cfg["vocab_size"]) for _ in range(rng.randint(1, 120))]
        prompts.append((rng.choice(heads) if rng.random() < 0.5 else []) + tail)
        params.append(SamplingParams(greedy=True, max_tokens=rng.randint(1, 60), ignore_eos=True))
    return prompts, params


@pytest.mark.gpu
@pytest.mark.parametrize("name,dtype,tol", [("C", "bfloat16", 3e-2), ("A", "float32", 5e-5), ("D", "bfloat16", 3e-2)])
@pytest.mark.parametrize("graphs,pages", [(True, 40), (False, 400)])
def test_many_requests(tmp_path, name, dtype, tol, graphs, pages):
    from tinyinfer_b200 import LLM
    cfg = helpers.TINY[name]
    folder = helpers.make_model_folder(tmp_path / "m", cfg, seed=4, dtype=dtype)
    prompts, params = requests_for(cfg, 40, seed=7)
    llm = LLM(folder, dtype=dtype, max_num_batched_tokens=96, max_num_seqs=6, kvcache_block_size=16,
              prefill_chunk=48, max_model_len=320, cuda_graphs=graphs, num_kvcache_blocks=pages,
              enable_prefix_caching=None if graphs else False)
    ids = [llm.add_request(p, sp) for p, sp in zip(prompts, params)]
    steps = 0
    while not llm.is_finished():
        assert llm.step() or llm.is_finished(), "the scheduler made no progress"   # the last call only reads tokens back
        steps += 1
        assert steps < 40 * 200, "the requests do not come to an end"
    llm.runner.check_status()
    llm.runner.manager.check_consistency()
    assert not llm.runner.manager.live_requests
    if pages == 400:
        assert llm.scheduler.num_preemptions == 0
    model = plain.read_model_folder(folder, torch.float64)
    for p, sp, i in zip(prompts, params, ids):
        seq = llm.sequences[i]
        generated = seq.token_ids[seq.num_prompt_tokens:]
        assert len(generated) == sp.max_tokens and seq.finish_reason == "max_tokens"
        logits = plain.forward(model[0], model[1], list(p) + generated).numpy()
        for k, tok in enumerate(generated):
            row = logits[len(p) - 1 + k]
            assert row.max() - row[tok] <= tol * np.abs(logits).max(), (i, k, tok, int(row.argmax()))
