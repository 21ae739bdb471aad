"""Generation through the Python entry point and the command line, against the plain
implementation. Greedy tokens are checked by teacher forcing: at every generated position the
engine's token must have (up to rounding) the largest plain logit, so a tie flipped by rounding
does not fail the test while a wrong token does."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers
import plain_qwen3 as plain
import torch_ops
from tinyinfer_b200.sampling import SamplingParams

ROOT = Path(__file__).resolve().parent.parent


def check_greedy(folder, prompt, generated, tol):
    cfg, w = plain.read_model_folder(folder, torch.float64)
    logits = plain.forward(cfg, w, list(prompt) + list(generated)).numpy()
    for i, tok in enumerate(generated):
        row = logits[len(prompt) - 1 + i]
        assert row.max() - row[tok] <= tol * np.abs(logits).max(), (i, tok, int(row.argmax()))


def generate_and_check(llm, folder, cfg, tol):
    requests = helpers.random_requests(cfg, [1, 7, 16, 33, 50], seed=6)
    prompts = list(requests.values())
    outs = llm.generate(prompts, SamplingParams(greedy=True, max_tokens=8))
    assert [len(o["token_ids"]) for o in outs] == [8] * 5
    for p, o in zip(prompts, outs):
        assert o["all_token_ids"] == p + o["token_ids"] and o["finish_reason"] == "max_tokens"
        assert o["statistics"]["output_tokens"] == 8 and o["statistics"]["ttft"] > 0
        check_greedy(folder, p, o["token_ids"], tol)
    # one request at a time gives the same tokens as the batch did
    for p, o in zip(prompts[:3], outs[:3]):
        alone = llm.generate([p], SamplingParams(greedy=True, max_tokens=8))[0]
        check_greedy(folder, p, alone["token_ids"], tol)
    assert not llm.runner.manager.live_requests
    llm.runner.manager.check_consistency()
    return prompts, outs


def test_generate_with_plain_ops_on_cpu(tmp_path, monkeypatch):
    """The entry point's loop (schedule, step, sample, postprocess) with the kernels replaced by
    their plain statements; few pages, small budgets, so portions, waiting and reuse happen."""
    from tinyinfer_b200 import ops
    import tinyinfer_b200.engine.llm as llm_mod
    for name in torch_ops.ALL:
        monkeypatch.setattr(ops, name, getattr(torch_ops, name))
    monkeypatch.setattr(llm_mod, "require_cuda", lambda d: torch.device("cpu"))
    cfg = helpers.TINY_A
    folder = helpers.make_model_folder(tmp_path / "m", cfg, seed=3)
    llm = llm_mod.LLM(folder, dtype="float32", device="cpu", max_num_batched_tokens=24, max_num_seqs=3,
                      kvcache_block_size=4, num_kvcache_blocks=30, prefill_chunk=8, max_model_len=128, track_nll=True)
    prompts, outs = generate_and_check(llm, folder, cfg, 1e-5)
    # the perplexity statistic: exp of the mean NLL of the generated tokens under the plain model
    pcfg, w = plain.read_model_folder(folder, torch.float64)
    logp = torch.log_softmax(plain.forward(pcfg, w, prompts[2] + outs[2]["token_ids"]), dim=-1)
    nll = -sum(float(logp[len(prompts[2]) - 1 + i, t]) for i, t in enumerate(outs[2]["token_ids"]))
    assert abs(outs[2]["statistics"]["perplexity"] - np.exp(nll / 8)) < 1e-3 * np.exp(nll / 8)
    assert llm.runner.manager.stats()["groups"][0]["pages_taken"] > 30


def test_the_package_refuses_to_run_without_cuda(tmp_path):
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from tinyinfer_b200 import LLM
    folder = helpers.make_model_folder(tmp_path / "m", helpers.TINY_A, seed=3)
    with pytest.raises(RuntimeError, match="CUDA"):
        LLM(folder, num_kvcache_blocks=8)
    with pytest.raises(RuntimeError, match="CUDA"):
        LLM(folder, device="cpu", num_kvcache_blocks=8)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 3e-2)])
@pytest.mark.parametrize("name,page", [("A", 4), ("B", 8), ("Bw", 8), ("D", 64)])
def test_greedy_generation_on_the_gpu(tmp_path, name, page, dtype, tol):
    from tinyinfer_b200 import LLM
    cfg = helpers.TINY[name]
    folder = helpers.make_model_folder(tmp_path / "m", cfg, seed=3, dtype=dtype)
    llm = LLM(folder, dtype=dtype, max_num_batched_tokens=24, max_num_seqs=3, kvcache_block_size=page,
              num_kvcache_blocks=max(6, 120 // page), prefill_chunk=8, max_model_len=128)
    generate_and_check(llm, folder, cfg, tol)
    llm.runner.check_status()


@pytest.mark.gpu
def test_temperature_sampling_is_reproducible_and_follows_the_plain_sampler(tmp_path):
    from tinyinfer_b200 import LLM
    cfg = helpers.TINY_B
    folder = helpers.make_model_folder(tmp_path / "m", cfg, seed=1)
    requests = helpers.random_requests(cfg, [2, 11, 29, 64, 100], seed=7)
    prompts = list(requests.values())

    def run():
        llm = LLM(folder, dtype="float32", max_num_batched_tokens=64, max_num_seqs=4, kvcache_block_size=8,
                  num_kvcache_blocks=64, prefill_chunk=16, max_model_len=256, seed=5)
        params = [SamplingParams(temperature=1.0, topk=0, max_tokens=16, seed=77),
                  SamplingParams(temperature=0.7, topk=20, max_tokens=16),
                  SamplingParams(greedy=True, max_tokens=16),
                  SamplingParams(temperature=1.0, topk=100, max_tokens=16, seed=77),
                  SamplingParams(temperature=1.3, topk=5, max_tokens=16)]
        return llm.generate(prompts, params), params
    a, params = run()
    b, _ = run()
    assert [o["token_ids"] for o in a] == [o["token_ids"] for o in b]
    assert len({tuple(o["token_ids"]) for o in a}) == 5
    # teacher-forced check of every sampled token with the plain sampler on the plain logits
    pcfg, w = plain.read_model_folder(folder, torch.float64)
    agree = total = 0
    for i, (p, o, sp) in enumerate(zip(prompts, a, params)):
        logits = plain.forward(pcfg, w, p + o["token_ids"]).float().numpy()
        for step, tok in enumerate(o["token_ids"]):
            want = plain.sample(logits[len(p) - 1 + step], greedy=sp.greedy, temperature=sp.temperature,
                                topk=sp.topk, seed=5 if sp.seed is None else sp.seed, stream=i, step=step)
            agree += int(want == tok)
            total += 1
    assert agree >= total - 1, (agree, total)       # rounding may flip one near-tie


@pytest.mark.gpu
def test_command_line(tmp_path):
    folder = helpers.make_model_folder(tmp_path / "m", helpers.TINY_A, seed=3)
    cmd = [sys.executable, str(ROOT / "examples" / "generate.py"), "--model", str(folder), "--dtype", "fp32",
           "--prompt-ids", "5,17,3,200", "--prompt-len", "9", "--greedy", "--max-tokens", "6",
           "--max-num-seqs", "2", "--max-num-batched-tokens", "16", "--block-size", "4",
           "--num-kvcache-blocks", "32", "--max-model-len", "64"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    rows = [json.loads(l) for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(rows) == 2 and all(len(r["token_ids"]) == 6 for r in rows)
    check_greedy(folder, [5, 17, 3, 200], rows[0]["token_ids"], 5e-5)
    bad = subprocess.run(cmd + ["--speculative"], capture_output=True, text=True, timeout=600)
    assert bad.returncode != 0 and "does not build" in bad.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 3e-2)])
def test_page_pressure_waits_and_preempts_but_gives_the_same_tokens(tmp_path, dtype, tol):
    """With so few pages that prompts wait and a running request is preempted and recomputed, every
    request still gets the tokens it gets with plenty of pages (greedy, checked by teacher forcing)."""
    from tinyinfer_b200 import LLM
    cfg = helpers.TINY["C"]
    folder = helpers.make_model_folder(tmp_path / "m", cfg, seed=5, dtype=dtype)
    requests = helpers.random_requests(cfg, [60, 45, 70, 30, 55, 20], seed=9)
    prompts = list(requests.values())
    params = SamplingParams(greedy=True, max_tokens=40)
    roomy = LLM(folder, dtype=dtype, max_num_batched_tokens=64, max_num_seqs=4, kvcache_block_size=16,
                num_kvcache_blocks=64, prefill_chunk=32, max_model_len=160)
    want = roomy.generate(prompts, params)
    assert roomy.scheduler.num_preemptions == 0
    tight = LLM(folder, dtype=dtype, max_num_batched_tokens=64, max_num_seqs=4, kvcache_block_size=16,
                num_kvcache_blocks=14, prefill_chunk=32, max_model_len=160)
    got = tight.generate(prompts, params)
    assert tight.scheduler.num_preemptions > 0, "the pool was not tight enough to preempt"
    assert all(o["finish_reason"] == "max_tokens" and len(o["token_ids"]) == 40 for o in got)
    assert sum(o["statistics"]["preemptions"] for o in got) == tight.scheduler.num_preemptions
    for p, o in zip(prompts, got):
        check_greedy(folder, p, o["token_ids"], tol)
    same = sum(a["token_ids"] == b["token_ids"] for a, b in zip(want, got))
    assert same >= len(prompts) - 1          # a near-tie may flip under another batching
    tight.runner.check_status()
    tight.runner.manager.check_consistency()
    assert not tight.runner.manager.live_requests


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 3e-2)])
def test_shared_prompt_heads_are_taken_from_the_prefix_cache(tmp_path, dtype, tol):
    """Prompts with a common head: later ones take its pages over instead of computing them, while
    the first still runs and after it has ended, and a small pool hands kept pages out again.
    The tokens are those of an engine without the prefix cache and of the plain implementation."""
    from tinyinfer_b200 import LLM
    cfg = helpers.TINY["A"]
    folder = helpers.make_model_folder(tmp_path / "m", cfg, seed=6, dtype=dtype)
    head = helpers.random_requests(cfg, [53], seed=21)["r0"]
    tails = list(helpers.random_requests(cfg, [7, 19, 2, 30, 11, 16], seed=22).values())
    prompts = [head + t for t in tails] + [head[:40]]
    params = SamplingParams(greedy=True, max_tokens=12)
    common = dict(dtype=dtype, max_num_batched_tokens=48, max_num_seqs=3, kvcache_block_size=8,
                  prefill_chunk=24, max_model_len=128)
    cold = LLM(folder, num_kvcache_blocks=64, enable_prefix_caching=False, **common)
    want = cold.generate(prompts, params)
    assert all(o["num_cached_tokens"] == 0 for o in want)
    for pages in (64, 30):
        llm = LLM(folder, num_kvcache_blocks=pages, **common)
        assert llm.config.enable_prefix_caching
        got = llm.generate(prompts, params)
        cached = [o["num_cached_tokens"] for o in got]
        assert cached[0] == 0 and all(c % 8 == 0 for c in cached)
        # requests admitted beside the first find nothing or a first portion; those admitted after
        # the head has been stored take over its six full pages
        assert sum(cached) >= 96, cached
        if pages == 64:
            assert cached[4:6] == [48, 48], cached
            assert cached[6] == 32                                  # 40 tokens: 4 pages, one token left to run
        for p, o in zip(prompts, got):
            check_greedy(folder, p, o["token_ids"], tol)
        same = sum(a["token_ids"] == b["token_ids"] for a, b in zip(want, got))
        assert same >= len(prompts) - 1          # a near-tie may flip when the head is not run again
        # the same prompts once more: everything but the last page of each comes from the cache
        again = llm.generate(prompts, params)
        assert sum(o["num_cached_tokens"] for o in again) > sum(cached)
        for p, o in zip(prompts, again):
            check_greedy(folder, p, o["token_ids"], tol)
        llm.runner.check_status()
        llm.runner.manager.check_consistency()
        assert not llm.runner.manager.live_requests
        served = sum(cached) + sum(o["num_cached_tokens"] for o in again)
        hits = llm.runner.manager.stats()["prefix_hit_tokens"]     # counts a prompt that had to wait each time it asked
        assert hits == served if pages == 64 else hits >= served


@pytest.mark.gpu
def test_prefix_cache_is_off_where_a_window_gives_pages_back(tmp_path):
    from tinyinfer_b200 import LLM
    cfg = helpers.TINY["Bw"]                    # has sliding-window layers
    folder = helpers.make_model_folder(tmp_path / "m", cfg, seed=2, dtype="float32")
    kw = dict(dtype="float32", max_num_batched_tokens=32, max_num_seqs=2, kvcache_block_size=8,
              num_kvcache_blocks=32, max_model_len=96)
    assert LLM(folder, **kw).config.enable_prefix_caching is False
    with pytest.raises(ValueError, match="enable_prefix_caching"):
        LLM(folder, enable_prefix_caching=True, **kw)


def test_a_kernel_status_that_is_set_stops_generation(tmp_path, monkeypatch):
    """The kernels' status words come home with the sampled tokens; a step during which one was set
    (here by hand: nothing on a CPU sets it) raises when its tokens are read back, instead of handing
    them on: in the same call without overlap, in the next call with it."""
    from tinyinfer_b200 import ops
    import tinyinfer_b200.engine.llm as llm_mod
    for name in torch_ops.ALL:
        monkeypatch.setattr(ops, name, getattr(torch_ops, name))
    monkeypatch.setattr(llm_mod, "require_cuda", lambda d: torch.device("cpu"))
    folder = helpers.make_model_folder(tmp_path / "m", helpers.TINY_A, seed=3)
    words = ops.status_words(torch.device("cpu"))
    for overlap in (False, True):
        for word, code, text in ((0, 15, "gave up waiting"), (1, 1, "without a page"), (0, 23, "more key tiles")):
            llm = llm_mod.LLM(folder, dtype="float32", device="cpu", max_num_batched_tokens=24, max_num_seqs=3,
                              kvcache_block_size=4, num_kvcache_blocks=30, max_model_len=128, overlap_steps=overlap)
            llm.add_request([5, 6, 7], SamplingParams(greedy=True, max_tokens=6))
            llm.step()
            words[word] = code
            with pytest.raises(ops.KernelError, match=text):
                llm.step()                                   # the step that runs while the word is set
                assert overlap
                llm.step()                                   # with overlap its tokens are read back one call later
            assert words.tolist() == [0, 0]                  # reported once, then cleared
    words.zero_()


def test_overlapped_steps_give_the_tokens_of_steps_one_by_one(tmp_path, monkeypatch):
    """Launching a step before the tokens of the one before are read back changes nothing that a request
    sees: the same tokens, greedy and sampled, the same reasons to end (token limit, end-of-sequence token,
    which is found one step late and whose extra step is dropped), the same prefix-cache hits, every page
    given back."""
    from tinyinfer_b200 import ops
    import tinyinfer_b200.engine.llm as llm_mod
    for name in torch_ops.ALL:
        monkeypatch.setattr(ops, name, getattr(torch_ops, name))
    monkeypatch.setattr(llm_mod, "require_cuda", lambda d: torch.device("cpu"))
    cfg = helpers.TINY_A
    folder = helpers.make_model_folder(tmp_path / "m", cfg, seed=3)
    requests = helpers.random_requests(cfg, [1, 7, 16, 33, 50, 21, 9], seed=6)
    prompts = list(requests.values())
    prompts.append(prompts[3][:20] + [3, 1, 4])              # shares a head with another prompt
    params = [SamplingParams(greedy=i % 2 == 0, temperature=0.9, topk=40, max_tokens=3 + 2 * i, seed=11)
              for i in range(len(prompts))]

    def run(overlap, eos):
        llm = llm_mod.LLM(folder, dtype="float32", device="cpu", max_num_batched_tokens=24, max_num_seqs=3,
                          kvcache_block_size=4, num_kvcache_blocks=40, prefill_chunk=8, max_model_len=128,
                          overlap_steps=overlap, eos_token_id=eos, track_nll=True)
        outs = llm.generate(prompts, params)
        assert not llm.runner.manager.live_requests and llm.is_finished()
        llm.runner.manager.check_consistency()
        return outs, llm.runner.steps_run

    plain_outs, plain_steps = run(False, -1)
    # an end-of-sequence token that some request really draws part-way
    eos = plain_outs[5]["token_ids"][4]
    for end in (-1, eos):
        a, steps_a = run(False, end)
        b, steps_b = run(True, end)
        assert [o["token_ids"] for o in a] == [o["token_ids"] for o in b]
        assert [o["finish_reason"] for o in a] == [o["finish_reason"] for o in b]
        assert [o["num_cached_tokens"] for o in a] == [o["num_cached_tokens"] for o in b]
        for x, y in zip(a, b):
            # the same tokens under the same model; the extra step of a request that ended on a token puts one
            # more row into that step's batch, which moves the others' float32 sums by rounding
            assert abs(x["statistics"]["perplexity"] - y["statistics"]["perplexity"]) <= (
                0.0 if end < 0 else 1e-4 * x["statistics"]["perplexity"])
        if end >= 0:
            assert "eos" in [o["finish_reason"] for o in a]
        assert steps_b >= steps_a                            # a request that ended on a token ran one step more
