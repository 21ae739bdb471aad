"""The engine on the GPU against the plain implementation, in 32-bit and in bfloat16, in every
way of cutting the work: each request alone and whole; most of it in one step and the last 32
tokens one by one; in portions of changing size down to two tokens; and mixed, up to four live
requests, portions of some beside decoded tokens of others, with so few pages that they are used
again. The cache pool is poisoned with NaN so that a read outside a request's own keys shows."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
# Relative to the largest |logit| of the plain implementation. 32-bit: accumulation order only.
# bfloat16: activations are rounded to 8 bits of mantissa about ten times a layer.
TOL = {"float32": 5e-5, "bfloat16": 3e-2}
LENGTHS = [1, 7, 33, 90, 61, 47, 2, 70, 18, 120, 64, 65]


def traces_for(requests):
    return {
        "whole": helpers.trace_whole(requests),
        "tail": helpers.trace_decode_tail(requests, tail=32),
        "chunked": helpers.trace_chunked(requests, seed=1),
        "mixed": helpers.trace_mixed(requests, seed=2),
    }


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page", [("A", 4), ("B", 8), ("Bw", 8), ("C", 16), ("D", 64)])
def test_every_cut_matches_plain(tmp_path, name, page, dtype):
    from tinyinfer_b200.engine.replay import TraceSession
    cfg = helpers.TINY[name]
    folder = helpers.make_model_folder(tmp_path / name, cfg, seed=3, dtype=dtype)
    requests = helpers.random_requests(cfg, LENGTHS, seed=5)
    want = helpers.plain_logits(folder, requests)
    results = {}
    for tag, steps in traces_for(requests).items():
        session = TraceSession(folder, dtype, helpers.peak_tokens(steps, max(64, page)), page_size=page,
                               poison_cache=True)
        got = helpers.collect(session, steps)
        session.runner.check_status()
        assert {r: len(v) for r, v in got.items()} == {r: len(t) for r, t in requests.items()}, tag
        bad = helpers.first_bad(got, want, TOL[dtype])
        assert bad is None, (tag, bad)
        session.runner.manager.check_consistency()
        if tag == "mixed":
            stats = session.runner.manager.stats()["groups"]
            assert all(g["pages_taken"] > g["pages"] for g in stats), "pages were not used again"
        results[tag] = got
    # the cuts against each other: the same position, whatever the batching
    for tag in ("tail", "chunked", "mixed"):
        worst = max(float(np.abs(results[tag][r][p] - results["whole"][r][p]).max())
                    for r in requests for p in range(len(requests[r])))
        scale = max(float(np.abs(w).max()) for w in want.values())
        assert worst / scale <= TOL[dtype], (tag, worst / scale)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(tmp_path, dtype):
    """A request decoded token by token from its very first token for several hundred steps."""
    from tinyinfer_b200.engine.replay import TraceSession
    cfg = helpers.TINY["Bw"]
    folder = helpers.make_model_folder(tmp_path / "m", cfg, seed=9, dtype=dtype)
    requests = helpers.random_requests(cfg, [400], seed=1)
    want = helpers.plain_logits(folder, requests)
    toks = requests["r0"]
    steps = [{"step": i, "entries": [{"id": "r0", "tokens": [toks[i]], "want": [0]}],
              "end": ["r0"] if i == len(toks) - 1 else []} for i in range(len(toks))]
    session = TraceSession(folder, dtype, 448, page_size=8, poison_cache=True)
    got = helpers.collect(session, steps)
    assert helpers.first_bad(got, want, TOL[dtype]) is None
    # the first tokens: positions 0, 1, 2 exactly where a sequence starts
    for p in range(3):
        err = np.abs(got["r0"][p] - want["r0"][p]).max() / np.abs(want["r0"]).max()
        assert err <= TOL[dtype]


def test_graph_replay_equals_eager_steps(tmp_path):
    """Decode steps replayed from a captured CUDA graph give the very logits of eager steps."""
    from tinyinfer_b200.engine.replay import TraceSession
    cfg = helpers.TINY["D"]
    folder = helpers.make_model_folder(tmp_path / "m", cfg, seed=2, dtype="bfloat16")
    requests = helpers.random_requests(cfg, [300, 280, 290], seed=3)
    steps = []
    for i in range(240):           # three requests side by side, one token each a step
        steps.append({"step": i, "entries": [{"id": r, "tokens": [t[i]], "want": [0]} for r, t in requests.items()],
                      "end": []})
    out = {}
    for graphs in (False, True):
        session = TraceSession(folder, "bfloat16", 3 * 320, page_size=64, cuda_graphs=graphs, poison_cache=True)
        out[graphs] = helpers.collect(session, steps)
        session.runner.check_status()
        assert (session.runner.graph_replays > 200) == graphs
    for r in requests:
        for p in range(240):
            assert np.array_equal(out[True][r][p], out[False][r][p]), (r, p)
    want = helpers.plain_logits(folder, {r: t[:240] for r, t in requests.items()})
    assert helpers.first_bad(out[True], want, TOL["bfloat16"]) is None


def test_an_id_that_comes_back_gets_its_own_pages(tmp_path):
    """With CUDA graphs on, a decode step for the same requests as the step before patches the staged
    arrays instead of rebuilding them. A request that ends after such a step and whose id comes back
    in the next one, with one token, is another request: other pages, another state slot. Both live
    requests are compared with the plain implementation while the pool hands the ended request's page
    out again."""
    from tinyinfer_b200.engine.replay import TraceSession
    cfg = helpers.TINY["C"]
    folder = helpers.make_model_folder(tmp_path / "m", cfg, seed=7, dtype="bfloat16")
    rng = np.random.default_rng(4)
    first = [int(t) for t in rng.integers(0, cfg["vocab_size"], 12)]       # one page of 16
    again = [int(t) for t in rng.integers(0, cfg["vocab_size"], 68)]       # its fifth page is the ended request's
    other = [int(t) for t in rng.integers(0, cfg["vocab_size"], 40 + 4 + 68)]  # 7 + 5 pages: the whole pool of 12
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": first[:8], "want": [7]},
                                     {"id": "b", "tokens": other[:40], "want": [39]}], "end": []}]
    for i in range(4):                                                     # decode-only steps of "a" and "b"
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": [first[8 + i]], "want": [0]},
                                                      {"id": "b", "tokens": [other[40 + i]], "want": [0]}],
                      "end": ["a"] if i == 3 else []})
    for i in range(68):                                                    # the id "a" is back, one token a step
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": [again[i]], "want": [0]},
                                                      {"id": "b", "tokens": [other[44 + i]], "want": [0]}], "end": []})
    session = TraceSession(folder, "bfloat16", 192, page_size=16, poison_cache=True, cuda_graphs=True)
    got, upto, names = {}, {}, {}
    for st in steps:
        out = session.run_step(st)
        for row, e in enumerate(st["entries"]):
            name = names.setdefault(e["id"], e["id"])
            s0 = upto.get(name, 0)
            got.setdefault(name, {})[s0 + e["want"][0]] = out[row]
            upto[name] = s0 + len(e["tokens"])
        for rid in st["end"]:
            names[rid] = rid + "2"                                         # what comes under this id now is another request
        session.runner.manager.check_consistency()
    assert session.runner.graph_replays > 60
    assert session.runner.manager.stats()["groups"][0]["pages_taken"] > 12, "the ended request's page was not used again"
    assert session.runner.manager.stats()["groups"][0]["free_pages"] == 0
    want = helpers.plain_logits(folder, {"a": first, "a2": again, "b": other})
    bad = helpers.first_bad(got, want, TOL["bfloat16"])
    assert bad is None, bad


BIG = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096,
    num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    intermediate_size=12288, rms_norm_eps=1e-6, rope_theta=1000000.0, attention_bias=False,
    tie_word_embeddings=False, max_position_embeddings=4096)


@pytest.fixture(scope="module")
def benchmark_sized_model(tmp_path_factory):
    """Two layers with every width of the benchmark model (hidden 4096, 32/8 heads of 128, feed-forward
    12288, vocabulary 151,936, untied head), written once in 32-bit, with the plain implementation's
    logits for four short requests: from the weights as written, and from the matrices rounded to
    bfloat16, which is what an engine run in bfloat16 holds after loading this folder."""
    folder = helpers.make_model_folder(tmp_path_factory.mktemp("big") / "m", BIG, seed=6, dtype="float32", std=0.02)
    requests = helpers.random_requests(BIG, [150, 70, 33, 190], seed=2)
    want = {"float32": helpers.plain_logits(folder, requests),
            "bfloat16": helpers.plain_logits(folder, requests, matrices_as=torch.bfloat16)}
    return folder, requests, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_widths_of_the_benchmark_model_in_every_cut(benchmark_sized_model, dtype):
    """The shapes the tensor-core kernels are tuned for (and the 32-bit kernels at the same widths),
    through the engine in all four ways of cutting the work, with pages of 64 that are used again."""
    from tinyinfer_b200.engine.replay import TraceSession
    folder, requests, want = benchmark_sized_model
    cuts = {"whole": helpers.trace_whole(requests),
            "tail": helpers.trace_decode_tail(requests, tail=32),
            "chunked": helpers.trace_chunked(requests, seed=3),
            "mixed": helpers.trace_mixed(requests, seed=4, max_live=3)}
    model = None
    for tag, steps in cuts.items():
        session = TraceSession(folder, dtype, helpers.peak_tokens(steps), page_size=64, poison_cache=True,
                               model=model)
        model = session.model                      # six gigabytes of weights are loaded once for the four cuts
        got = helpers.collect(session, steps)
        session.runner.check_status()
        assert {r: len(v) for r, v in got.items()} == {r: len(t) for r, t in requests.items()}, tag
        bad = helpers.first_bad(got, want[dtype], TOL[dtype])
        assert bad is None, (tag, bad)
        session.runner.manager.check_consistency()
        if tag == "mixed":
            stats = session.runner.manager.stats()["groups"]
            assert all(g["pages_taken"] > g["pages"] for g in stats), "pages were not used again"
        del got, session


LONG = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=1031, hidden_size=1024,
    num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
    intermediate_size=3072, rms_norm_eps=1e-6, rope_theta=1000000.0, attention_bias=False,
    tie_word_embeddings=False, max_position_embeddings=4096)


def test_long_prompts_on_the_kernels_for_many_tokens(tmp_path):
    """Prompts of hundreds and thousands of tokens in large portions, in bfloat16: the steps in which the products
    run in the pair form (512 tokens and more), prompt attention with two query tiles a CTA (1,290 tokens x 32
    heads of 64), its tiles as halves (590 tokens), and with the keys shared out over CTAs (250 tokens behind
    1,950), next to single decoded tokens. Logits at the ends of the portions and of every decoded token
    against the plain implementation."""
    from tinyinfer_b200.engine.replay import TraceSession
    folder = helpers.make_model_folder(tmp_path / "m", LONG, seed=9, dtype="float32", std=0.03)
    requests = helpers.random_requests(LONG, [1300, 600, 2200], seed=5)
    want = helpers.plain_logits(folder, requests, matrices_as=torch.bfloat16)
    a, b, c = (requests[r] for r in requests)
    ra, rb, rc = list(requests)
    ends = lambda n: [n - 2, n - 1]
    steps = [
        {"step": 0, "entries": [{"id": ra, "tokens": a[:1290], "want": [0, 511, 1000, 1289]}], "end": []},
        {"step": 1, "entries": [{"id": ra, "tokens": a[1290:1291], "want": [0]},
                                {"id": rb, "tokens": b[:590], "want": [5, 589]}], "end": []},
        {"step": 2, "entries": [{"id": ra, "tokens": a[1291:1292], "want": [0]},
                                {"id": rb, "tokens": b[590:591], "want": [0]},
                                {"id": rc, "tokens": c[:1950], "want": [1949]}], "end": []},
        {"step": 3, "entries": [{"id": rc, "tokens": c[1950:], "want": [0, 100, 249]},
                                {"id": ra, "tokens": a[1292:1293], "want": [0]}], "end": []},
        {"step": 4, "entries": [{"id": ra, "tokens": a[1293:], "want": ends(7)},
                                {"id": rb, "tokens": b[591:], "want": ends(9)}], "end": [ra, rb, rc]},
    ]
    session = TraceSession(folder, "bfloat16", helpers.peak_tokens(steps), page_size=64, poison_cache=True)
    got = helpers.collect(session, steps)
    session.runner.check_status()
    bad = helpers.first_bad(got, want, TOL["bfloat16"])
    assert bad is None, bad
    assert sum(len(v) for v in got.values()) == sum(len(e["want"]) for st in steps for e in st["entries"])
    session.runner.manager.check_consistency()


def run_trace_program(folder, dtype, out, steps, max_tokens, page_size=16):
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
           "--out", str(out), "--max-tokens", str(max_tokens), "--page-size", str(page_size)]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    res = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stderr[-3000:]
    assert [l for l in res.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    """bin/trace_run as a user calls it: steps on standard input, <step>.f32 files out."""
    cfg = helpers.TINY["B"]
    folder = helpers.make_model_folder(tmp_path / "m", cfg, seed=4, dtype=dtype)
    requests = helpers.random_requests(cfg, [40, 3, 77, 64, 20, 65], seed=8)
    want = helpers.plain_logits(folder, requests)
    steps = helpers.trace_mixed(requests, seed=3)
    out = tmp_path / "out"
    run_trace_program(folder, dtype, out, steps, helpers.peak_tokens(steps))
    upto = {}
    scale = max(float(np.abs(w).max()) for w in want.values())
    for st in steps:
        wanted = sum(len(e["want"]) for e in st["entries"])
        data = np.fromfile(out / f"{st['step']}.f32", dtype="<f4").reshape(wanted, cfg["vocab_size"])
        row = 0
        for e in st["entries"]:
            s = upto.get(e["id"], 0)
            for w in e["want"]:
                err = np.abs(data[row] - want[e["id"]][s + w]).max() / scale
                assert err <= TOL[dtype], (st["step"], e["id"], s + w, err)
                row += 1
            upto[e["id"]] = s + len(e["tokens"])
