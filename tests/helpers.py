"""Test helpers: tiny Qwen3 configurations, model folders in temporary places, traces cut in the
ways the engine must be indifferent to, and the comparison with the plain implementation."""
from __future__ import annotations

import json
import random
from pathlib import Path
from typing import Dict, List, Sequence

import numpy as np
import torch

import plain_qwen3 as plain

# Two tiny configurations that differ in every size and option (A and B: the two the benchmark's
# correctness workloads name, B with a head size that is not hidden / heads and three kv heads), the
# same B with a sliding-window layer (Bw), and two whose head sizes reach the tensor-core kernels.
TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=256, hidden_size=64,
    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
    intermediate_size=128, rms_norm_eps=1e-6, rope_theta=10000.0, attention_bias=False,
    tie_word_embeddings=True, max_position_embeddings=512)
TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=384, hidden_size=96,
    num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=3, head_dim=32,
    intermediate_size=160, rms_norm_eps=1e-5, rope_theta=1000000.0, attention_bias=False,
    tie_word_embeddings=False, max_position_embeddings=1024)
TINY_BW = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=389, hidden_size=96,
    num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=2, head_dim=32,
    intermediate_size=176, rms_norm_eps=1e-5, rope_theta=1000000.0, attention_bias=False,
    tie_word_embeddings=False, max_position_embeddings=1024, sliding_window=40,
    layer_types=["full_attention", "sliding_attention", "full_attention"])
TINY_C = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=1000, hidden_size=320,
    num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
    intermediate_size=448, rms_norm_eps=1e-6, rope_theta=500000.0, attention_bias=False,
    tie_word_embeddings=False, max_position_embeddings=2048)
TINY_D = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=515, hidden_size=256,
    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1, head_dim=128,
    intermediate_size=384, rms_norm_eps=1e-6, rope_theta=1000000.0, attention_bias=False,
    tie_word_embeddings=True, max_position_embeddings=2048, sliding_window=96,
    use_sliding_window=True, max_window_layers=1)
TINY = {"A": TINY_A, "B": TINY_B, "Bw": TINY_BW, "C": TINY_C, "D": TINY_D}


def make_model_folder(folder, cfg: dict, seed: int, dtype: str = "float32", std: float = 0.05) -> Path:
    """Writes a random model through the framework's own random-weights mode."""
    from tinyinfer_b200.config import Qwen3Config
    from tinyinfer_b200.weights import write_random_model
    import tinyinfer_b200.models  # noqa: F401
    return write_random_model(folder, Qwen3Config.from_dict(cfg), seed, dtype=dtype, std=std)


def random_requests(cfg: dict, lengths: Sequence[int], seed: int) -> Dict[str, List[int]]:
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(cfg["vocab_size"]) for _ in range(n)] for i, n in enumerate(lengths)}


# ----------------------------------------------------------------------------- traces
def trace_whole(requests) -> List[dict]:
    """Each request alone and whole, logits wanted everywhere."""
    return [{"step": k, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
             "end": [rid]} for k, (rid, toks) in enumerate(requests.items())]


def trace_decode_tail(requests, tail: int = 32) -> List[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps, k = [], 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": k, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        k += 1
        for p in range(head, len(toks)):
            steps.append({"step": k, "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
            k += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def chunk_plan(n: int, rng: random.Random) -> List[int]:
    """Portions of changing size, down to two tokens, that sum to n."""
    sizes, left = [], n
    menu = [2, 3, 5, 7, 2, 13, 16, 17, 31, 2, 64, 9]
    while left > 0:
        c = min(left, rng.choice(menu))
        if left - c == 1:          # never leave a single trailing token by accident: merge it
            c = left
        sizes.append(c)
        left -= c
    return sizes


def trace_chunked(requests, seed: int = 0) -> List[dict]:
    rng = random.Random(seed)
    steps, k = [], 0
    for rid, toks in requests.items():
        start = 0
        plan = chunk_plan(len(toks), rng)
        for ci, c in enumerate(plan):
            steps.append({"step": k, "entries": [{"id": rid, "tokens": toks[start:start + c],
                                                  "want": list(range(c))}],
                          "end": [rid] if ci == len(plan) - 1 else []})
            start += c
            k += 1
    return steps


def trace_mixed(requests, seed: int = 0, max_live: int = 4, decode_tail: int = 12) -> List[dict]:
    """Up to ``max_live`` requests live at a time; every step batches portions of some prompts
    beside single decoded tokens of others; a request is left out of a step now and then;
    finished requests end, so their pages go to those that start later."""
    rng = random.Random(seed)
    plans = {}
    for rid, toks in requests.items():
        tail = min(decode_tail, max(0, len(toks) - 2))
        plans[rid] = chunk_plan(len(toks) - tail, rng) + [1] * tail
    waiting = list(requests)
    live: List[str] = []
    done_upto = {rid: 0 for rid in requests}
    steps, k = [], 0
    while waiting or live:
        while waiting and len(live) < max_live:
            live.append(waiting.pop(0))
        chosen = [rid for rid in live if rng.random() > 0.2] or [live[0]]
        entries, ended = [], []
        for rid in chosen:
            c = plans[rid].pop(0)
            s = done_upto[rid]
            entries.append({"id": rid, "tokens": requests[rid][s:s + c], "want": list(range(c))})
            done_upto[rid] = s + c
            if not plans[rid]:
                ended.append(rid)
        for rid in ended:
            live.remove(rid)
        steps.append({"step": k, "entries": entries, "end": ended})
        k += 1
    return steps


def peak_tokens(steps, grain: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``grain``."""
    held: Dict[str, int] = {}
    peak = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum((n + grain - 1) // grain * grain for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


# ----------------------------------------------------------------------------- running
def collect(session, steps) -> Dict[str, Dict[int, np.ndarray]]:
    """Runs ``steps`` through a TraceSession; returns request -> position -> logits row."""
    got: Dict[str, Dict[int, np.ndarray]] = {}
    upto: Dict[str, int] = {}
    for st in steps:
        out = session.run_step(st)
        row = 0
        for e in st["entries"]:
            s = upto.get(e["id"], 0)
            for w in e["want"]:
                got.setdefault(e["id"], {})[s + w] = out[row]
                row += 1
            upto[e["id"]] = s + len(e["tokens"])
        for rid in st["end"]:
            upto.pop(rid, None)
        assert out is None or row == out.shape[0]
    return got


def plain_logits(folder, requests, matrices_as=None) -> Dict[str, np.ndarray]:
    """``matrices_as=torch.bfloat16``: the matrices of the folder (every tensor of two dimensions)
    are rounded to that type first, as an engine does that loads a 32-bit folder to run in bfloat16."""
    cfg, w = plain.read_model_folder(folder, torch.float64)
    if matrices_as is not None:
        w = {n: t.to(matrices_as).to(torch.float64) if t.dim() == 2 else t for n, t in w.items()}
    return {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in requests.items()}


def worst_error(got, want) -> float:
    """Largest |engine - plain| over all collected rows, relative to the largest |plain| logit."""
    worst, scale = 0.0, 0.0
    for rid, rows in got.items():
        scale = max(scale, float(np.abs(want[rid]).max()))
        for pos, row in rows.items():
            assert np.isfinite(row).all(), f"non-finite logits at {rid}[{pos}]"
            worst = max(worst, float(np.abs(row.astype(np.float64) - want[rid][pos]).max()))
    return worst / scale


def first_bad(got, want, tol: float):
    """(request, position, error) of the first row beyond ``tol`` (relative), or None."""
    scale = max(float(np.abs(w).max()) for w in want.values())
    for rid in sorted(got):
        for pos in sorted(got[rid]):
            err = float(np.abs(got[rid][pos].astype(np.float64) - want[rid][pos]).max()) / scale
            if not err <= tol:
                return rid, pos, err
    return None
