#!/usr/bin/env python3
"""Times one kernel family of tinyinfer_b200 at the shapes of a model, or a whole engine step with
few layers: the workload for per-kernel rooflines and for profiler captures.

    python benchmarks/kernel_microbench.py --kernel gemm --m 8 --n 6144 --k 4096
    python benchmarks/kernel_microbench.py --kernel gated_gemm --m 2048 --n 12288 --k 4096
    python benchmarks/kernel_microbench.py --kernel attention_decode --batch 8 --context 4096
    python benchmarks/kernel_microbench.py --kernel attention_prefill --tokens 2048
    python benchmarks/kernel_microbench.py --kernel rope_append --tokens 2048
    python benchmarks/kernel_microbench.py --kernel sample --batch 64 --topk 100
    python benchmarks/kernel_microbench.py --kernel decode_step --batch 8 --context 4096 --layers 4
    python benchmarks/kernel_microbench.py --kernel prefill_step --tokens 2048 --layers 4

Each call is timed with CUDA events around a captured CUDA graph of ``--iters`` launches (so host
overhead does not count); the weights rotate over several copies larger than L2 together. Prints
one JSON line with microseconds per call, GB/s and TFLOP/s, and their fraction of the measured
peaks (MEASURED_PEAKS.json beside bench.py, else the fallback figures)."""
import argparse
import json
import os
import random
import sys

ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from tinyinfer_b200 import ops  # noqa: E402


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        d = json.load(open(path))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def graph_time(fn, iters, use_graph=True):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if use_graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(iters):
                fn()
        g.replay()
        torch.cuda.synchronize()
        start.record()
        g.replay()
        end.record()
    else:
        start.record()
        for _ in range(iters):
            fn()
        end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters * 1e3          # microseconds


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--kernel", required=True, choices=["gemm", "gated_gemm", "attention_decode", "attention_prefill",
                                                       "rmsnorm", "rope_append", "sample", "decode_step", "prefill_step"])
    ap.add_argument("--topk", type=int, default=0, help="sample: top-k of every row (0: none; -1: every row greedy)")
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--prefix", type=int, default=0, help="attention_prefill: keys already in the cache before the tokens")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--preset", default="8b", help="decode_step / prefill_step: whose layer sizes (8b, 1.7b, 32b)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--pair-form", choices=["auto", "never", "always"], default="auto",
                    help="gemm, gated_gemm, steps: products of many tokens in the pair form where the library chooses it, "
                         "never, or always")
    ap.add_argument("--pair-min-ctas", type=int, default=None,
                    help="attention_prefill: fewest CTAs for which the two-tile kernel runs (default: the product's)")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    if a.pair_min_ctas is not None:
        ops.PAIR_MIN_CTAS = a.pair_min_ctas
    if a.pair_form == "never":
        ops.set_pair_form(False)
    elif a.pair_form == "always":
        ops.PAIR_MIN_TOKENS = 1
    hbm, tflops, source = peaks()
    torch.manual_seed(0)
    out = {"kernel": a.kernel, "peaks": source}

    if a.kernel in ("gemm", "gated_gemm"):
        gated = a.kernel == "gated_gemm"
        rows = 2 * a.n if gated else a.n
        x = torch.randn(a.m, a.k, device=dev).bfloat16()
        copies = max(2, min(8, int(400e6 // (rows * a.k * 2)) + 1))
        ws = [(torch.randn(rows, a.k, device=dev) * 0.02).bfloat16() for _ in range(copies)]
        i = [0]

        def fn():
            w = ws[i[0] % copies]
            i[0] += 1
            return ops.gated_linear(x, w) if gated else ops.linear(x, w)
        us = graph_time(fn, a.iters, not a.no_graph)
        byts = rows * a.k * 2 + a.m * a.k * 2 + a.m * a.n * 2
        flops = 2.0 * a.m * rows * a.k
        out.update(m=a.m, n=a.n, k=a.k, us=us, gbs=byts / us / 1e3, tflops=flops / us / 1e6)
    elif a.kernel == "rmsnorm":
        x = torch.randn(a.m, a.n, device=dev).bfloat16()
        w = torch.ones(a.n, device=dev)
        us = graph_time(lambda: ops.rmsnorm(x, w, 1e-6), a.iters, not a.no_graph)
        out.update(rows=a.m, size=a.n, us=us, gbs=2 * a.m * a.n * 2 / us / 1e3, tflops=0.0)
    elif a.kernel == "sample":
        n, v = a.batch, a.vocab
        logits = torch.randn(n, v, device=dev) * 3.0
        temp = torch.full((n,), 0.7, device=dev)
        topk = torch.full((n,), max(a.topk, 0), dtype=torch.int32, device=dev)
        greedy = torch.full((n,), 1 if a.topk < 0 else 0, dtype=torch.int32, device=dev)
        seed = torch.arange(n, dtype=torch.int64, device=dev)
        stream_id = torch.arange(n, dtype=torch.int32, device=dev)
        step = torch.zeros(n, dtype=torch.int32, device=dev)
        us = graph_time(lambda: ops.sample(logits, temp, topk, greedy, seed, stream_id, step), a.iters, not a.no_graph)
        out.update(rows=n, vocab=v, topk=a.topk, us=us, gbs=n * v * 4 / us / 1e3, tflops=0.0)
    elif a.kernel == "rope_append":
        hq, hkv, d, page, t = a.heads, a.kv_heads, a.head_dim, a.page_size, a.tokens
        qkv = torch.randn(t, (hq + 2 * hkv) * d, device=dev).bfloat16()
        pages = (t + page - 1) // page
        kv = torch.zeros(2, pages + 1, hkv, page, d, device=dev).bfloat16()
        bt = torch.arange(pages, dtype=torch.int32, device=dev)[None, :].contiguous()
        pos = torch.arange(t, dtype=torch.int32, device=dev)
        seq = torch.zeros(t, dtype=torch.int32, device=dev)
        w = torch.ones(d, device=dev)
        inv_freq = (1e6 ** (-torch.arange(0, d, 2, device=dev).float() / d)).contiguous()
        us = graph_time(lambda: ops.qk_norm_rope_append(
            qkv, num_heads=hq, num_kv_heads=hkv, head_dim=d, q_norm_weight=w, k_norm_weight=w, eps=1e-6, positions=pos,
            token_seq=seq, kv_cache=kv, block_table=bt, inv_freq=inv_freq, rotary_dim=d), a.iters, not a.no_graph)
        out.update(tokens=t, us=us, gbs=2 * t * (hq + 2 * hkv) * d * 2 / us / 1e3, tflops=0.0)
    elif a.kernel in ("attention_decode", "attention_prefill"):
        hq, hkv, d, page = a.heads, a.kv_heads, a.head_dim, a.page_size
        if a.kernel == "attention_decode":
            lens, q_lens = [a.context] * a.batch, [1] * a.batch
        else:
            lens, q_lens = [a.prefix + a.tokens], [a.tokens]
        per = [(n + page - 1) // page for n in lens]
        copies = max(1, min(6, int(300e6 // (sum(lens) * hkv * d * 4)) + 1))
        kvs = [torch.randn(2, sum(per) + 1, hkv, page, d, device=dev).bfloat16() for _ in range(copies)]
        table, nxt = [], 0
        for k in per:
            table.append(list(range(nxt, nxt + k)) + [-1] * (max(per) - k))
            nxt += k
        bt = torch.tensor(table, dtype=torch.int32, device=dev)
        pos = torch.tensor([p for n, ql in zip(lens, q_lens) for p in range(n - ql, n)], dtype=torch.int32, device=dev)
        seq = torch.tensor([s for s, ql in enumerate(q_lens) for _ in range(ql)], dtype=torch.int32, device=dev)
        q = torch.randn(pos.shape[0], hq, d, device=dev).bfloat16()
        rows_l, tiles_l, pair_tiles = ops.plan_attention(q_lens, [n - ql for n, ql in zip(lens, q_lens)])

        class Step:
            decode_rows = torch.tensor(rows_l or [0], dtype=torch.int32, device=dev)
            num_decode = len(rows_l)
            prefill_tiles = torch.tensor(tiles_l or [0, 0, 0, 0], dtype=torch.int32, device=dev)
            num_prefill_tiles = len(tiles_l) // 4
            num_pair_tiles = pair_tiles
            max_context = max(lens)
        i = [0]

        def fn():
            kv = kvs[i[0] % copies]
            i[0] += 1
            return ops.paged_attention(q, kv, positions=pos, token_seq=seq, block_table=bt, scale=d ** -0.5, step=Step)
        us = graph_time(fn, a.iters, not a.no_graph)
        if a.kernel == "attention_decode":
            byts = sum(lens) * hkv * d * 2 * 2
            flops = 4.0 * sum(lens) * hq * d
        else:
            byts = (a.prefix + a.tokens) * hkv * d * 2 * 2 + 2 * a.tokens * hq * d * 2
            flops = 4.0 * d * hq * (a.tokens * a.prefix + a.tokens * (a.tokens + 1) / 2)
        out.update(batch=len(lens), context=max(lens), us=us, gbs=byts / us / 1e3, tflops=flops / us / 1e6)
    else:
        from tinyinfer_b200 import EngineConfig
        from tinyinfer_b200.cli import preset_config
        from tinyinfer_b200.engine.batch import StepEntry
        from tinyinfer_b200.engine.llm import LLM
        cfg = preset_config(a.preset, num_hidden_layers=a.layers)
        eng = EngineConfig(max_num_batched_tokens=max(2048, a.tokens), max_num_seqs=a.batch, max_model_len=a.context,
                           kvcache_block_size=a.page_size, dtype="bfloat16", cuda_graphs=not a.no_graph,
                           num_kvcache_blocks=(a.context // a.page_size) * a.batch + 8 + a.tokens // a.page_size)
        llm = LLM(cfg, eng, random_weights=2)
        r = llm.runner
        rng = random.Random(0)
        for t in r.storage.kv:
            t.normal_(0, 1)
        steps = a.iters
        if a.kernel == "prefill_step":
            toks = [rng.randrange(1000) for _ in range(a.tokens)]

            def one(k):
                r.step([StepEntry(f"p{k}", toks, [a.tokens - 1])])
                r.release(f"p{k}")
        else:
            rids = [f"d{k}" for k in range(a.batch)]
            for rid in rids:
                r.admit(rid)
                r.manager.extend(rid, a.context - steps - 4)
                r.manager.commit(rid, a.context - steps - 4)

            def one(k):
                ops.argmax(r.step([StepEntry(rid, [rng.randrange(1000)], [0]) for rid in rids]))
        for k in range(3):
            one(k)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for k in range(3, 3 + steps):
            one(k)
        end.record()
        torch.cuda.synchronize()
        r.check_status()
        out.update(layers=a.layers, batch=a.batch, context=a.context, tokens=a.tokens,
                   us=start.elapsed_time(end) / steps * 1e3, gbs=0.0, tflops=0.0)
    ops.check_kernel_status()
    out["hbm_frac"] = out["gbs"] / hbm
    out["tensor_frac"] = out["tflops"] / tflops
    print(json.dumps(out))


if __name__ == "__main__":
    main()
