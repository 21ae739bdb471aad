#!/usr/bin/env python3
"""Wall-clock throughput of LLM.generate over a synthetic workload, with the options and the
printed figures of the reference's benchmarks/benchmark_throughput.py:12-20,50-73
(output_tokens_per_s, computed_plus_output_tokens_per_s, requests_per_s, TTFT and TPOT per
request). The reference's workloads are text prompts (benchmarks/workloads.py); here seeded
random token ids of the same length classes stand in: short (32-64 tokens), long_prefill
(2-4 K tokens), shared_prefix (a common 512-token head and short tails). A fourth workload,
mixed, is a continuous-batching mix: prompts of 16-1024 tokens, 16-512 generated tokens each, half
of the requests greedy and half at temperature 0.7."""
import argparse
import json
import os
import random
import sys
import time

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from tinyinfer_b200.cli import add_engine_options, build_llm  # noqa: E402
from tinyinfer_b200.sampling import SamplingParams  # noqa: E402


def workload(name, vocab, rng, n):
    def ids(k):
        return [rng.randrange(vocab) for _ in range(k)]
    if name == "short":
        return [ids(rng.randint(32, 64)) for _ in range(n)]
    if name == "long_prefill":
        return [ids(rng.randint(2048, 4096)) for _ in range(n)]
    head = ids(512)
    return [head + ids(rng.randint(16, 64)) for _ in range(n)]


def main():
    ap = argparse.ArgumentParser()
    add_engine_options(ap)
    ap.add_argument("--workload", choices=["short", "long_prefill", "shared_prefix", "mixed"], default="short")
    ap.add_argument("--num-requests", type=int, default=16)
    ap.add_argument("--max-tokens", type=int, default=128)
    args = ap.parse_args()
    llm = build_llm(args)
    rng = random.Random(args.seed)
    vocab = llm.model.spec.vocab_size
    if args.workload == "mixed":
        prompts = [[rng.randrange(vocab) for _ in range(rng.randint(16, 1024))] for _ in range(args.num_requests)]
        params = [SamplingParams(greedy=i % 2 == 0, temperature=0.7, topk=100, max_tokens=rng.randint(16, 512),
                                 ignore_eos=True, seed=i) for i in range(args.num_requests)]
    else:
        prompts = workload(args.workload, vocab, rng, args.num_requests)
        params = SamplingParams(greedy=True, max_tokens=args.max_tokens, ignore_eos=True)
    warm = [rng.randrange(vocab) for _ in range(len(prompts[0]))]      # not a timed prompt: nothing of it is shared
    llm.generate([warm], SamplingParams(greedy=True, max_tokens=2, ignore_eos=True))
    t0 = time.perf_counter()
    outs = llm.generate(prompts, params)
    wall = time.perf_counter() - t0
    out_tokens = sum(len(o["token_ids"]) for o in outs)
    prompt_tokens = sum(len(p) for p in prompts)
    print(json.dumps({
        "workload": args.workload, "requests": len(prompts), "wall_s": wall, "steps": llm.runner.steps_run,
        "graph_replays": llm.runner.graph_replays, "preemptions": llm.scheduler.num_preemptions,
        "prefix_caching": bool(llm.config.enable_prefix_caching),
        "cached_prompt_tokens": sum(o["num_cached_tokens"] for o in outs),
        "output_tokens_per_s": out_tokens / wall,
        "computed_plus_output_tokens_per_s": (prompt_tokens + out_tokens) / wall,
        "requests_per_s": len(prompts) / wall,
        "mean_ttft_s": sum(o["statistics"]["ttft"] for o in outs) / len(outs),
        "mean_tpot_s": sum(o["statistics"]["tpot"] or 0.0 for o in outs) / len(outs)}))


if __name__ == "__main__":
    main()
