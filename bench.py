#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens/s of a Qwen3-8B-shaped model with random
weights (bfloat16), plus a 2,048-token prefill, decode at batch 1 and 64, an end-to-end number
through the Python entry point, and the decode step's HBM roofline.

    python bench.py --gpus 1 --steps K --warmup W        prints ONE JSON line

A step is one decode step of the whole batch. ``value`` is timed on the device with CUDA events
around K steps that are fed from host token lists without reading results back; ``e2e`` runs the
same K steps through ``LLM.step()`` (scheduler, pinned host-to-device copy of the step's inputs,
sampling, device-to-host read of the tokens). The weights (15 GB) exceed L2, so no flush is
needed between steps. Peaks come from MEASURED_PEAKS.json beside this file if present.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        data = json.loads(path.read_text())
        return {k: float(data.get(k, FALLBACK_PEAKS[k])) for k in FALLBACK_PEAKS}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-i", "0",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        clocks, maxes, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                maxes.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None,
                "sm_max_mhz": max(maxes) if maxes else None, "samples": len(clocks),
                "reasons": sorted(reasons)}


def model_numbers(cfg, layers):
    """Bytes a decode step must read and flops of a prefill, from the configuration."""
    h, i, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    d, hq, hkv = cfg.resolved_head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    per_layer = h * (hq + 2 * hkv) * d + hq * d * h + 3 * h * i          # matrix elements
    norms = 2 * h + 2 * d
    weight_bytes = layers * (per_layer * 2 + norms * 4) + v * h * 2 + h * 4  # lm_head read once
    kv_bytes_per_token = layers * 2 * hkv * d * 2
    return dict(per_layer=per_layer, weight_bytes=weight_bytes, kv_bytes_per_token=kv_bytes_per_token)


def prefill_flops(cfg, layers, t, wanted_rows):
    h, v = cfg.hidden_size, cfg.vocab_size
    d, hq = cfg.resolved_head_dim, cfg.num_attention_heads
    per_layer = model_numbers(cfg, layers)["per_layer"]
    gemm = 2.0 * per_layer * t * layers
    attn = 4.0 * d * hq * (t * (t + 1) / 2.0) * layers               # causal q.k and p.v
    return gemm + attn + 2.0 * v * h * wanted_rows


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0: all)")
    ap.add_argument("--model-size", default="8b")
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--skip-points", action="store_true", help="only the headline batch")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference does not install offline: pip finds no torch>=2.4 in the wheelhouse, and with "
                          "--no-deps its extension fails to build (linear.cu: cutlass/cutlass.h not found; "
                          "third_party/cutlass is not shipped); its engine also needs a real checkpoint with a tokenizer"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine is single-GPU by design (got --gpus {args.gpus})")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from tinyinfer_b200 import EngineConfig, SamplingParams
    from tinyinfer_b200.cli import PRESETS
    from tinyinfer_b200.config import Qwen3Config
    from tinyinfer_b200.engine.batch import StepEntry
    from tinyinfer_b200.engine.llm import LLM
    from tinyinfer_b200 import ops

    peaks, peak_source = load_peaks()
    full = Qwen3Config.from_dict(dict(PRESETS[args.model_size], architectures=["Qwen3ForCausalLM"]))
    layers_full = full.num_hidden_layers
    layers = args.layers or layers_full
    cfg = Qwen3Config.from_dict(dict(PRESETS[args.model_size], architectures=["Qwen3ForCausalLM"],
                                     num_hidden_layers=layers))
    page = args.page_size
    ctx_len = args.context
    batches = [args.batch] if args.skip_points else sorted({1, args.batch, 64})
    max_batch = max(batches)
    pages_per_req = (ctx_len + page - 1) // page
    engine = EngineConfig(max_num_batched_tokens=max(2048, max_batch), max_num_seqs=max_batch,
                          max_model_len=ctx_len, kvcache_block_size=page,
                          num_kvcache_blocks=pages_per_req * max_batch + 8, dtype="bfloat16",
                          max_live_requests=max_batch + 2)
    llm = LLM(cfg, engine, random_weights=2)
    runner = llm.runner
    numbers = model_numbers(cfg, layers)
    rng = random.Random(0)
    vocab = cfg.vocab_size

    def event_time(fn):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end)

    def fast_forward(rid, length):
        """Gives request ``rid`` pages for ``length`` tokens without computing them: the cache
        holds the random values it was filled with, which costs a decode step the same reads."""
        runner.admit(rid)
        runner.manager.extend(rid, length)
        runner.manager.commit(rid, length)

    for t in runner.storage.kv:
        if t is not None:
            t.normal_(0.0, 1.0)

    # ------------------------------------------------------------------ prefill of 2,048 tokens
    prompt = [rng.randrange(vocab) for _ in range(2048)]

    def prefill_once(tag):
        runner.step([StepEntry(tag, prompt, [len(prompt) - 1])])
        runner.release(tag)
    for i in range(2):
        prefill_once(f"pw{i}")
    prefill_ms = min(event_time(lambda i=i: prefill_once(f"p{i}")) for i in range(3))
    pf_flops = prefill_flops(cfg, layers, len(prompt), 1)
    prefill = {"value": len(prompt) / (prefill_ms / 1e3), "tokens": len(prompt), "ms": prefill_ms,
               "frac": pf_flops / (prefill_ms / 1e3) / (peaks["bf16_tflops_sustained"] * 1e12),
               "tflops": pf_flops / (prefill_ms / 1e3) / 1e12, "peak_tflops": peaks["bf16_tflops_sustained"]}

    # ------------------------------------------------------------------ decode, device-timed
    def decode_run(batch, steps, warmup, sample_clocks=False):
        total = steps + warmup
        start_len = ctx_len - total
        rids = [f"d{batch}_{i}" for i in range(batch)]
        for rid in rids:
            fast_forward(rid, start_len)
        feeds = [[rng.randrange(vocab) for _ in range(batch)] for _ in range(total)]

        def one(step_tokens):
            logits = runner.step([StepEntry(rid, [tok], [0]) for rid, tok in zip(rids, step_tokens)])
            ops.argmax(logits)
        for k in range(warmup):
            one(feeds[k])
        sampler = ClockSampler()
        if sample_clocks:
            sampler.start()
        launches0 = ops.launch_count()
        ms = event_time(lambda: [one(feeds[warmup + k]) for k in range(steps)])
        launches = ops.launch_count() - launches0
        clocks = sampler.stop() if sample_clocks else None
        mean_ctx = start_len + warmup + (steps + 1) / 2.0
        for rid in rids:
            runner.release(rid)
        return dict(ms_per_step=ms / steps, tok_s=batch * steps / (ms / 1e3), launches=launches, clocks=clocks,
                    bytes=numbers["weight_bytes"] + batch * mean_ctx * numbers["kv_bytes_per_token"])

    head = decode_run(args.batch, args.steps, args.warmup, sample_clocks=True)
    points = {}
    for b in batches:
        if b == args.batch:
            points[f"decode_b{b}"] = head["tok_s"]
        else:
            points[f"decode_b{b}"] = decode_run(b, max(8, args.steps // 2), args.warmup)["tok_s"]
    achieved = head["bytes"] / (head["ms_per_step"] / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "peaks": peak_source}

    # ------------------------------------------------------------------ end to end through LLM.step()
    total = args.steps + args.warmup
    slack = 2 * args.batch + 8                         # tokens decoded while other prompts still prefill
    prompt_len = ctx_len - total - slack - 1
    params = SamplingParams(greedy=True, max_tokens=total + slack, ignore_eos=True)
    for _ in range(args.batch):
        llm.add_request([rng.randrange(vocab) for _ in range(prompt_len)], params)
    while llm.scheduler.waiting:                      # prompts, in portions, until all decode
        llm.step()
    for _ in range(args.warmup - 1):
        llm.step()
    h2d0 = runner.buffers.bytes_copied
    t0 = time.perf_counter()
    e2e_ms = event_time(lambda: [llm.step() for _ in range(args.steps)])
    wall_ms = (time.perf_counter() - t0) * 1e3
    h2d = (runner.buffers.bytes_copied - h2d0) / args.steps
    e2e = {"value": args.batch * args.steps / (max(e2e_ms, wall_ms) / 1e3), "unit": "tokens/s",
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": args.batch * 4, "ms_per_step": max(e2e_ms, wall_ms) / args.steps}

    out = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen3-{args.model_size.upper()} shape, random weights)",
        "value": head["tok_s"],
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random-init weights",
        "config": {"model": f"qwen3-{args.model_size}-shape", "layers": layers, "layers_full": layers_full,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.resolved_head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": args.batch, "seq_len": ctx_len, "prefill_tokens": len(prompt),
                   "page_size": page, "parallelism": "single-gpu",
                   "l2": f"inputs>L2 (weights {numbers['weight_bytes'] / 1e9:.1f} GB read per step)",
                   "cache_fill": "random for device-timed decode, real prefill for e2e"},
        "clocks": head["clocks"], "e2e": e2e, "gpu_launches": head["launches"],
        "prefill": prefill, "roofline": roofline, "points": points,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
