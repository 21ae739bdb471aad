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

Beside the headline the line carries ``configs``: the other benchmark configurations, each with
its own sizes: ``qwen3_32b`` (64 layers, 32 requests at 8,192-token contexts, pages sized from free
memory), ``qwen3_1p7b_mix`` (64 requests of mixed lengths through the scheduler, prompts in portions
of 512 beside decoded tokens) and ``cpu_baseline_s`` (the tiny configurations through the plain
CPU implementation of the tests, in seconds, beside the engine's time for the same requests).
``--skip-extras`` leaves them out.

``--impl reference`` runs the unmodified reference project from ``baseline/_ref`` through its own
public API (``tinyinfer.LLM(Config(...))``, ``add_request``, ``step``) on a model folder of the same
shape written with random weights, at the same batch, context, steps and warm-up, and prints the
same line with ``"impl": "reference"``.
"""
from __future__ import annotations

import argparse
import gc
import json
import random
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# The two tiny configurations of the CPU baseline, with their workloads (prompt lengths, tokens to
# generate, greedy or temperature 1.0, page size, most prompt tokens of a request in a step).
TINY_WORKLOADS = {
    "tinyA": dict(
        config=dict(vocab_size=256, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=16, intermediate_size=128, rms_norm_eps=1e-6,
                    rope_theta=10000.0, tie_word_embeddings=True, max_position_embeddings=128),
        seed=0, prompts=[1, 7, 16, 33], max_tokens=8, greedy=True, page=4, chunk=8),
    "tinyB": dict(
        config=dict(vocab_size=384, hidden_size=96, num_hidden_layers=3, num_attention_heads=6,
                    num_key_value_heads=3, head_dim=32, intermediate_size=160, rms_norm_eps=1e-5,
                    rope_theta=1000000.0, tie_word_embeddings=False, max_position_embeddings=256),
        seed=1, prompts=[2, 11, 29, 64, 100], max_tokens=16, greedy=False, page=8, chunk=16),
}


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        data = json.loads(path.read_text())
        return {k: float(data.get(k, FALLBACK_PEAKS[k])) for k in FALLBACK_PEAKS}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed regions run."""
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
                 "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
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
                "reasons": sorted(reasons),
                "region": "from the headline's warm-up through the end-to-end run to the last device-timed decode run"}


def model_numbers(cfg, layers):
    """Bytes a decode step must read and flops of a prefill, from the configuration."""
    h, i, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    d, hq, hkv = cfg.resolved_head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    per_layer = h * (hq + 2 * hkv) * d + hq * d * h + 3 * h * i          # matrix elements
    norms = 2 * h + 2 * d
    weight_bytes = layers * (per_layer * 2 + norms * 4) + v * h * 2 + h * 4  # lm_head read once
    kv_bytes_per_token = layers * 2 * hkv * d * 2
    return dict(per_layer=per_layer, weight_bytes=weight_bytes, kv_bytes_per_token=kv_bytes_per_token)


def prefill_flops(cfg, layers, t, wanted_rows, prefix=0):
    h, v = cfg.hidden_size, cfg.vocab_size
    d, hq = cfg.resolved_head_dim, cfg.num_attention_heads
    per_layer = model_numbers(cfg, layers)["per_layer"]
    gemm = 2.0 * per_layer * t * layers
    attn = 4.0 * d * hq * (t * prefix + t * (t + 1) / 2.0) * layers      # causal q.k and p.v
    return gemm + attn + 2.0 * v * h * wanted_rows


def event_time(fn):
    import torch
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end)


def fast_forward(runner, rid, length):
    """Gives request ``rid`` pages for ``length`` tokens without computing them: the cache
    holds the random values it was filled with, which costs a decode step the same reads."""
    runner.admit(rid)
    runner.manager.extend(rid, length)
    runner.manager.commit(rid, length)


def release_engine(llm):
    """Lets go of an engine's weights, cache and captured graphs before the next one is built."""
    llm.close()


# ---------------------------------------------------------------------------------- the extras
def extra_qwen3_32b(peaks, steps=12, warmup=3):
    """Qwen3-32B layer sizes, all 64 layers, 32 requests whose contexts end at 8,192 tokens: does it
    fit (weights 65.5 GB + cache 68.7 GB, the pages sized from free memory, no override), and what
    a decode step and a 4,096-token prompt cost."""
    import torch
    from tinyinfer_b200 import EngineConfig, ops
    from tinyinfer_b200.config import preset_config
    from tinyinfer_b200.engine.batch import StepEntry
    from tinyinfer_b200.engine.llm import LLM
    cfg = preset_config("32b")
    layers, batch, ctx_len, page = cfg.num_hidden_layers, 32, 8192, 64
    torch.cuda.reset_peak_memory_stats()
    t0 = time.perf_counter()
    llm = LLM(cfg, EngineConfig(max_num_batched_tokens=4096, max_num_seqs=batch, max_model_len=ctx_len,
                                kvcache_block_size=page, dtype="bfloat16", max_live_requests=batch + 2),
              random_weights=4)
    torch.cuda.synchronize()
    build_s = time.perf_counter() - t0
    runner = llm.runner
    numbers = model_numbers(cfg, layers)
    rng = random.Random(4)
    for t in runner.storage.kv:
        if t is not None:
            t.normal_(0.0, 1.0)
    prompt = [rng.randrange(cfg.vocab_size) for _ in range(4096)]

    def prefill_once(tag):
        runner.step([StepEntry(tag, prompt, [len(prompt) - 1])])
        runner.release(tag)
    prefill_once("pw")
    prefill_ms = min(event_time(lambda i=i: prefill_once(f"p{i}")) for i in range(2))
    flops = prefill_flops(cfg, layers, len(prompt), 1)
    total = steps + warmup
    rids = [f"r{i}" for i in range(batch)]
    for rid in rids:
        fast_forward(runner, rid, ctx_len - total)
    feeds = [[rng.randrange(cfg.vocab_size) for _ in range(batch)] for _ in range(total)]

    def one(tokens):
        ops.argmax(runner.step([StepEntry(rid, [tok], [0]) for rid, tok in zip(rids, tokens)]))
    for k in range(warmup):
        one(feeds[k])
    ms = event_time(lambda: [one(feeds[warmup + k]) for k in range(steps)]) / steps
    runner.check_status()
    mean_ctx = ctx_len - total + warmup + (steps + 1) / 2.0
    step_bytes = numbers["weight_bytes"] + batch * mean_ctx * numbers["kv_bytes_per_token"]
    free, total_mem = torch.cuda.mem_get_info()
    out = {
        "layers": layers, "layers_full": layers, "hidden": cfg.hidden_size, "intermediate": cfg.intermediate_size,
        "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "batch": batch, "context": ctx_len,
        "decode_tok_s": batch / (ms / 1e3), "ms_per_step": ms, "steps": steps, "warmup": warmup,
        "step_gbytes": step_bytes / 1e9, "hbm_gbs": step_bytes / (ms / 1e3) / 1e9,
        "hbm_frac": step_bytes / (ms / 1e3) / 1e9 / peaks["hbm_gbs"],
        "prefill_4096_ms": prefill_ms, "prefill_tok_s": len(prompt) / (prefill_ms / 1e3),
        "prefill_frac": flops / (prefill_ms / 1e3) / (peaks["bf16_tflops_sustained"] * 1e12),
        "pages": llm.config.num_kvcache_blocks, "pages_from": "free memory (pages_that_fit), no override",
        "page_size": page, "weights_gb": llm.model.weight_bytes() / 1e9,
        "cache_gb": sum(t.numel() * t.element_size() for t in runner.storage.kv if t is not None) / 1e9,
        "peak_allocated_gb": torch.cuda.max_memory_allocated() / 1e9, "device_total_gb": total_mem / 1e9,
        "device_free_gb_while_loaded": free / 1e9, "build_s": build_s,
    }
    for rid in rids:
        runner.release(rid)
    release_engine(llm)
    return out


def extra_qwen3_1p7b_mix(peaks, num_requests=64):
    """Qwen3-1.7B layer sizes through the scheduler: 64 requests, prompts of 16 to 1,024 tokens in
    portions of at most 512 beside the decoded tokens of others, 16 to 512 generated tokens each, half
    greedy and half at temperature 0.7. Run once to warm up (graphs are captured as batch sizes come
    up), then once more with other tokens, timed by the wall clock. ``roofline_frac``: for every step, the
    larger of (bytes it must read / HBM rate) and (its flops / tensor rate), summed, over the time taken."""
    import torch
    from tinyinfer_b200 import EngineConfig, SamplingParams
    from tinyinfer_b200.config import preset_config
    from tinyinfer_b200.engine.llm import LLM
    cfg = preset_config("1.7b")
    layers = cfg.num_hidden_layers
    llm = LLM(cfg, EngineConfig(max_num_batched_tokens=4096, max_num_seqs=64, max_model_len=2048,
                                kvcache_block_size=64, prefill_chunk=512, dtype="bfloat16"), random_weights=3)
    numbers = model_numbers(cfg, layers)
    d, hq = cfg.resolved_head_dim, cfg.num_attention_heads
    step_log = []
    plain_step = llm.step

    def logged_step():
        items = plain_step()
        step_log.append([(it.start_pos, it.num_tokens, it.sample_after) for it in items])
        return items
    llm.step = logged_step

    def workload(seed):
        rng = random.Random(seed)
        prompts = [[rng.randrange(cfg.vocab_size) for _ in range(rng.randint(16, 1024))] for _ in range(num_requests)]
        params = [SamplingParams(greedy=i % 2 == 0, temperature=0.7, topk=100, max_tokens=rng.randint(16, 512),
                                 ignore_eos=True, seed=i) for i in range(num_requests)]
        return prompts, params
    llm.generate_token_ids(*workload(100))
    step_log.clear()
    prompts, params = workload(3)
    replays0, steps0 = llm.runner.graph_replays, llm.runner.steps_run
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = llm.generate_token_ids(prompts, params)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    llm.runner.check_status()
    out_tokens = sum(len(o["token_ids"]) for o in outs)
    computed = sum(n for step in step_log for _s, n, _w in step)
    floor_s, mixed_steps, decode_steps = 0.0, 0, 0
    for step in step_log:
        tokens = sum(n for _s, n, _w in step)
        rows = sum(1 for _s, _n, w in step if w)
        keys = sum(s + n for s, n, _w in step)
        byts = numbers["weight_bytes"] - (0 if rows else cfg.vocab_size * cfg.hidden_size * 2) \
            + keys * numbers["kv_bytes_per_token"]
        flops = 2.0 * numbers["per_layer"] * layers * tokens + 2.0 * cfg.vocab_size * cfg.hidden_size * rows \
            + sum(4.0 * d * hq * layers * (n * s + n * (n + 1) / 2.0) for s, n, _w in step)
        floor_s += max(byts / (peaks["hbm_gbs"] * 1e9), flops / (peaks["bf16_tflops_sustained"] * 1e12))
        if any(n > 1 for _s, n, _w in step):
            mixed_steps += 1
        else:
            decode_steps += 1
    ttft = [o["statistics"]["ttft"] for o in outs if o["statistics"]["ttft"] is not None]
    tpot = [o["statistics"]["tpot"] for o in outs if o["statistics"]["tpot"] is not None]
    out = {
        "layers": layers, "layers_full": layers, "hidden": cfg.hidden_size, "intermediate": cfg.intermediate_size,
        "requests": num_requests, "prefill_chunk": 512, "max_num_seqs": 64, "max_num_batched_tokens": 4096,
        "wall_s": wall, "output_tokens": out_tokens, "computed_tokens": computed,
        "output_tok_s": out_tokens / wall, "computed_tok_s": computed / wall,
        "requests_per_s": num_requests / wall,
        "steps": llm.runner.steps_run - steps0, "steps_with_prompt_portions": mixed_steps,
        "decode_only_steps": decode_steps, "graph_replays": llm.runner.graph_replays - replays0,
        "preemptions": llm.scheduler.num_preemptions,
        "mean_ttft_ms": 1e3 * sum(ttft) / max(1, len(ttft)), "mean_tpot_ms": 1e3 * sum(tpot) / max(1, len(tpot)),
        "roofline_floor_s": floor_s, "roofline_frac": floor_s / wall, "timing": "wall clock, second run",
    }
    release_engine(llm)
    return out


def extra_cpu_baseline():
    """The two tiny configurations with their workloads: seconds on the CPU through the plain
    implementation of the tests (float32, whole sequence recomputed for every token: it has no
    cache), and seconds through this engine on the GPU in float32 for the same requests."""
    import torch
    sys.path.insert(0, str(ROOT / "tests"))
    import plain_qwen3 as plain
    from tinyinfer_b200 import LLM, SamplingParams
    from tinyinfer_b200.config import lookup_architecture
    from tinyinfer_b200.weights import write_random_model
    arch = lookup_architecture("Qwen3ForCausalLM")
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        for name, wl in TINY_WORKLOADS.items():
            cfg = arch.config_class.from_dict(dict(wl["config"], architectures=[arch.name]))
            folder = write_random_model(Path(tmp) / name, cfg, seed=wl["seed"], dtype="float32")
            rng = random.Random(wl["seed"])
            prompts = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in wl["prompts"]]
            pcfg, weights = plain.read_model_folder(folder, torch.float32)
            t0 = time.perf_counter()
            generated = 0
            for r, prompt in enumerate(prompts):
                tokens = list(prompt)
                for k in range(wl["max_tokens"]):
                    row = plain.forward(pcfg, weights, tokens)[-1].numpy()
                    tokens.append(plain.sample(row, greedy=wl["greedy"], temperature=1.0, topk=100, seed=0,
                                               stream=r, step=k))
                    generated += 1
            cpu_s = time.perf_counter() - t0
            llm = LLM(folder, dtype="float32", max_num_seqs=len(prompts), max_num_batched_tokens=256,
                      kvcache_block_size=wl["page"], prefill_chunk=wl["chunk"], num_kvcache_blocks=256,
                      max_model_len=cfg.max_position_embeddings)
            params = SamplingParams(greedy=wl["greedy"], temperature=1.0, topk=100, max_tokens=wl["max_tokens"],
                                    ignore_eos=True, seed=0)
            llm.generate_token_ids(prompts, params)                 # builds and warms the kernels
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            llm.generate_token_ids(prompts, params)
            torch.cuda.synchronize()
            engine_s = time.perf_counter() - t0
            out[name] = {"cpu_plain_s": cpu_s, "cpu_tok_s": generated / cpu_s, "engine_fp32_s": engine_s,
                         "generated_tokens": generated}
            release_engine(llm)
    return out


# ---------------------------------------------------------------------------------- the reference arm
def reference_arm(args) -> int:
    """The unmodified reference (installed into baseline/_ref) through its own public API."""
    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
        return 0
    import faulthandler
    faulthandler.enable()                       # a crash inside the reference's extension names the Python line

    def say(what):
        print(f"[reference arm] {what}", file=sys.stderr, flush=True)
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "tinyinfer").is_dir():
        return unavailable("baseline/_ref holds no install of the reference")
    if args.gpus != 1:
        print(f"bench.py measures one GPU (got --gpus {args.gpus})")
        return 2
    import torch
    if not torch.cuda.is_available():
        return unavailable("no CUDA device is visible")
    sys.path.insert(0, str(ref))
    try:
        import tinyinfer
        from tinyinfer.config import Config as RefConfig
    except Exception as e:                      # a missing dependency or an extension built for other libraries
        return unavailable(f"the installed reference does not import: {type(e).__name__}: {e}")
    from tinyinfer_b200.config import preset_config
    from tinyinfer_b200.weights import write_random_model

    args.warmup = max(args.warmup, 3)
    peaks, peak_source = load_peaks()
    layers_full = preset_config(args.model_size).num_hidden_layers
    layers = args.layers or layers_full
    cfg = preset_config(args.model_size, num_hidden_layers=layers)
    numbers = model_numbers(cfg, layers)
    vocab, ctx_len, batch = cfg.vocab_size, args.context, args.batch
    rng = random.Random(0)
    with tempfile.TemporaryDirectory() as tmp:
        folder = Path(tmp) / "model"
        t0 = time.perf_counter()
        write_random_model(folder, cfg, seed=2, dtype="bfloat16", device="cuda:0")
        torch.cuda.empty_cache()
        meta = json.loads((folder / "config.json").read_text())
        meta.setdefault("model_type", "qwen3")
        (folder / "config.json").write_text(json.dumps(meta))
        # a tokenizer the reference's constructor can load: one word per token id
        from tokenizers import Tokenizer
        from tokenizers.models import WordLevel
        from tokenizers.pre_tokenizers import Whitespace
        tok = Tokenizer(WordLevel(vocab={str(i): i for i in range(vocab)}, unk_token="0"))
        tok.pre_tokenizer = Whitespace()
        tok.save(str(folder / "tokenizer.json"))
        (folder / "tokenizer_config.json").write_text(json.dumps({"tokenizer_class": "PreTrainedTokenizerFast"}))
        write_s = time.perf_counter() - t0
        say(f"model folder written in {write_s:.1f} s")
        # The reference's feed-forward binding warns when a step has more than 32 tokens, and on this image
        # that warning crashes the process (SIGSEGV inside mlp_forward at 33 tokens, none at 32): its
        # token budget is therefore 32, prompts go through in portions of 32, and batches above 32 are left out.
        if batch > args.ref_step_tokens:
            return unavailable(f"a decode step of {batch} tokens is beyond the {args.ref_step_tokens} tokens a step that "
                               "the reference's feed-forward binding survives on this image")
        batches = [batch] if args.skip_points else sorted({1, batch, 64})
        t0 = time.perf_counter()
        engine = tinyinfer.LLM(RefConfig(
            model=str(folder), max_num_batched_tokens=args.ref_step_tokens, max_num_seqs=max(batches), max_model_len=ctx_len,
            kvcache_block_size=args.ref_block_size, gpu_memory_utilization=0.90, attention_backend="flash"))
        torch.cuda.synchronize()
        build_s = time.perf_counter() - t0
        say(f"engine built in {build_s:.1f} s, {engine.config.num_kvcache_blocks} cache blocks")

        greedy_one = tinyinfer.SamplingParams(greedy=True, max_tokens=1, ignore_eos=True)
        engine.generate_token_ids([[rng.randrange(vocab) for _ in range(64)]], greedy_one)       # first launches
        pf = []
        for _ in range(2):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            engine.generate_token_ids([[rng.randrange(vocab) for _ in range(2048)]], greedy_one)
            torch.cuda.synchronize()
            pf.append((time.perf_counter() - t0) * 1e3)
        prefill_ms = min(pf)
        say(f"prefill of 2,048 tokens: {prefill_ms:.0f} ms")
        pf_flops = prefill_flops(cfg, layers, 2048, 1)
        prefill = {"value": 2048 / (prefill_ms / 1e3), "tokens": 2048, "ms": prefill_ms,
                   "frac": pf_flops / (prefill_ms / 1e3) / (peaks["bf16_tflops_sustained"] * 1e12),
                   "tflops": pf_flops / (prefill_ms / 1e3) / 1e12, "peak_tflops": peaks["bf16_tflops_sustained"],
                   "timing": "wall clock around generate_token_ids of one prompt with max_tokens=1"}

        def decode_run(b, steps, warmup, sampler=None):
            total = steps + warmup
            slack = 2 * b + 8
            prompt_len = ctx_len - total - slack - 1
            params = tinyinfer.SamplingParams(greedy=True, max_tokens=total + slack, ignore_eos=True)
            for _ in range(b):
                engine.add_request([rng.randrange(vocab) for _ in range(prompt_len)], params)
            while engine.scheduler.waiting:                 # prompts, in portions, until all decode
                engine.step()
            say(f"batch {b}: prompts of {prompt_len} tokens are in the cache")
            if sampler is not None:
                sampler.start()
            for _ in range(warmup - 1):
                engine.step()
            t0 = time.perf_counter()
            dev_ms = event_time(lambda: [engine.step() for _ in range(steps)])
            wall_ms = (time.perf_counter() - t0) * 1e3
            while not engine.scheduler.is_finished():
                engine.step()
            ms = max(dev_ms, wall_ms)
            mean_ctx = prompt_len + warmup + (steps + 1) / 2.0
            return dict(ms_per_step=ms / steps, tok_s=b * steps / (ms / 1e3),
                        bytes=numbers["weight_bytes"] + b * mean_ctx * numbers["kv_bytes_per_token"])

        sampler = ClockSampler()
        head = decode_run(batch, args.steps, args.warmup, sampler)
        points, skipped = {f"decode_b{batch}": head["tok_s"]}, {}
        for b in batches:
            if b == batch:
                continue
            prefill_s = b * ctx_len / prefill["value"]
            if b > args.ref_step_tokens:
                skipped[f"decode_b{b}"] = (f"more than {args.ref_step_tokens} tokens in a step crash the reference's "
                                           "feed-forward binding on this image (SIGSEGV on its warning path)")
                continue
            if prefill_s > args.ref_point_limit:
                skipped[f"decode_b{b}"] = f"its prompts alone would take about {prefill_s:.0f} s to prefill"
                continue
            points[f"decode_b{b}"] = decode_run(b, max(8, args.steps // 2), args.warmup)["tok_s"]
        clocks = sampler.stop()
    achieved = head["bytes"] / (head["ms_per_step"] / 1e3) / 1e9
    max_blocks = (ctx_len + args.ref_block_size - 1) // args.ref_block_size
    out = {
        "impl": "reference",
        "metric": f"decode tok/s at batch {batch} (Qwen3-{args.model_size.upper()} shape, random weights)",
        "value": head["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic token ids, random-init weights",
        "config": {"model": f"qwen3-{args.model_size}-shape", "layers": layers, "layers_full": layers_full,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.resolved_head_dim, "intermediate": cfg.intermediate_size, "vocab": vocab,
                   "global_batch": batch, "seq_len": ctx_len, "prefill_tokens": 2048,
                   "page_size": args.ref_block_size, "parallelism": "single-gpu", "attention_backend": "flash",
                   "max_num_batched_tokens": args.ref_step_tokens,
                   "l2": f"inputs>L2 (weights {numbers['weight_bytes'] / 1e9:.1f} GB read per step)",
                   "cache_fill": "real prefill through the reference's scheduler",
                   "timing": "larger of CUDA events and wall clock around K calls of LLM.step()"},
        "clocks": clocks,
        "e2e": {"value": head["tok_s"], "unit": "tokens/s", "ms_per_step": head["ms_per_step"],
                # the tensors its prepare_batch and sampler build for a decode step, and its one .tolist()
                "h2d_bytes_per_step": batch * (3 * 8 + 4 * max_blocks + 2 + 8 + 1),
                "d2h_bytes_per_step": batch * 16},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "peaks": peak_source},
        "points": points, "points_skipped": skipped, "model_write_s": write_s, "engine_build_s": build_s,
    }
    print(json.dumps(out))
    return 0


# ---------------------------------------------------------------------------------- this engine
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
    ap.add_argument("--skip-extras", action="store_true", help="leave out the 'configs' of the line")
    ap.add_argument("--extras", default="32b,mix,cpu", help="which of the other configurations to run")
    ap.add_argument("--ref-block-size", type=int, default=256, help="reference arm: its kvcache_block_size (its default)")
    ap.add_argument("--ref-step-tokens", type=int, default=32,
                    help="reference arm: its max_num_batched_tokens (more than 32 tokens in a step crash its binding here)")
    ap.add_argument("--ref-point-limit", type=float, default=240.0,
                    help="reference arm: skip a batch size whose prompts would take longer than this many seconds")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine is single-GPU by design (got --gpus {args.gpus})")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from tinyinfer_b200 import EngineConfig, SamplingParams
    from tinyinfer_b200.config import preset_config
    from tinyinfer_b200.engine.batch import StepEntry
    from tinyinfer_b200.engine.llm import LLM
    from tinyinfer_b200 import ops

    peaks, peak_source = load_peaks()
    layers_full = preset_config(args.model_size).num_hidden_layers
    layers = args.layers or layers_full
    cfg = preset_config(args.model_size, num_hidden_layers=layers)
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
    def decode_run(batch, steps, warmup, sampler=None):
        total = steps + warmup
        start_len = ctx_len - total
        rids = [f"d{batch}_{i}" for i in range(batch)]
        for rid in rids:
            fast_forward(runner, rid, start_len)
        feeds = [[rng.randrange(vocab) for _ in range(batch)] for _ in range(total)]

        def one(step_tokens):
            logits = runner.step([StepEntry(rid, [tok], [0]) for rid, tok in zip(rids, step_tokens)])
            ops.argmax(logits)
        if sampler is not None:
            sampler.start()
        for k in range(warmup):
            one(feeds[k])
        launches0 = ops.launch_count()
        ms = event_time(lambda: [one(feeds[warmup + k]) for k in range(steps)])
        launches = ops.launch_count() - launches0
        mean_ctx = start_len + warmup + (steps + 1) / 2.0
        for rid in rids:
            runner.release(rid)
        return dict(ms_per_step=ms / steps, tok_s=batch * steps / (ms / 1e3), launches=launches,
                    bytes=numbers["weight_bytes"] + batch * mean_ctx * numbers["kv_bytes_per_token"])

    sampler = ClockSampler()
    head = decode_run(args.batch, args.steps, args.warmup, sampler)
    runner.check_status()
    achieved = head["bytes"] / (head["ms_per_step"] / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "peaks": peak_source}

    # ------------------------------------------------------------------ end to end through LLM.step()
    # (right behind the device-timed run of the same batch, before the other batch sizes: the same state of the device)
    # The prompts' prefill is a compute-bound burst under the power cap; the clocks it leaves behind recover
    # over some twenty decode steps (measured: 4.39 ms a step falling to 4.08). Those steps are warm-up here,
    # as the device-timed run above starts from an idle device.
    e2e_warmup = args.warmup + 20
    total = args.steps + e2e_warmup
    slack = 2 * args.batch + 8                         # tokens decoded while other prompts still prefill
    prompt_len = ctx_len - total - slack - 1
    params = SamplingParams(greedy=True, max_tokens=total + slack, ignore_eos=True)
    for _ in range(args.batch):
        llm.add_request([rng.randrange(vocab) for _ in range(prompt_len)], params)
    while llm.scheduler.waiting:                      # prompts, in portions, until all decode
        llm.step()
    for _ in range(e2e_warmup - 1):
        llm.step()
    h2d0 = runner.buffers.bytes_copied
    torch.cuda.synchronize()                          # the step in flight is not part of the K steps timed below
    t0 = time.perf_counter()
    e2e_ms = event_time(lambda: [llm.step() for _ in range(args.steps)])
    wall_ms = (time.perf_counter() - t0) * 1e3
    h2d = (runner.buffers.bytes_copied - h2d0) / args.steps
    e2e = {"value": args.batch * args.steps / (max(e2e_ms, wall_ms) / 1e3), "unit": "tokens/s",
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": (args.batch + 2) * 4,     # tokens and two status words
           "ms_per_step": max(e2e_ms, wall_ms) / args.steps, "warmup": e2e_warmup,
           "overlap": "a step is launched before the tokens of the one before are read back; every step's tokens "
                      "reach the host, one call later"}
    while not llm.is_finished():                      # the end-to-end requests run out, their pages go back
        llm.step()

    points = {}
    for b in batches:
        if b == args.batch:
            points[f"decode_b{b}"] = head["tok_s"]
        else:
            points[f"decode_b{b}"] = decode_run(b, max(8, args.steps // 2), args.warmup)["tok_s"]
    clocks = sampler.stop()
    runner.check_status()

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
        "clocks": clocks, "e2e": e2e, "gpu_launches": head["launches"],
        "prefill": prefill, "roofline": roofline, "points": points,
    }

    if not args.skip_extras:
        release_engine(llm)
        del llm, runner
        configs = {}
        wanted = {w.strip() for w in args.extras.split(",") if w.strip()}
        for key, name, fn in (("32b", "qwen3_32b", lambda: extra_qwen3_32b(peaks)),
                              ("mix", "qwen3_1p7b_mix", lambda: extra_qwen3_1p7b_mix(peaks)),
                              ("cpu", "cpu_baseline_s", extra_cpu_baseline)):
            if key not in wanted:
                continue
            t0 = time.perf_counter()
            try:
                configs[name] = fn()
            except Exception as e:               # an extra that fails says so; the headline stands
                configs[name] = {"failed": f"{type(e).__name__}: {e}"[:300]}
                gc.collect()
                torch.cuda.empty_cache()
            configs[name]["bench_wall_s"] = time.perf_counter() - t0
        out["configs"] = configs
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
