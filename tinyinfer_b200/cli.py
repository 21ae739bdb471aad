"""Command line of the engine, in the manner of the reference's example scripts: the same option
names and meanings where it has them (--model, --max-num-batched-tokens, --max-num-seqs,
--max-model-len, --block-size / --kvcache-block-size, --gpu-memory-utilization:
examples/advance07_sd.py:19-32, benchmarks/benchmark_throughput.py:12-20; --max-tokens,
--temperature, --greedy: examples/advance01_ui.py:11-21). Options the reference has for parts
that are not built here (--attention-backend, --quantization, --speculative, --host, --port) are
refused with a clear message rather than ignored.
"""
from __future__ import annotations

import argparse
import json
import random
import sys
from typing import List, Optional

from . import models  # noqa: F401  (registers the built-in architecture and its presets)
from .config import EngineConfig, known_presets, parse_dtype, preset_config  # noqa: F401


def add_engine_options(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--model", help="folder with config.json and *.safetensors")
    ap.add_argument("--random-config", choices=sorted(known_presets()),
                    help="instead of --model: a size that a registered architecture offers, with random weights")
    ap.add_argument("--seed", type=int, default=0, help="seed of the random weights")
    ap.add_argument("--dtype", default="bfloat16", help="bfloat16 (bf16) or float32 (fp32)")
    ap.add_argument("--max-num-batched-tokens", type=int, default=4096)
    ap.add_argument("--max-num-seqs", type=int, default=64)
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--block-size", "--kvcache-block-size", dest="block_size", type=int, default=64)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.90)
    ap.add_argument("--num-kvcache-blocks", type=int, default=0, help="0: sized from free memory")
    ap.add_argument("--prefill-chunk", type=int, default=0, help="most prompt tokens of a request per step")
    ap.add_argument("--no-prefix-caching", action="store_true",
                    help="compute every prompt from its first token, even if an earlier one began alike")
    ap.add_argument("--device", default="cuda:0")
    for flag in ("--attention-backend", "--quantization", "--speculative", "--draft-model",
                 "--max-draft-tokens", "--host", "--port"):
        ap.add_argument(flag, nargs="?", const=True, default=None, help=argparse.SUPPRESS)


def engine_config_from(args) -> EngineConfig:
    for name in ("attention_backend", "quantization", "speculative", "draft_model", "max_draft_tokens",
                 "host", "port"):
        if getattr(args, name, None) is not None:
            raise SystemExit(f"--{name.replace('_', '-')} belongs to a part of the reference that this "
                             "engine does not build (one attention path, no quantization, no "
                             "speculative decoding, no server)")
    return EngineConfig(
        max_num_batched_tokens=args.max_num_batched_tokens, max_num_seqs=args.max_num_seqs,
        max_model_len=args.max_model_len, gpu_memory_utilization=args.gpu_memory_utilization,
        kvcache_block_size=args.block_size, num_kvcache_blocks=args.num_kvcache_blocks,
        prefill_chunk=args.prefill_chunk, dtype=parse_dtype(args.dtype), device=args.device,
        enable_prefix_caching=False if args.no_prefix_caching else None)


def build_llm(args):
    from .engine.llm import LLM
    cfg = engine_config_from(args)
    if args.model:
        return LLM(args.model, cfg)
    if args.random_config:
        return LLM(preset_config(args.random_config), cfg, random_weights=args.seed)
    raise SystemExit("give --model DIR or --random-config NAME")


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="tinyinfer_b200", description="Generate with a model of a registered architecture on one B200.")
    add_engine_options(ap)
    ap.add_argument("--prompt", action="append", default=[], help="text prompt (needs a tokenizer in --model)")
    ap.add_argument("--prompt-ids", action="append", default=[], help="prompt as comma-separated token ids")
    ap.add_argument("--prompt-len", type=int, action="append", default=[],
                    help="a random prompt of this many tokens (uniform ids)")
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--topk", type=int, default=100)
    ap.add_argument("--greedy", action="store_true")
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--sampling-seed", type=int, default=None)
    args = ap.parse_args(argv)

    from .sampling import SamplingParams
    llm = build_llm(args)
    vocab = llm.model.spec.vocab_size
    rng = random.Random(args.seed)
    prompts: list = list(args.prompt)
    prompts += [[int(x) for x in s.split(",") if x.strip()] for s in args.prompt_ids]
    prompts += [[rng.randrange(vocab) for _ in range(n)] for n in args.prompt_len]
    if not prompts:
        raise SystemExit("no prompt: use --prompt, --prompt-ids or --prompt-len")
    params = SamplingParams(temperature=args.temperature, topk=args.topk, max_tokens=args.max_tokens,
                            ignore_eos=args.ignore_eos, greedy=args.greedy, seed=args.sampling_seed)
    for i, out in enumerate(llm.generate(prompts, params)):
        stats = out["statistics"]
        print(json.dumps({"request": i, "token_ids": out["token_ids"], "text": out.get("text"),
                          "finish_reason": out["finish_reason"], "ttft": stats["ttft"],
                          "tpot": stats["tpot"], "decode_throughput": stats["decode_throughput"]}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
