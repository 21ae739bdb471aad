"""Knobs of the engine, with the reference's names and defaults where it has them
(tinyinfer/config.py:7-30, checks :55-67)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class EngineConfig:
    max_num_batched_tokens: int = 4096      # token budget of one step
    max_num_seqs: int = 64                  # requests in one step
    max_live_requests: int = 0              # requests that hold cache at a time; 0: 4 x max_num_seqs
    max_model_len: int = 4096               # prompt + completion of one request
    gpu_memory_utilization: float = 0.90    # share of device memory the engine may take
    kvcache_block_size: int = 64            # tokens in a page (the reference's default is 256)
    num_kvcache_blocks: int = 0             # pages per cache group; 0: sized from free memory
    prefill_chunk: int = 0                  # most prompt tokens of one request in a step; 0: budget only
    dtype: str = "bfloat16"                 # "bfloat16" or "float32"
    seed: int = 0                           # base of the sampling streams
    eos_token_id: int = -1                  # -1: taken from the model's configuration, if any
    cuda_graphs: bool = True                # replay captured decode steps
    overlap_steps: bool = True              # launch a step before the tokens of the one before are read back
    track_nll: bool = False                 # sum each request's token NLL (the perplexity statistic)
    enable_prefix_caching: Optional[bool] = None   # keep full pages for later prompts with the same
                                                   # start; None: on where the model allows it
    device: str = "cuda:0"

    def validate(self) -> None:
        if self.max_num_seqs <= 0:
            raise ValueError("max_num_seqs must be positive")
        if self.max_num_batched_tokens <= 0:
            raise ValueError("max_num_batched_tokens must be positive")
        if self.max_model_len <= 0:
            raise ValueError("max_model_len must be positive")
        if not 0 < self.gpu_memory_utilization <= 1:
            raise ValueError("gpu_memory_utilization must be in (0, 1]")
        if self.kvcache_block_size <= 0:
            raise ValueError("kvcache_block_size must be positive")
        if self.num_kvcache_blocks < 0:
            raise ValueError("num_kvcache_blocks must not be negative")
        if self.max_live_requests < 0:
            raise ValueError("max_live_requests must not be negative")
        if self.prefill_chunk < 0:
            raise ValueError("prefill_chunk must not be negative")
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {self.dtype!r}")


    @property
    def live_requests(self) -> int:
        return self.max_live_requests if self.max_live_requests > 0 else 4 * self.max_num_seqs


def parse_dtype(name: Optional[str]) -> str:
    """Accepts the spellings of the command lines ('bf16', 'fp32', ...)."""
    table = {"bf16": "bfloat16", "bfloat16": "bfloat16", "fp32": "float32", "float32": "float32",
             "float": "float32"}
    key = (name or "bfloat16").lower()
    if key not in table:
        raise ValueError(f"unknown dtype {name!r}; use bfloat16 or float32")
    return table[key]
