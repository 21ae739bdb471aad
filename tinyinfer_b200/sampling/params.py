"""Per-request sampling options, with the reference's names, defaults and checks
(tinyinfer/sampling_params.py:5-18). ``seed`` is new: the reference draws from the global CUDA
generator (tinyinfer/layers/sampler.py:70); here every request has a counter-based stream."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class SamplingParams:
    temperature: float = 1.0
    topk: int = 100                 # values below the k-th largest are masked; 0 switches it off
    max_tokens: int = 64            # most tokens to generate
    ignore_eos: bool = False
    greedy: bool = False
    seed: Optional[int] = None      # None: the engine's seed

    def __post_init__(self):
        if self.temperature <= 0.0:
            raise ValueError("temperature must be positive")
        if self.topk < 0:
            raise ValueError("topk must not be negative (0 switches it off)")
        if self.max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
