"""Trace replay: feeds given token ids through the model step by step and hands back logits.
It samples nothing and owns no forward pass, cache or loader: it drives ``ModelRunner.step``,
the same function generation uses. ``bin/trace_run`` is its command line.

A trace is a sequence of steps ``{"step": k, "entries": [{"id", "tokens", "want"}], "end": [ids]}``.
All entries of a step run as one batch; ``end`` names requests whose pages are given back after
the step. The reference has no such tool; its nearest relative feeds fixed chunks for perplexity
(tinyinfer/quantization/PPL.py:40-113).
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .batch import StepEntry
from .loading import load_model, require_cuda
from .runner import ModelRunner

TOKEN_GRAIN = 64        # a request's token count is rounded up to this when the pool is sized


def pool_pages(max_tokens: int, page_size: int) -> int:
    """Pages that hold ``max_tokens`` tokens when every live request's count is rounded up to a
    multiple of max(64, page_size)."""
    grain = max(TOKEN_GRAIN, page_size)
    rounded = (max_tokens + grain - 1) // grain * grain
    return max(1, (rounded + page_size - 1) // page_size)


class TraceSession:
    def __init__(self, model_dir, dtype: str, max_tokens: int, *, page_size: int = 16,
                 device="cuda:0", max_live: int = 8, poison_cache: bool = False, model=None,
                 cuda_graphs: bool = True):
        if model is None:
            require_cuda(device)
            model, _ = load_model(model_dir, dtype, device)
        self.model = model
        limit = model.spec.max_positions
        self.runner = ModelRunner(
            model, page_size=page_size, num_pages=pool_pages(max_tokens, page_size),
            max_requests=max_live, max_tokens_per_step=max(max_tokens, 1), max_model_len=limit,
            poison_cache=poison_cache, cuda_graphs=cuda_graphs)

    def run_step(self, step: dict) -> Optional[np.ndarray]:
        """Runs one step; returns float32 logits [wanted, vocab] or None if nothing is wanted."""
        entries = [StepEntry(e["id"], list(e["tokens"]), list(e.get("want", ())))
                   for e in step.get("entries", [])]
        logits = self.runner.step(entries)
        self.runner.check_status()              # a step whose kernels gave up must not hand out logits
        for rid in step.get("end", []):
            if rid in self.runner.manager:
                self.runner.release(rid)
        if logits.shape[0] == 0:
            return None
        return logits.detach().to("cpu", torch.float32).numpy()
