"""Turns rows of logits into tokens, every row with its own options
(tinyinfer/layers/sampler.py:13-75 of the reference: greedy rows take the argmax, the others
temperature, top-k threshold and Gumbel-max). One kernel launch for the whole batch."""
from __future__ import annotations

from typing import List, Sequence

import torch

from .. import ops
from .params import SamplingParams


class Sampler:
    def __init__(self, device, engine_seed: int = 0):
        self.device = torch.device(device)
        self.engine_seed = int(engine_seed)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               stream_ids: Sequence[int], steps: Sequence[int], with_nll: bool = False):
        """``logits`` float32 [N, V]; row i is drawn with ``params[i]`` from the random stream
        (seed, ``stream_ids[i]``, ``steps[i]``): the request's number and how many tokens it has
        generated. Returns python ints (one device-to-host copy); with ``with_nll`` a pair
        (tokens, negative log-likelihood of each token under its row's softmax)."""
        tokens = self._sample_device(logits, params, stream_ids, steps)
        if tokens is None:
            return ([], []) if with_nll else []
        if not with_nll:
            return tokens.tolist()
        # tinyinfer/engine/model_runner.py:446-454 of the reference: tokens and NLL leave together
        pair = torch.stack((tokens.to(torch.float64), ops.token_nll(logits, tokens).to(torch.float64))).tolist()
        return [int(t) for t in pair[0]], pair[1]

    def _sample_device(self, logits, params, stream_ids, steps):
        n = logits.shape[0]
        if n == 0:
            return None
        vocab = logits.shape[1]
        if all(p.greedy for p in params):
            return ops.argmax(logits)
        # the reference refuses top-k above the vocabulary (sampler.py:56-57); here it is 'off'
        host = torch.tensor(
            [[float(p.temperature) for p in params]], dtype=torch.float32)
        ints = torch.tensor([
            [0 if p.topk >= vocab else p.topk for p in params],
            [1 if p.greedy else 0 for p in params],
            [int(s) & 0x7FFFFFFF for s in stream_ids],
            [int(s) & 0x7FFFFFFF for s in steps]], dtype=torch.int32)
        seeds = torch.tensor([self.engine_seed if p.seed is None else int(p.seed) for p in params],
                             dtype=torch.int64)
        temp = host.to(self.device)[0].contiguous()
        ints = ints.to(self.device)
        return ops.sample(logits, temp, ints[0].contiguous(), ints[1].contiguous(),
                          seeds.to(self.device), ints[2].contiguous(), ints[3].contiguous())
