"""Turns rows of logits into tokens, every row with its own options
(tinyinfer/layers/sampler.py:13-75 of the reference: greedy rows take the argmax, the others
temperature, top-k threshold and Gumbel-max). One kernel launch for the whole batch."""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from .params import SamplingParams


class Sampler:
    def __init__(self, device, engine_seed: int = 0):
        self.device = torch.device(device)
        self.engine_seed = int(engine_seed)
        self._staging = None               # pinned host words the per-row parameters are staged in
        self._staging_np = None

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               stream_ids: Sequence[int], steps: Sequence[int], with_nll: bool = False,
               status: Optional[torch.Tensor] = None):
        """``logits`` float32 [N, V]; row i is drawn with ``params[i]`` from the random stream
        (seed, ``stream_ids[i]``, ``steps[i]``): the request's number and how many tokens it has
        generated. Returns python ints (one device-to-host copy); with ``with_nll`` a pair
        (tokens, negative log-likelihood of each token under its row's softmax).
        ``status``: the device's status words (``ops.status_words``); they come home in the same copy
        as the tokens, and KernelError is raised instead of tokens if a kernel of the step set one."""
        n = logits.shape[0]
        tokens = self._sample_device(logits, params, stream_ids, steps, status)
        if tokens is None:
            return ([], []) if with_nll else []
        if not with_nll:
            host = tokens.tolist()
            nlls = None
        else:
            # tinyinfer/engine/model_runner.py:446-454 of the reference: tokens and NLL leave together
            both = torch.cat((tokens.to(torch.float64), ops.token_nll(logits, tokens[:n]).to(torch.float64))).tolist()
            host, nlls = [int(t) for t in both[:tokens.shape[0]]], both[tokens.shape[0]:]
        if len(host) > n:
            ops.raise_on_status(self.device, *host[n:n + 2])
        return (host[:n], nlls) if with_nll else host[:n]

    def _sample_device(self, logits, params, stream_ids, steps, status=None):
        n = logits.shape[0]
        if n == 0:
            return None
        vocab = logits.shape[1]
        if all(p.greedy for p in params):
            return ops.argmax(logits, extra=status)
        # the reference refuses top-k above the vocabulary (sampler.py:56-57); here it is 'off'.
        # All per-row parameters travel in ONE staged array: [seed low/high words | temperature bits |
        # top-k | greedy | stream | step], each a run of `width` 32-bit words.
        width = (n + 3) // 4 * 4                                   # runs start on 16-byte boundaries
        words = 7 * width
        if self._staging is None or self._staging.numel() < words:
            self._staging = torch.empty(max(words, 7 * 64), dtype=torch.int32,
                                        pin_memory=self.device.type == "cuda")
            self._staging_np = self._staging.numpy()
        host = self._staging_np
        seeds = np.asarray([self.engine_seed if p.seed is None else int(p.seed) for p in params], dtype=np.int64)
        host[:2 * n] = seeds.view(np.int32)
        host[2 * width:2 * width + n] = np.asarray([float(p.temperature) for p in params], dtype=np.float32).view(np.int32)
        host[3 * width:3 * width + n] = [0 if p.topk >= vocab else p.topk for p in params]
        host[4 * width:4 * width + n] = [1 if p.greedy else 0 for p in params]
        host[5 * width:5 * width + n] = [int(x) & 0x7FFFFFFF for x in stream_ids]
        host[6 * width:6 * width + n] = [int(x) & 0x7FFFFFFF for x in steps]
        dev = self._staging[:words].to(self.device, non_blocking=True)
        return ops.sample(logits, dev[2 * width:2 * width + n].view(torch.float32), dev[3 * width:3 * width + n],
                          dev[4 * width:4 * width + n], dev[:2 * n].view(torch.int64),
                          dev[5 * width:5 * width + n], dev[6 * width:6 * width + n], extra=status)
