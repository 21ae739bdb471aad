"""Turns rows of logits into tokens, every row with its own options
(tinyinfer/layers/sampler.py:13-75 of the reference: greedy rows take the argmax, the others
temperature, top-k threshold and Gumbel-max). One kernel launch for the whole batch."""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from .params import SamplingParams


class Drawn:
    """Tokens on their way to the host (``Sampler.sample_async``)."""

    def __init__(self, tokens, packed, n, with_nll, device, arrived=None, give_back=None):
        self.tokens = tokens              # int32 device tensor [n (+ status words)], or None if nothing was drawn
        self._packed, self._n, self._with_nll, self._device, self._arrived = packed, n, with_nll, device, arrived
        self._give_back = give_back

    def result(self):
        if self.tokens is None:
            return ([], []) if self._with_nll else []
        if self._arrived is not None:
            self._arrived.synchronize()
        values = self._packed.tolist()
        if self._give_back is not None:
            self._give_back()
            self._give_back = None
        count = self.tokens.shape[0]
        host = [int(t) for t in values[:count]]
        if count > self._n:
            ops.raise_on_status(self._device, *host[self._n:self._n + 2])
        return (host[:self._n], values[count:]) if self._with_nll else host[:self._n]


class Sampler:
    def __init__(self, device, engine_seed: int = 0):
        self.device = torch.device(device)
        self.engine_seed = int(engine_seed)
        self._staging = [None, None]       # pinned host words the per-row parameters are staged in
        self._staging_np = [None, None]
        self._turn = 0
        self._host_pool = {}               # dtype -> pinned buffers that drawn tokens are copied into

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               stream_ids: Sequence[int], steps: Sequence[int], with_nll: bool = False,
               status: Optional[torch.Tensor] = None):
        """``logits`` float32 [N, V]; row i is drawn with ``params[i]`` from the random stream
        (seed, ``stream_ids[i]``, ``steps[i]``): the request's number and how many tokens it has
        generated. Returns python ints (one device-to-host copy); with ``with_nll`` a pair
        (tokens, negative log-likelihood of each token under its row's softmax).
        ``status``: the device's status words (``ops.status_words``); they come home in the same copy
        as the tokens, and KernelError is raised instead of tokens if a kernel of the step set one."""
        return self.sample_async(logits, params, stream_ids, steps, with_nll, status).result()

    def sample_async(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                     stream_ids: Sequence[int], steps: Sequence[int], with_nll: bool = False,
                     status: Optional[torch.Tensor] = None) -> "Drawn":
        """As ``sample``, without waiting: the kernels and the copy to the host are enqueued and a handle
        comes back. ``handle.tokens`` is the int32 device tensor of the drawn tokens (a later step may take
        its inputs from it on the device); ``handle.result()`` waits for the copy and returns what
        ``sample`` returns."""
        n = logits.shape[0]
        tokens = self._sample_device(logits, params, stream_ids, steps, status)
        if tokens is None:
            return Drawn(None, None, 0, with_nll, self.device)
        packed = tokens
        if with_nll:
            # tinyinfer/engine/model_runner.py:446-454 of the reference: tokens and NLL leave together
            packed = torch.cat((tokens.to(torch.float64), ops.token_nll(logits, tokens[:n]).to(torch.float64)))
        if self.device.type != "cuda":
            return Drawn(tokens, packed, n, with_nll, self.device)
        # pinned buffers go round: a handle gives its buffer back when its result has been read
        pool = self._host_pool.setdefault(packed.dtype, [])
        words = packed.shape[0]
        buf = next((b for b in pool if b.shape[0] >= words), None)
        if buf is None:
            buf = torch.empty(max(words, 1024), dtype=packed.dtype, pin_memory=True)
        else:
            pool.remove(buf)
        host = buf[:words]
        host.copy_(packed, non_blocking=True)
        arrived = torch.cuda.Event()
        arrived.record()
        return Drawn(tokens, host, n, with_nll, self.device, arrived, lambda: pool.append(buf))

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
        # two staging arrays in turn: the copy of the call before may not have run yet when this one is
        # filled (a step is launched before the one before it has been read back); the one before that has
        self._turn ^= 1
        if self._staging[self._turn] is None or self._staging[self._turn].numel() < words:
            self._staging[self._turn] = torch.empty(max(words, 7 * 64), dtype=torch.int32,
                                                    pin_memory=self.device.type == "cuda")
            self._staging_np[self._turn] = self._staging[self._turn].numpy()
        host = self._staging_np[self._turn]
        seeds = np.asarray([self.engine_seed if p.seed is None else int(p.seed) for p in params], dtype=np.int64)
        host[:2 * n] = seeds.view(np.int32)
        host[2 * width:2 * width + n] = np.asarray([float(p.temperature) for p in params], dtype=np.float32).view(np.int32)
        host[3 * width:3 * width + n] = [0 if p.topk >= vocab else p.topk for p in params]
        host[4 * width:4 * width + n] = [1 if p.greedy else 0 for p in params]
        host[5 * width:5 * width + n] = [int(x) & 0x7FFFFFFF for x in stream_ids]
        host[6 * width:6 * width + n] = [int(x) & 0x7FFFFFFF for x in steps]
        dev = self._staging[self._turn][:words].to(self.device, non_blocking=True)
        return ops.sample(logits, dev[2 * width:2 * width + n].view(torch.float32), dev[3 * width:3 * width + n],
                          dev[4 * width:4 * width + n], dev[:2 * n].view(torch.int64),
                          dev[5 * width:5 * width + n], dev[6 * width:6 * width + n], extra=status)
