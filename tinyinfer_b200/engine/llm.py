"""The Python entry point: ``LLM(...).generate(prompts, SamplingParams)``, in the manner of the
reference (tinyinfer/llm.py:4-6, tinyinfer/engine/llm_engine.py:28-230): the same method names
(generate, generate_token_ids, add_request, step) and result keys (token_ids, all_token_ids,
num_cached_tokens, statistics, text)."""
from __future__ import annotations

import json
from itertools import count
from pathlib import Path
from typing import Dict, List, Optional, Sequence as Seq, Union

import torch

from ..cache import prefix_caching_possible
from ..config import EngineConfig
from ..sampling import Sampler, SamplingParams
from .batch import StepEntry
from .loading import build_random_model, load_model, require_cuda
from .runner import ModelRunner, pages_that_fit
from .scheduler import Scheduler
from .sequence import PENDING, ScheduledItem, Sequence


class _InFlight:
    """A launched step whose sampled tokens are still on the device."""

    def __init__(self, items, sampling, drawn, row_of):
        self.items, self.sampling, self.drawn, self.row_of = items, sampling, drawn, row_of


class LLM:
    def __init__(self, model: Union[str, Path, object], engine_config: Optional[EngineConfig] = None,
                 *, random_weights: Optional[int] = None, tokenizer=None, **overrides):
        """``model``: a folder with config.json and safetensors, or (with ``random_weights=seed``)
        a typed model configuration whose weights are drawn on the device.
        ``overrides`` set fields of ``EngineConfig`` by name (max_num_seqs=..., dtype=...)."""
        self.config = engine_config or EngineConfig()
        for key, value in overrides.items():
            if not hasattr(self.config, key):
                raise TypeError(f"unknown engine option {key!r}")
            setattr(self.config, key, value)
        self.config.validate()
        device = require_cuda(self.config.device)
        if random_weights is not None:
            self.model_config = model
            self.model = build_random_model(model, random_weights, self.config.dtype, device)
            self.model_dir = None
        else:
            self.model, self.model_config = load_model(model, self.config.dtype, device)
            self.model_dir = Path(model)
        spec = self.model.spec
        # tinyinfer/config.py:39-40: a request is never longer than the model's positions
        self.config.max_model_len = min(self.config.max_model_len, spec.max_positions)
        page = self.config.kvcache_block_size
        num_pages = self.config.num_kvcache_blocks
        if num_pages == 0:
            torch.cuda.empty_cache()        # what loading held for a moment counts as free again
            free, _total = torch.cuda.mem_get_info(device)
            num_pages = pages_that_fit(self.model, page, free, self.config.gpu_memory_utilization,
                                       self.config.max_num_batched_tokens, self.config.max_num_seqs)
            per_request = (self.config.max_model_len + page - 1) // page
            num_pages = min(num_pages, per_request * self.config.max_num_seqs)
            if num_pages <= 0:
                raise RuntimeError("no device memory left for the cache")
            self.config.num_kvcache_blocks = num_pages
        possible = prefix_caching_possible(self.model.cache_needs())
        if self.config.enable_prefix_caching and not possible:
            raise ValueError("enable_prefix_caching: this model has windows or mixer state, whose "
                             "pages cannot stand for a prompt's first tokens")
        if self.config.enable_prefix_caching is None:
            self.config.enable_prefix_caching = possible
        self.runner = ModelRunner(
            self.model, page_size=page, num_pages=num_pages, max_requests=self.config.live_requests,
            prefix_caching=self.config.enable_prefix_caching,
            max_seqs_per_step=self.config.max_num_seqs,
            max_tokens_per_step=self.config.max_num_batched_tokens,
            max_model_len=self.config.max_model_len, cuda_graphs=self.config.cuda_graphs)
        eos = self.config.eos_token_id
        if eos < 0:
            model_eos = getattr(self.model_config, "eos_token_id", None)
            eos = -1 if model_eos is None else int(model_eos)
        self.tokenizer = tokenizer
        if self.tokenizer is None and self.model_dir is not None:
            self.tokenizer = _load_tokenizer(self.model_dir)
        if eos < 0 and self.tokenizer is not None and getattr(self.tokenizer, "eos_token_id", None) is not None:
            eos = int(self.tokenizer.eos_token_id)
        self.scheduler = Scheduler(self.config, self.runner.manager, eos_token_id=eos)
        self.sampler = Sampler(device, self.config.seed)
        self._ids = count()
        self.sequences: Dict[int, Sequence] = {}
        self._in_flight: Optional[_InFlight] = None      # the step whose tokens have not been read back yet

    def close(self) -> None:
        """Gives the device memory back (weights, cache, graphs); the engine cannot be used afterwards."""
        self.runner.close()

    # ------------------------------------------------------------------ requests
    def add_request(self, token_ids: Seq[int], params: Optional[SamplingParams] = None) -> int:
        vocab = self.model.spec.vocab_size
        for t in token_ids:
            if not 0 <= int(t) < vocab:
                raise ValueError(f"token id {t} is outside the vocabulary of {vocab}")
        seq = Sequence(next(self._ids), list(token_ids), params or SamplingParams())
        self.scheduler.add(seq)
        self.sequences[seq.seq_id] = seq
        return seq.seq_id

    def step(self) -> List[ScheduledItem]:
        """schedule -> run -> sample -> postprocess; returns what was scheduled. The kernels' status
        words come home with the sampled tokens: a step whose kernels gave up on a wait or met a token
        without a page raises KernelError instead of handing on tokens drawn from its logits.

        With ``overlap_steps`` (the default) a call launches a step and only then reads back the tokens of
        the step the call before launched: the host schedules and stages step n + 1 while the device runs
        step n, and the tokens that step n + 1 needs from step n reach it on the device. What depends on
        counts alone (how far a request is, whether it has reached its token limit) is settled when a step
        is launched; what depends on the token (end of sequence, the prefix cache's page hashes, timing
        marks) when it has been read back, one call later. A request that ends on an end-of-sequence token
        has then already run in the next step; that step's token for it is dropped. Call ``step`` until
        ``is_finished()``: the last call launches nothing and reads the last tokens back."""
        before = self._in_flight
        if before is None:
            items = self.scheduler.schedule()
        else:
            items = self.scheduler.schedule_ahead()
            if not items:
                # nothing fits as things stand: read the step in flight back first, then schedule with
                # everything known (making room, if need be, changes requests; none may be waiting for a token)
                self._in_flight = None
                self._retire(before)
                before = None
                items = self.scheduler.schedule()
        launched = self._launch(items, before) if items else None
        if launched is not None and not self.config.overlap_steps:
            self._retire(launched)
            launched = None
        self._in_flight = launched
        if before is not None:
            self._retire(before)
        return items

    def is_finished(self) -> bool:
        """No request waits, runs, or has a token on its way back."""
        return self._in_flight is None and self.scheduler.is_finished()

    def _launch(self, items: List[ScheduledItem], before) -> "_InFlight":
        entries = []
        for it in items:
            tokens = it.seq.token_ids[it.start_pos:it.start_pos + it.num_tokens]
            feed_row = -1
            if tokens[-1] == PENDING:          # sampled by the step in flight: it stays on the device
                feed_row = before.row_of[it.seq.seq_id]
                tokens = tokens[:-1] + [0]
            entries.append(StepEntry(it.seq.seq_id, tokens, [it.num_tokens - 1] if it.sample_after else [], feed_row))
        fed = before.drawn.tokens if before is not None else None
        logits = self.runner.step(entries, fed_tokens=fed)
        sampling = [it for it in items if it.sample_after]
        drawn = self.sampler.sample_async(
            logits, [it.seq.sampling_params for it in sampling],
            [it.seq.seq_id for it in sampling], [it.seq.num_completion_tokens for it in sampling],
            with_nll=self.config.track_nll, status=self.runner.status_words())
        self.scheduler.advance(items)
        return _InFlight(items, sampling, drawn, {it.seq.seq_id: row for row, it in enumerate(sampling)})

    def _retire(self, flight: "_InFlight") -> None:
        tokens = flight.drawn.result()
        if self.config.track_nll:
            tokens, nlls = tokens
            for it, nll in zip(flight.sampling, nlls):
                if not it.seq.is_finished:
                    it.seq.sum_nll += nll
        self.scheduler.retire(flight.items, {it.seq.seq_id: tok for it, tok in zip(flight.sampling, tokens)})

    # ------------------------------------------------------------------ generation
    def generate_token_ids(self, prompts: Seq[Seq[int]],
                           sampling_params: Union[SamplingParams, Seq[SamplingParams], None] = None):
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            params = [sampling_params or SamplingParams()] * len(prompts)
        else:
            params = list(sampling_params)
        if len(params) != len(prompts):
            raise ValueError("prompts and sampling params length mismatch")
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        while not self.is_finished():
            if not self.step() and not self.is_finished():
                raise RuntimeError("scheduler made no progress while requests remain")
        out = []
        for i in ids:
            seq = self.sequences.pop(i)
            out.append({"token_ids": seq.token_ids[seq.num_prompt_tokens:],
                        "all_token_ids": list(seq.token_ids),
                        "num_cached_tokens": seq.num_cached_tokens,
                        "finish_reason": seq.finish_reason,
                        "statistics": seq.statistics()})
        return out

    def generate(self, prompts, sampling_params=None):
        """``prompts``: strings (needs the folder's tokenizer) or lists of token ids."""
        as_text = [isinstance(p, str) for p in prompts]
        if any(as_text):
            if self.tokenizer is None:
                raise RuntimeError("text prompts need a tokenizer in the model folder; pass token ids")
            prompts = [self.tokenizer.encode(p, add_special_tokens=False) if t else p
                       for p, t in zip(prompts, as_text)]
        outputs = self.generate_token_ids(prompts, sampling_params)
        if self.tokenizer is not None:
            for out in outputs:
                out["text"] = self.tokenizer.decode(out["token_ids"], skip_special_tokens=True)
        return outputs


def _load_tokenizer(folder: Path):
    """The folder's tokenizer, if it has one (tinyinfer/engine/llm_engine.py:41)."""
    if not any((folder / f).is_file() for f in ("tokenizer.json", "tokenizer.model", "vocab.json")):
        return None
    try:
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(str(folder))
    except Exception:
        return None
