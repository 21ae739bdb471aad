"""A request on its way through the engine: its tokens, how far its keys are computed, its
timing marks. Mirrors the reference's Sequence (tinyinfer/engine/sequence.py:25-170) without the
process-global page size and counter; the pages themselves are the cache manager's business."""
from __future__ import annotations

import math
import time
from dataclasses import dataclass
from enum import Enum, auto
from typing import List, Optional

from ..sampling.params import SamplingParams


class SequenceStatus(Enum):
    WAITING = auto()     # not all of its prompt is computed yet
    RUNNING = auto()     # decoding
    FINISHED = auto()


PENDING = -1      # stands in token_ids for a token that has been sampled on the device but not read back yet


class Sequence:
    def __init__(self, seq_id: int, token_ids: List[int], sampling_params: SamplingParams):
        if not token_ids:
            raise ValueError("token_ids cannot be empty")
        self.seq_id = seq_id
        self.status = SequenceStatus.WAITING
        self.sampling_params = sampling_params
        self.token_ids = [int(t) for t in token_ids]       # prompt + generated so far
        self.num_prompt_tokens = len(self.token_ids)
        self.num_prefill_tokens = len(self.token_ids)       # grows if the request is recomputed
        self.num_computed_tokens = 0                        # tokens whose keys are in the cache
        self.num_cached_tokens = 0                          # prompt tokens found in a prefix cache
        self.num_preemptions = 0
        self.finish_reason: Optional[str] = None
        self.stopping = None           # (position, reason): it ends once the token of that place has been read back
        self.admitted = False
        self.sum_nll = 0.0
        self.arrival_time = time.perf_counter()
        self.first_scheduled_time: Optional[float] = None
        self.first_token_time: Optional[float] = None
        self.finished_time: Optional[float] = None
        self.output_token_times: List[float] = []

    @property
    def num_tokens(self) -> int:
        return len(self.token_ids)

    @property
    def num_completion_tokens(self) -> int:
        return self.num_tokens - self.num_prompt_tokens

    @property
    def last_token(self) -> int:
        return self.token_ids[-1]

    @property
    def is_finished(self) -> bool:
        return self.status is SequenceStatus.FINISHED

    @property
    def prefill_done(self) -> bool:
        return self.num_computed_tokens >= self.num_prefill_tokens

    @property
    def needs_decode(self) -> bool:
        # the newest token has no keys yet: it is the next step's input (sequence.py:103-105)
        return self.prefill_done and self.num_computed_tokens < self.num_tokens

    def mark_scheduled(self) -> None:
        if self.first_scheduled_time is None:
            self.first_scheduled_time = time.perf_counter()

    def append_token(self, token: int) -> None:
        self.token_ids.append(int(token))
        self._stamp_token()

    def append_pending(self) -> int:
        """Makes room for a token that a step in flight is sampling; returns its position."""
        self.token_ids.append(PENDING)
        return len(self.token_ids) - 1

    def resolve(self, position: int, token: int) -> None:
        """The token that was pending at ``position`` has been read back."""
        if self.token_ids[position] != PENDING:
            raise RuntimeError(f"request {self.seq_id}: position {position} was not waiting for a token")
        self.token_ids[position] = int(token)
        self._stamp_token()

    def _stamp_token(self) -> None:
        now = time.perf_counter()
        if self.first_token_time is None:
            self.first_token_time = now
        self.output_token_times.append(now)

    def mark_finished(self, reason: str) -> None:
        self.status = SequenceStatus.FINISHED
        self.finish_reason = reason
        self.finished_time = time.perf_counter()

    def stop_reason(self, eos_token_id: int, max_model_len: int) -> Optional[str]:
        """Why generation ends now, or None (tinyinfer/engine/sequence.py:152-170; the end-of-
        sequence token stays in the output)."""
        return self.length_stop(max_model_len) or self.token_stop(eos_token_id, self.last_token)

    def length_stop(self, max_model_len: int) -> Optional[str]:
        """The reasons to end that depend on counts alone: known before the last token is."""
        if self.num_completion_tokens >= self.sampling_params.max_tokens:
            return "max_tokens"
        if self.num_tokens >= max_model_len:
            return "max_model_len"
        return None

    def token_stop(self, eos_token_id: int, token: int) -> Optional[str]:
        if (not self.sampling_params.ignore_eos and eos_token_id >= 0
                and self.num_completion_tokens > 0 and token == eos_token_id):
            return "eos"
        return None

    def statistics(self) -> dict:
        """Token counts, latencies in seconds and rates (tinyinfer/engine/sequence.py:174-275)."""
        out_tokens = self.num_completion_tokens
        decode_tokens = max(0, out_tokens - 1)

        def span(a, b):
            return None if a is None or b is None else b - a

        decode_time = span(self.first_token_time, self.finished_time)
        e2e = span(self.arrival_time, self.finished_time)
        itls = [b - a for a, b in zip(self.output_token_times, self.output_token_times[1:])]

        def pct(q):
            if not itls:
                return None
            ordered = sorted(itls)
            return ordered[round((len(ordered) - 1) * q)]

        return {
            "prompt_tokens": self.num_prompt_tokens, "output_tokens": out_tokens,
            "decode_tokens": decode_tokens, "total_tokens": self.num_tokens,
            "cached_tokens": self.num_cached_tokens,
            "cache_hit_rate": self.num_cached_tokens / self.num_prompt_tokens,
            "preemptions": self.num_preemptions, "finish_reason": self.finish_reason,
            "queue_time": span(self.arrival_time, self.first_scheduled_time),
            "prefill_time": span(self.first_scheduled_time, self.first_token_time),
            "decode_time": decode_time, "ttft": span(self.arrival_time, self.first_token_time),
            "service_time": span(self.first_scheduled_time, self.finished_time),
            "e2e_latency": e2e,
            "tpot": decode_time / decode_tokens if decode_time is not None and decode_tokens else None,
            "tpot_p50": pct(0.50), "tpot_p95": pct(0.95), "tpot_p99": pct(0.99),
            "mean_itl": sum(itls) / len(itls) if itls else None,
            "min_itl": min(itls) if itls else None, "max_itl": max(itls) if itls else None,
            "decode_throughput": decode_tokens / decode_time if decode_time and decode_tokens else None,
            "request_throughput": out_tokens / e2e if e2e else None,
            "perplexity": math.exp(self.sum_nll / out_tokens) if out_tokens else None,
        }


@dataclass
class ScheduledItem:
    """A request's share of one step (tinyinfer/engine/sequence.py:282-289)."""
    seq: Sequence
    start_pos: int
    num_tokens: int
    is_prefill: bool
    sample_after: bool
