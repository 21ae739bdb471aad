"""Continuous batching above the step function: admits requests, cuts prompts into portions under
a token budget, decodes round-robin, finishes and frees.

The policy is the reference's (tinyinfer/engine/scheduler.py:63-166 schedule, :169-236
postprocess): decode first, in round-robin order; while anything waits, decoding may take at
most max_num_seqs - 1 requests and 80 % of the token budget (:69-70); then portions of waiting
prompts with what is left, a prompt's pages being taken when it is admitted (:134-137). Unlike the
reference, prompts that were begun are continued, oldest first, before new ones are admitted. Added:
a cap on one request's portion (``prefill_chunk``; the reference has a TODO there, :143), and a
decided behaviour when pages run out, which the reference lacks (it stops with "scheduler made
no progress", tinyinfer/engine/llm_engine.py:199-200):

* a prompt that cannot get its pages waits; a decoding request that cannot get its next page
  sits the step out;
* if therefore a step would run nothing while requests remain, the running request admitted
  last is preempted: its pages are given back and it returns to the head of the waiting queue
  to be recomputed from its tokens so far (its generated tokens are kept);
* a request that cannot fit even alone is finished with reason ``cache_exhausted``; a prompt
  that can never fit is refused when it is added.
"""
from __future__ import annotations

from collections import deque
from typing import Deque, Dict, List

from ..cache import CacheManager
from ..config import EngineConfig
from .sequence import ScheduledItem, Sequence, SequenceStatus


class Scheduler:
    def __init__(self, config: EngineConfig, manager: CacheManager, eos_token_id: int = -1):
        self.max_num_seqs = config.max_num_seqs
        self.max_num_batched_tokens = config.max_num_batched_tokens
        self.max_model_len = config.max_model_len
        self.prefill_chunk = config.prefill_chunk
        self.eos_token_id = eos_token_id
        self.manager = manager
        self.waiting: Deque[Sequence] = deque()
        self.running: Deque[Sequence] = deque()
        self.retiring: List[Sequence] = []         # their last token is still on its way to the host
        self.num_preemptions = 0
        self.finished_early: List[Sequence] = []   # ended by the scheduler, not by a token

    # ------------------------------------------------------------------ queue
    def add(self, seq: Sequence) -> None:
        if seq.num_tokens >= self.max_model_len:
            raise ValueError(f"prompt of {seq.num_tokens} tokens does not fit max_model_len "
                             f"{self.max_model_len}")
        need = self.manager.pages_for(seq.num_tokens + 1)
        for g in self.manager.groups:
            if need > g.pool.num_pages:
                raise ValueError(f"prompt of {seq.num_tokens} tokens needs {need} pages, the cache "
                                 f"has {g.pool.num_pages}")
        self.waiting.append(seq)

    def is_finished(self) -> bool:
        return not self.waiting and not self.running and not self.retiring

    # ------------------------------------------------------------------ schedule
    def schedule(self) -> List[ScheduledItem]:
        while True:
            items = self._schedule_once()
            if items or self.is_finished():
                return items
            if not self._make_room():
                return items

    def _schedule_once(self) -> List[ScheduledItem]:
        items: List[ScheduledItem] = []
        token_budget = self.max_num_batched_tokens
        seq_budget = self.max_num_seqs
        decode_seq_budget = seq_budget if not self.waiting else max(0, seq_budget - 1)
        decode_token_budget = token_budget if not self.waiting else max(0, int(0.8 * token_budget))

        # phase A: one token for every running request the budgets allow, round-robin
        for _ in range(len(self.running)):
            if decode_token_budget < 1 or decode_seq_budget <= 0:
                break
            seq = self.running[0]
            self.running.rotate(-1)
            if not seq.needs_decode:
                continue
            start = seq.num_computed_tokens
            if not self.manager.can_extend(seq.seq_id, start + 1):
                continue                                   # no page for its next token: sits out
            self.manager.extend(seq.seq_id, start + 1)
            seq.mark_scheduled()
            items.append(ScheduledItem(seq, start, 1, is_prefill=False, sample_after=True))
            token_budget -= 1
            seq_budget -= 1
            decode_token_budget -= 1
            decode_seq_budget -= 1

        # phase B: portions of waiting prompts with the remaining budget. Prompts that already hold
        # pages go first, in the order they arrived, then new ones are admitted: a prompt that was begun
        # is finished before another is begun, so the pages it holds soon serve a request that decodes
        # and ends. (Taking the waiting requests in turn, as the reference does, scheduler.py:126-164,
        # begins every prompt before it finishes any; with more prompts than pages for them all, each
        # holds its share of the pool, none can go on, and preemption only moves the pages around.)
        order = [q for q in self.waiting if q.admitted] + [q for q in self.waiting if not q.admitted]
        for seq in order:
            if token_budget <= 0 or seq_budget <= 0:
                break
            if not seq.admitted:
                if not self.manager.can_admit():
                    break
                # with a prefix cache the request takes over kept pages that its tokens begin
                # with (tinyinfer/engine/scheduler.py:132-137); what they cover is not run again
                rc = self.manager.admit(seq.seq_id, seq.token_ids[:seq.num_prefill_tokens])
                if not self.manager.can_extend(seq.seq_id, seq.num_prefill_tokens):
                    self.manager.release(seq.seq_id)       # its pages are not there yet: it waits
                    continue
                self.manager.extend(seq.seq_id, seq.num_prefill_tokens)
                seq.admitted = True
                seq.num_computed_tokens = rc.length
                seq.num_cached_tokens = rc.length
            remaining = seq.num_prefill_tokens - seq.num_computed_tokens
            chunk = min(remaining, token_budget)
            if self.prefill_chunk > 0:
                chunk = min(chunk, self.prefill_chunk)
            start = seq.num_computed_tokens
            seq.mark_scheduled()
            items.append(ScheduledItem(seq, start, chunk, is_prefill=True,
                                       sample_after=start + chunk == seq.num_prefill_tokens))
            token_budget -= chunk
            seq_budget -= 1
        return items

    def _make_room(self) -> bool:
        """Nothing could be scheduled although requests remain: free pages by preemption.
        Returns False if nothing can be done (then the caller reports no progress)."""
        held = [s for s in list(self.running) + list(self.waiting) if s.admitted]
        if len(held) >= 2:
            self._preempt(max(held, key=lambda s: s.seq_id))     # the one admitted last
            return True
        if held:
            # it holds all the pages there are to hold and still cannot go on
            seq = held[0]
            seq.mark_finished("cache_exhausted")
            self._drop(seq)
            self.finished_early.append(seq)
            return True
        return False

    def _preempt(self, seq: Sequence) -> None:
        self.manager.release(seq.seq_id)
        seq.admitted = False
        seq.num_computed_tokens = 0
        seq.num_prefill_tokens = seq.num_tokens            # recompute everything it has so far
        seq.num_preemptions += 1
        self.num_preemptions += 1
        if seq in self.running:
            self.running.remove(seq)
        if seq in self.waiting:
            self.waiting.remove(seq)
        seq.status = SequenceStatus.WAITING
        self.waiting.appendleft(seq)

    def _drop(self, seq: Sequence) -> None:
        if seq in self.running:
            self.running.remove(seq)
        if seq in self.waiting:
            self.waiting.remove(seq)
        if seq.admitted:
            self.manager.release(seq.seq_id)
            seq.admitted = False

    def schedule_ahead(self) -> List[ScheduledItem]:
        """The next step's items while a step is still in flight: what can be scheduled as things stand,
        without making room (preemption changes requests whose last token is not known yet)."""
        return self._schedule_once()

    # ------------------------------------------------------------------ after the step
    def advance(self, items: List[ScheduledItem]) -> None:
        """The first half of ``postprocess``, at the moment a step is LAUNCHED: everything that follows
        from counts alone. Every scheduled request moves on by its tokens; one that gets a token from this
        step gets a place for it (``PENDING``); a request that reaches its token or length limit with that
        token leaves the queues now (it is not scheduled again) and waits in ``retiring`` for ``retire``."""
        for item in items:
            seq = item.seq
            seq.num_computed_tokens = item.start_pos + item.num_tokens
            if not item.sample_after:
                continue
            last = seq.append_pending()
            reason = seq.length_stop(self.max_model_len)
            if reason is not None:
                seq.stopping = (last, reason)               # it ends when the token of this place is known
                if seq in self.running:
                    self.running.remove(seq)
                if seq in self.waiting:
                    self.waiting.remove(seq)
                self.retiring.append(seq)
            elif item.is_prefill:
                self.waiting.remove(seq)
                seq.status = SequenceStatus.RUNNING
                self.running.append(seq)

    def retire(self, items: List[ScheduledItem], sampled: Dict[int, int]) -> List[Sequence]:
        """The second half, when the step's tokens have been read back: they take their places, the
        end-of-sequence token is looked for, full pages join the prefix cache, finished requests give
        their pages back. A request that ended while a later step with it was already in flight is
        skipped here when that step retires. Returns the requests that finished."""
        finished: List[Sequence] = []
        for item in items:
            seq = item.seq
            if seq.is_finished:
                continue                                    # ended by an earlier step's token
            if item.sample_after:
                position = item.start_pos + item.num_tokens
                token = sampled[seq.seq_id]
                seq.resolve(position, token)
                reason = seq.token_stop(self.eos_token_id, token)
                if seq.stopping is not None and seq.stopping[0] == position:
                    reason = seq.stopping[1]
                if reason is not None:
                    del seq.token_ids[position + 1:]        # a place made for a token of a later step in flight
                    seq.num_computed_tokens = min(seq.num_computed_tokens, position)
                    seq.mark_finished(reason)
                    finished.append(seq)
            if seq.seq_id in self.manager:
                # full pages join the prefix cache, once every token whose key is stored is known (only
                # the newest two places can still be waiting)
                stored = self.manager.get(seq.seq_id).length
                if all(t >= 0 for t in seq.token_ids[max(0, stored - 2):stored]):
                    self.manager.note_tokens(seq.seq_id, seq.token_ids)
        for seq in finished:
            if seq in self.retiring:
                self.retiring.remove(seq)
            self._drop(seq)
        return finished

    def postprocess(self, items: List[ScheduledItem], sampled: Dict[int, int]) -> List[Sequence]:
        """Advances every scheduled request, appends sampled tokens, moves finished prompts to
        the running queue, finishes and frees. Returns the requests that finished."""
        finished: List[Sequence] = []
        for item in items:
            seq = item.seq
            seq.num_computed_tokens = item.start_pos + item.num_tokens
            if seq.seq_id in self.manager:
                self.manager.note_tokens(seq.seq_id, seq.token_ids)   # full pages join the prefix cache
            if not item.sample_after:
                continue                                    # a portion inside the prompt: no token
            seq.append_token(sampled[seq.seq_id])
            reason = seq.stop_reason(self.eos_token_id, self.max_model_len)
            if reason is not None:
                seq.mark_finished(reason)
                finished.append(seq)
            elif item.is_prefill:
                self.waiting.remove(seq)
                seq.status = SequenceStatus.RUNNING
                self.running.append(seq)
        for seq in finished:
            self._drop(seq)
        return finished
