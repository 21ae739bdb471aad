"""One step's batch: the tokens it brings, flattened, with everything a kernel needs to know
about whose they are. It replaces the reference's module-global Context
(tinyinfer/utils/context.py:8-36) and the tensors of prepare_batch
(tinyinfer/engine/model_runner.py:310-357) by one explicit object.

All index arrays live in ONE int32 device buffer filled by ONE host-to-device copy from pinned
memory; the fields below are views into it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import torch


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places among them whose logits
    are wanted (indices into ``tokens``)."""
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()
    feed_row: int = -1       # >= 0: the entry's LAST token is not known on the host yet: it is row feed_row of
                             # the device tensor of sampled tokens handed to the step (its value here is ignored)


@dataclass
class CacheView:
    """What a mixer sees of the cache entry it works on in this step."""
    kv: Optional[torch.Tensor]            # [2, pages, kv_heads, page_size, head_dim] or None
    block_table: Optional[torch.Tensor]   # int32 [S, max_blocks], -1 where no page is held
    page_size: int
    writes: bool                          # False: read what another entry of the run order wrote
    state: Optional[torch.Tensor]         # [slots, *shape] or None


@dataclass
class StepContext:
    num_tokens: int
    num_seqs: int
    num_logit_rows: int
    token_ids: torch.Tensor        # int32 [T]
    positions: torch.Tensor        # int32 [T]  absolute position of each token in its request
    token_seq: torch.Tensor        # int32 [T]  which entry of the step the token belongs to
    cu_seqlens: torch.Tensor       # int32 [S + 1]
    q_starts: torch.Tensor         # int32 [S]  position of each entry's first token
    context_lens: torch.Tensor     # int32 [S]  length of each request after this step
    state_slots: torch.Tensor      # int32 [S]
    logit_rows: torch.Tensor       # int32 [N]  flat rows whose logits are wanted
    block_tables: List[torch.Tensor]      # per cache group: int32 [S, max_blocks]
    status: Optional[torch.Tensor]        # int32 [1] device word set by kernels on a bad index
    # host copies, for choosing kernels and grids without a device read
    q_lens: List[int] = field(default_factory=list)
    starts: List[int] = field(default_factory=list)
    max_q_len: int = 0
    max_context: int = 0
    num_real_seqs: int = 0         # entries before the padding rows of a graph-sized batch
    # the attention kernels' split of the batch: rows of single decoded tokens, and tiles
    # [entry, first row, rows, first position] of prompt portions
    decode_rows: Optional[torch.Tensor] = None
    num_decode: int = 0
    prefill_tiles: Optional[torch.Tensor] = None
    num_prefill_tiles: int = 0
    num_pair_tiles: int = 0        # the first so many tiles have more than 128 rows (two query tiles a CTA)
    # tokens that come from the device: per entry the flat row of its last token (-1: none) and the row of
    # the sampled-token tensor that holds it
    feed_dst: Optional[torch.Tensor] = None
    feed_src: Optional[torch.Tensor] = None
    num_feeds: int = 0
    # filled by the runner: entry of the run order -> CacheView
    views: Dict[int, CacheView] = field(default_factory=dict)

    def cache_view(self, exec_step) -> CacheView:
        base = self.views[exec_step.cache]
        if base.writes == exec_step.writes_cache:
            return base
        return CacheView(base.kv, base.block_table, base.page_size, exec_step.writes_cache, base.state)


class BatchBuffers:
    """Pinned host staging and the device buffer the step's index arrays are copied into."""

    def __init__(self, device, max_tokens: int, max_seqs: int, max_blocks: int, num_groups: int):
        self.device = torch.device(device)
        self.max_tokens, self.max_seqs = max_tokens, max_seqs
        self.max_blocks, self.num_groups = max_blocks, num_groups
        words = (3 * max_tokens + 6 * max_seqs + 1 + max_tokens + num_groups * max_seqs * max_blocks
                 + max_seqs + 4 * (max_tokens // 64 + max_seqs) + 160)   # tiles: at most one per 64 tokens plus one per request
        self.host = torch.empty(words, dtype=torch.int32, pin_memory=self.device.type == "cuda")
        self.dev = torch.empty(words, dtype=torch.int32, device=self.device)
        if self.device.type == "cuda":
            from ..ops import page_status
            self.status = page_status(self.device)      # read by whoever reads the device's status words
        else:
            self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._copied = torch.cuda.Event() if self.device.type == "cuda" else None
        self._copy_pending = False
        self.bytes_copied = 0              # host-to-device bytes of all steps so far
        self._host_np = self.host.numpy()
        self._last = None                  # what advance_decode() needs to know of the last fixed-layout step

    def build(self, entries: Sequence[StepEntry], starts: Sequence[int], slots: Sequence[int],
              tables: Sequence[Sequence[Sequence[int]]], fixed_layout: bool = False,
              pad_to: int = 0, pad_pages: Sequence[int] = (), pad_slot: int = 0,
              admissions: Optional[Sequence[int]] = None) -> StepContext:
        """``starts[i]``: tokens entry i's request already holds; ``slots[i]``: its state slot;
        ``tables[g][i]``: its block table in cache group g. ``fixed_layout`` pads every block
        table to the widest possible, so that two steps with the same numbers of tokens and
        requests put every array at the same address (what a captured CUDA graph needs).
        ``pad_to`` fills the step up to that many requests with padding rows (token 0 at position 0
        of a request whose only page is ``pad_pages[g]`` and whose state slot is ``pad_slot``, a page
        and a slot no real request holds), so that one
        captured graph serves a range of batch sizes; their logits come last and are dropped.
        ``admissions[i]``: a number that tells entry i's request from every other request there ever
        was (the cache manager's admission serial); with it a step of single decoded tokens can be
        followed by ``advance_decode``."""
        num_real = len(entries)
        if pad_to > num_real:
            extra = pad_to - num_real
            entries = list(entries) + [StepEntry(("pad", i), [0], [0]) for i in range(extra)]
            starts = list(starts) + [0] * extra
            slots = list(slots) + [pad_slot] * extra
            tables = [list(tables[g]) + [[pad_pages[g]] if g < len(pad_pages) else []] * extra
                      for g in range(self.num_groups)]
        q_lens = [len(e.tokens) for e in entries]
        t, s = sum(q_lens), len(entries)
        if t > self.max_tokens or s > self.max_seqs:
            raise ValueError(f"step of {t} tokens / {s} requests exceeds the buffers "
                             f"({self.max_tokens} / {self.max_seqs})")
        ids: List[int] = []
        pos: List[int] = []
        seq: List[int] = []
        rows: List[int] = []
        cu = [0]
        for i, e in enumerate(entries):
            n = q_lens[i]
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {e.request_id!r}: wanted place {w} is not among its {n} tokens")
                rows.append(cu[-1] + w)
            ids.extend(max(0, int(x)) for x in e.tokens)    # a token yet to come from the device is staged as 0
            pos.extend(range(starts[i], starts[i] + n))
            seq.extend([i] * n)
            cu.append(cu[-1] + n)
        ctx_lens = [starts[i] + q_lens[i] for i in range(s)]
        widths = [max((len(tb) for tb in tables[g]), default=0) for g in range(self.num_groups)]
        widths = [self.max_blocks if fixed_layout else max(1, w) for w in widths]
        if max(widths, default=1) > self.max_blocks:
            raise ValueError("a block table is longer than the buffers allow")
        flat: List[int] = []
        offsets = {}

        def put(name, values):
            offsets[name] = (len(flat), len(values))
            flat.extend(values)
            flat.extend([0] * (-len(flat) % 4))             # keep every array 16-byte aligned

        put("ids", ids); put("pos", pos); put("seq", seq); put("cu", cu)
        put("starts", list(starts)); put("ctx", ctx_lens); put("slots", list(slots)); put("rows", rows)
        from ..ops import plan_attention
        decode_rows, tiles, num_pairs = plan_attention(q_lens, starts)
        put("dec", decode_rows); put("tiles", tiles)
        feed_dst = [cu[i + 1] - 1 if e.feed_row >= 0 else -1 for i, e in enumerate(entries)]
        feed_src = [max(0, e.feed_row) for e in entries]
        put("fdst", feed_dst); put("fsrc", feed_src)
        for g in range(self.num_groups):
            w = widths[g]
            padded: List[int] = []
            for tb in tables[g]:
                padded.extend(tb)
                padded.extend([-1] * (w - len(tb)))
            put(f"bt{g}", padded)
        n = len(flat)
        if self._copy_pending:                 # the last step's copy may still be reading the host buffer
            self._copied.synchronize()
        self.host[:n] = torch.tensor(flat, dtype=torch.int32)
        self.dev[:n].copy_(self.host[:n], non_blocking=True)
        self.bytes_copied += 4 * n
        if self._copied is not None:
            self._copied.record()
            self._copy_pending = True

        def view(name):
            o, ln = offsets[name]
            return self.dev[o:o + ln]

        ctx = StepContext(
            num_tokens=t, num_seqs=s, num_logit_rows=len(rows),
            token_ids=view("ids"), positions=view("pos"), token_seq=view("seq"),
            cu_seqlens=view("cu"), q_starts=view("starts"), context_lens=view("ctx"),
            state_slots=view("slots"), logit_rows=view("rows"),
            block_tables=[view(f"bt{g}").view(s, widths[g]) for g in range(self.num_groups)],
            status=self.status, q_lens=q_lens, starts=list(starts), max_q_len=max(q_lens, default=0),
            max_context=max(ctx_lens, default=0), decode_rows=view("dec"), num_decode=len(decode_rows),
            prefill_tiles=view("tiles"), num_prefill_tiles=len(tiles) // 4, num_pair_tiles=num_pairs,
            num_real_seqs=num_real,
            feed_dst=view("fdst"), feed_src=view("fsrc"), num_feeds=sum(1 for d in feed_dst if d >= 0))
        self._last = None
        if fixed_layout and admissions is not None and all(n == 1 for n in q_lens):
            self._last = dict(key=(tuple(admissions), s), ctx=ctx, words=n,
                              offsets=offsets, widths=widths, num_real=num_real,
                              table_lens=[[len(tb) for tb in tables[g][:num_real]] for g in range(self.num_groups)])
        return ctx

    def advance_decode(self, admissions: Sequence[int], pad_to: int, tokens: Sequence[int], starts: Sequence[int],
                       tables: Sequence[Sequence[Sequence[int]]],
                       feed_rows: Optional[Sequence[int]] = None) -> Optional[StepContext]:
        """The step after a step of single decoded tokens, for the same requests (the same admissions,
        not merely the same ids: a request that ended and whose id came back holds other pages and
        another state slot) in the same order, each with its next token: only the token ids, the positions and the pages that were added
        change, so the staging buffer is patched instead of rebuilt. Block tables must only have
        grown (no window gave pages back). Returns None if the last step was not such a step."""
        last = self._last
        if last is None or last["key"] != (tuple(admissions), max(pad_to, len(admissions))):
            return None
        n_real, off, host = last["num_real"], last["offsets"], self._host_np
        if self._copy_pending:
            self._copied.synchronize()
        host[off["ids"][0]:off["ids"][0] + n_real] = tokens
        host[off["pos"][0]:off["pos"][0] + n_real] = starts
        host[off["starts"][0]:off["starts"][0] + n_real] = starts
        ctx_lens = [st + 1 for st in starts]
        host[off["ctx"][0]:off["ctx"][0] + n_real] = ctx_lens
        if feed_rows is None:
            host[off["fdst"][0]:off["fdst"][0] + n_real] = -1
            num_feeds = 0
        else:                                   # entry i is flat row i of a step of single tokens
            host[off["fdst"][0]:off["fdst"][0] + n_real] = [i if r >= 0 else -1 for i, r in enumerate(feed_rows)]
            host[off["fsrc"][0]:off["fsrc"][0] + n_real] = [max(0, r) for r in feed_rows]
            num_feeds = sum(1 for r in feed_rows if r >= 0)
        for g in range(self.num_groups):
            base, w, lens = off[f"bt{g}"][0], last["widths"][g], last["table_lens"][g]
            for i, tb in enumerate(tables[g]):
                if len(tb) != lens[i]:
                    if len(tb) < lens[i] or len(tb) > w:
                        self._last = None
                        return None
                    host[base + i * w + lens[i]:base + i * w + len(tb)] = tb[lens[i]:]
                    lens[i] = len(tb)
        n = last["words"]
        self.dev[:n].copy_(self.host[:n], non_blocking=True)
        self.bytes_copied += 4 * n
        if self._copied is not None:
            self._copied.record()
            self._copy_pending = True
        ctx = last["ctx"]
        ctx.num_feeds = num_feeds
        ctx.starts = list(starts)
        ctx.max_context = max(ctx_lens)          # padding rows have context 1
        return ctx
