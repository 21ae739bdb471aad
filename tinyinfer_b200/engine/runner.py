"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

One call runs only the tokens it is given, as one flat batch, against the cache that earlier
calls left: portions of prompts beside single decoded tokens, cut anywhere. It is the only
forward path of the framework: generation, the trace replay and the benchmark all go through
``ModelRunner.step``. It corresponds to the reference's ModelRunner.run / prepare_batch
(tinyinfer/engine/model_runner.py:310-460) without the sampling, which is a separate call on
the returned logits.
"""
from __future__ import annotations

from typing import Hashable, List, Optional, Sequence

import torch

from ..cache import CacheManager, CacheStorage, bytes_per_page
from .batch import BatchBuffers, CacheView, StepContext, StepEntry


class ModelRunner:
    def __init__(self, model, *, page_size: int, num_pages: int, max_requests: int,
                 max_tokens_per_step: int, max_model_len: int, max_seqs_per_step: int = 0,
                 poison_cache: bool = False, cuda_graphs: bool = False,
                 prefix_caching: bool = False):
        """``max_requests``: requests that may hold cache at a time (state slots);
        ``max_seqs_per_step``: requests in one step (0: the same); ``cuda_graphs``: steps made of
        single decoded tokens only are captured once per batch size and replayed;
        ``prefix_caching``: full pages are kept under a hash of their tokens after their request
        ends (the caller admits requests with their tokens and reports them after each step)."""
        self.model = model
        self.device = model.device
        needs = model.cache_needs()
        self.manager = CacheManager(needs, page_size, num_pages, max_requests,
                                    prefix_caching=prefix_caching)
        self.storage = CacheStorage(needs, self.manager, model.dtype, self.device, poison=poison_cache)
        self.max_model_len = max_model_len
        max_blocks = (max_model_len + page_size - 1) // page_size
        self.buffers = BatchBuffers(self.device, max_tokens_per_step,
                                    max_seqs_per_step or max_requests, max_blocks,
                                    max(1, len(self.manager.groups)))
        self.steps_run = 0
        self.cuda_graphs = (cuda_graphs and self.device.type == "cuda"
                            and all(b.mixer.graph_safe and b.feed_forward.graph_safe for b in model.blocks))
        self._tables_only_grow = all(g.need.window is None for g in self.manager.groups)
        self._graphs = {}          # requests in the step -> (graph, static logits, kernels)
        self._graph_pool = None
        self.graph_replays = 0

    # ------------------------------------------------------------------ requests
    def admit(self, request_id: Hashable) -> None:
        self.manager.admit(request_id)

    def release(self, request_id: Hashable) -> None:
        self.manager.release(request_id)

    def length(self, request_id: Hashable) -> int:
        return self.manager.get(request_id).length

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry], fed_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs the entries' tokens and returns float32 logits [N, V] on the device, N being the
        number of wanted places, in the order of the entries and of each ``want``.
        A request id not seen before is admitted. Raises CacheExhausted before anything runs
        if the pages do not suffice for ALL entries; the cache is then as it was before the call.
        ``fed_tokens``: int32 device tensor of tokens sampled by the step before; an entry with
        ``feed_row >= 0`` takes its last token from there, on the device (the host need not have seen it)."""
        entries = [e for e in entries if len(e.tokens) > 0]
        ids = [e.request_id for e in entries]
        if len(set(ids)) != len(ids):
            raise ValueError("a request may appear once in a step")
        if not entries:
            return torch.empty((0, self.model.spec.vocab_size), dtype=torch.float32, device=self.device)
        vocab = self.model.spec.vocab_size
        starts: List[int] = []
        for e in entries:
            start = self.manager.get(e.request_id).length if e.request_id in self.manager else 0
            if start + len(e.tokens) > self.max_model_len:
                raise ValueError(f"request {e.request_id!r} would reach {start + len(e.tokens)} tokens, "
                                 f"the limit is {self.max_model_len}")
            known = e.tokens if e.feed_row < 0 else e.tokens[:-1]
            for tok in known:
                if not 0 <= int(tok) < vocab:
                    raise ValueError(f"token id {tok} is outside the vocabulary of {vocab}")
            if e.feed_row >= 0 and fed_tokens is None:
                raise ValueError(f"request {e.request_id!r} takes a token from the device, but none were handed over")
            starts.append(start)
        admitted_here = [rid for rid in ids if rid not in self.manager]
        try:
            for rid in admitted_here:
                self.admit(rid)
            self.manager.extend_many([(e.request_id, start + len(e.tokens)) for e, start in zip(entries, starts)])
        except Exception:
            for rid in admitted_here:          # a step that cannot run leaves the cache as it found it
                if rid in self.manager:
                    self.manager.release(rid)
            raise
        for slot in self.manager.take_fresh_slots():      # whoever admitted them: their state starts clean
            self.storage.reset_state_slot(slot)
        caches = [self.manager.get(rid) for rid in ids]
        num_groups = len(self.manager.groups)
        tables = [[rc.tables[g] for rc in caches] for g in range(num_groups)] or [[[] for _ in caches]]
        # a request is told from its namesakes of earlier by the serial of its admission: an id may
        # come back after its request has ended, with other pages and another state slot
        serials = [rc.serial for rc in caches]
        decode_only = self.cuda_graphs and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)
        pad_to = 0
        if decode_only:
            pad_to = min(graph_batch_size(len(entries)), self.buffers.max_seqs)
        ctx = None
        if decode_only and self._tables_only_grow:
            # the same requests as in the step before, one more token each: patch the staged arrays
            ctx = self.buffers.advance_decode(serials, pad_to, [max(0, int(e.tokens[0])) for e in entries], starts, tables,
                                              [e.feed_row for e in entries] if fed_tokens is not None else None)
        if ctx is None:
            ctx = self.buffers.build(entries, starts, [rc.state_slot for rc in caches], tables,
                                     fixed_layout=decode_only, pad_to=pad_to, admissions=serials,
                                     pad_pages=[CacheStorage.dump_page(self.manager, g) for g in range(num_groups)],
                                     pad_slot=CacheStorage.dump_slot(self.manager))
            self._bind_views(ctx)
        if ctx.num_feeds:
            from .. import ops
            ops.feed_tokens(ctx.token_ids, ctx.feed_dst, ctx.feed_src, fed_tokens)
        logits = self._graph_forward(ctx) if decode_only else self.model.forward(ctx)
        for e, start in zip(entries, starts):
            self.manager.commit(e.request_id, start + len(e.tokens))
        self.steps_run += 1
        return logits

    def _graph_forward(self, ctx: StepContext) -> torch.Tensor:
        """A step of single decoded tokens: replayed from a CUDA graph captured for this number
        of requests (batches are padded up to a few sizes, so a handful of graphs serve every batch
        size). The graph reads the step's arrays from the fixed device buffer that
        ``build`` has just filled; the attention launch is sized for the longest context a request
        may have, so one graph covers every context length (the kernel shares out the keys there are).
        The returned logits live in the graph's own memory until the next replay."""
        from ..ops import library
        ctx.max_context = self.max_model_len
        key = ctx.num_seqs
        hit = self._graphs.get(key)
        real = ctx.num_real_seqs
        if hit is not None:
            hit[0].replay()
            self.graph_replays += 1
            library.count_replayed_launches(hit[2])
            return hit[1][:real]
        logits = self.model.forward(ctx)              # eager once: also sets up every kernel it uses
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        launches_before = library.launch_count()
        with torch.cuda.graph(graph, pool=self._graph_pool):
            static_logits = self.model.forward(ctx)
        kernels_in_graph = library.launch_count() - launches_before
        library.count_replayed_launches(-kernels_in_graph)       # captured, not run
        if self._graph_pool is None:
            self._graph_pool = graph.pool()
        self._graphs[key] = (graph, static_logits, kernels_in_graph)
        return logits[:real]

    def _bind_views(self, ctx: StepContext) -> None:
        for entry in range(self.model.spec.num_cache_entries):
            g = self.manager.group_of_entry.get(entry)
            ctx.views[entry] = CacheView(
                kv=self.storage.kv[entry],
                block_table=ctx.block_tables[g] if g is not None else None,
                page_size=self.manager.page_size, writes=True, state=self.storage.state[entry])

    def close(self) -> None:
        """Lets go of the device memory this runner holds (cache pages, captured graphs and their pool,
        the model's tensors), so that another engine can be built in the same process."""
        from .. import ops
        self._graphs.clear()
        self._graph_pool = None
        self.buffers._last = None
        self.storage.kv.clear()
        self.storage.state.clear()
        for block in self.model.blocks:
            for part in (block.mixer, block.feed_forward, block.mixer_norm, block.feed_forward_norm):
                for name, value in list(vars(part).items()):
                    if isinstance(value, torch.Tensor):
                        setattr(part, name, None)
        self.model.embedding = self.model.head = None
        ops.release_scratch(self.device)
        if self.device.type == "cuda":
            import gc
            gc.collect()
            torch.cuda.empty_cache()

    def status_words(self) -> torch.Tensor:
        """The device's two status words (``ops.status_words``): kernels of a step set them when a
        bounded wait ran out or a token or key had no page. A sampler can take them home with the tokens."""
        from .. import ops
        return ops.status_words(self.device)

    def check_status(self) -> None:
        """Reads the status words and raises if a kernel of an earlier step set one (synchronises)."""
        from .. import ops
        ops.check_kernel_status()


_GRAPH_BATCH_SIZES = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512, 768, 1024)


def graph_batch_size(n: int) -> int:
    """The batch size of the captured graph that serves a decode step of ``n`` requests."""
    for size in _GRAPH_BATCH_SIZES:
        if size >= n:
            return size
    return n


def pages_that_fit(model, page_size: int, free_bytes: int, utilization: float,
                   max_tokens_per_step: int, max_requests: int) -> int:
    """Pages per group that the device can hold beside the step's activations: the reference's
    formula (tinyinfer/engine/model_runner.py:131-176) with an analytic activation bound in
    place of its dummy forward."""
    spec = model.spec
    widest = spec.hidden_size
    for layer in spec.layers:
        mixer, ffn = layer.mixer, layer.feed_forward
        widest = max(widest, getattr(mixer, "q_size", 0) + 2 * getattr(mixer, "kv_size", 0),
                     2 * getattr(ffn, "intermediate_size", 0))
    itemsize = model.dtype.itemsize
    activations = max_tokens_per_step * (4 * spec.hidden_size + 3 * widest) * itemsize
    activations += max_requests * spec.vocab_size * 4 * 3
    budget = int(free_bytes * utilization) - activations
    per_page = bytes_per_page(model.cache_needs(), page_size, model.dtype)
    if per_page == 0:
        return 1
    return max(0, budget // per_page)
