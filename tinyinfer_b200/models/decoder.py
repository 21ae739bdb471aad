"""The generic decoder: embedding, blocks run in the order the spec lists, final norm on the
wanted rows, output projection to float32 logits.

It plays the role of the reference's Qwen3ForCausalLM / Qwen3Model
(tinyinfer/models/qwen3.py:225-288) but knows no architecture: which mixer, feed-forward and
norm a layer has, and which layers run in which order on which cache entry, all come from the
``ModelSpec``. Only rows that want logits reach the final norm and the head, as in the
reference's runner (tinyinfer/engine/model_runner.py:381-395).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import ops
from ..config.specs import ModelSpec
from ..parts import CacheNeed, StateNeed, TensorSpec, build_block, build_norm


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, got {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.blocks = [build_block(layer, dtype, self.device) for layer in spec.layers]
        self.final_norm = build_norm(spec.final_norm, dtype, self.device)
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ tensors
    def _part_prefixes(self, i: int):
        n = self.spec.names
        base = n.layer.format(i=i)
        block = self.blocks[i]
        return [(base + n.mixer, block.mixer), (base + n.feed_forward, block.feed_forward),
                (base + n.mixer_norm, block.mixer_norm),
                (base + n.feed_forward_norm, block.feed_forward_norm)]

    def expected_tensors(self) -> Dict[str, TensorSpec]:
        """Checkpoint name -> what the tensor must look like, in a fixed order."""
        spec = self.spec
        out: Dict[str, TensorSpec] = {
            spec.names.embedding: TensorSpec((spec.vocab_size, spec.hidden_size))}
        for i in range(len(self.blocks)):
            for prefix, part in self._part_prefixes(i):
                for local, ts in part.tensors().items():
                    out[prefix + local] = ts
        for local, ts in self.final_norm.tensors().items():
            out[spec.names.final_norm + local] = ts
        if not spec.tie_embeddings:
            out[spec.names.head] = TensorSpec((spec.vocab_size, spec.hidden_size))
        return out

    def ignored_tensors(self) -> List[str]:
        """Names a checkpoint may carry that this model has no use for (a tied model's head,
        tinyinfer/utils/loader.py:103-105 of the reference)."""
        return [self.spec.names.head] if self.spec.tie_embeddings else []

    def load_tensors(self, tensors) -> None:
        """``tensors[name]``: the tensor of that name of ``expected_tensors()``, on the device, role
        applied. Every name is asked for once, in the order of ``expected_tensors()``, and a part's
        tensors are let go of as soon as the part has packed them: a mapping that makes each tensor
        when it is asked for (a reader of a file, a random draw) never has more than one part's
        tensors alive beside the model, which is what lets a model of 65 GB load into 180 GB."""
        spec = self.spec
        self.embedding = tensors[spec.names.embedding].contiguous()
        for i in range(len(self.blocks)):
            for prefix, part in self._part_prefixes(i):
                part.load({local: tensors[prefix + local] for local in part.tensors()})
        self.final_norm.load({local: tensors[spec.names.final_norm + local]
                              for local in self.final_norm.tensors()})
        self.head = self.embedding if spec.tie_embeddings else tensors[spec.names.head].contiguous()

    def weight_bytes(self) -> int:
        total = 0
        for name, ts in self.expected_tensors().items():
            n = 1
            for s in ts.shape:
                n *= s
            total += n * (self.dtype.itemsize if ts.role == "matrix" else 4)
        return total

    # ------------------------------------------------------------------ cache needs
    def cache_needs(self) -> List[Tuple[Optional[CacheNeed], Optional[StateNeed]]]:
        """For every cache entry of the run order: the pages and the state its writer wants."""
        needs: List[Tuple[Optional[CacheNeed], Optional[StateNeed]]] = \
            [(None, None)] * self.spec.num_cache_entries
        for step in self.spec.execution:
            if step.writes_cache:
                mixer = self.blocks[step.layer].mixer
                needs[step.cache] = (mixer.cache_need(), mixer.state_need())
        return needs

    # ------------------------------------------------------------------ forward
    # The frame around the blocks is three methods, so that a model whose frame differs (an embedding
    # that is scaled, logits that are capped, a norm elsewhere) overrides one of them in a subclass and
    # registers that class for its architecture; blocks, cache and step function stay as they are.
    def forward(self, step) -> torch.Tensor:
        """Runs the tokens of ``step`` (a StepContext) and returns float32 logits [N, V] at
        ``step.logit_rows``."""
        x = self.run_blocks(self.embed(step), step)
        if step.num_logit_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        return self.logits(x, step)

    def embed(self, step) -> torch.Tensor:
        """The residual stream [T, hidden] the first block starts from."""
        return ops.embedding(step.token_ids, self.embedding)

    def run_blocks(self, x: torch.Tensor, step) -> torch.Tensor:
        """The blocks in the order the spec lists, each on its cache entry."""
        link = None        # what a block's last product leaves for the next block's first norm (see parts.base)
        order = self.spec.execution
        for i, entry in enumerate(order):
            after = self.blocks[order[i + 1].layer].mixer_norm if i + 1 < len(order) else None
            x, link = self.blocks[entry.layer].forward_linked(x, link, after, step, step.cache_view(entry))
        return x

    def logits(self, x: torch.Tensor, step) -> torch.Tensor:
        """Float32 logits [N, V] of the rows ``step.logit_rows`` (there is at least one) of the last
        block's output."""
        h = self.final_norm.forward_rows(x, step.logit_rows)
        return ops.linear(h, self.head, out_float32=True)
