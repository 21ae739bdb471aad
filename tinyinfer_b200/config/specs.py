"""Typed descriptions of the parts a decoder is put together from.

A *spec* is plain data: the sizes and constants of one part and a ``kind`` string that a
registry of ``tinyinfer_b200.parts`` maps to the class that runs it. An architecture's
configuration (``tinyinfer_b200.config.qwen3``) turns the keys of its ``config.json`` into one
``ModelSpec``; nothing downstream reads ``config.json`` again, and no part knows which
architecture asked for it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last axis. ``kind='rmsnorm'``: w * x * rsqrt(mean(x^2) + eps)."""
    size: int
    eps: float
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class PositionSpec:
    """How positions enter a mixer. ``kind='rope'``: half-split rotation of the first
    ``rotary_dim`` features of every head with inv_freq[j] = theta ** (-2j / rotary_dim).
    ``kind='none'``: positions are not used."""
    kind: str = "rope"
    theta: float = 10000.0
    rotary_dim: int = 0


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention over a paged key/value cache."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    position: PositionSpec
    qk_norm: Optional[NormSpec] = None      # per-head norm of q and k before the rotation
    bias: bool = False                      # bias on the q, k, v and o projections
    window: Optional[int] = None            # None: all keys; n: the last n keys (itself included)
    kind: str = "attention"

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim


@dataclass(frozen=True)
class GatedMLPSpec:
    """Dense gated feed-forward: down(act(gate(x)) * up(x)), no bias."""
    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class LayerSpec:
    """One block: which mixer, which feed-forward, their norms and how they are arranged.
    ``arrangement='pre_norm'``: x += mixer(norm1(x)); x += feed_forward(norm2(x))."""
    mixer: object
    feed_forward: object
    mixer_norm: NormSpec
    feed_forward_norm: NormSpec
    arrangement: str = "pre_norm"


@dataclass(frozen=True)
class ExecStep:
    """One entry of the run order. ``layer`` indexes ``ModelSpec.layers`` (a layer may be named
    more than once). ``cache`` names the cache entry the mixer works on; ``writes_cache`` is
    False for an entry that only reads what an earlier entry wrote there."""
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class TensorNames:
    """Checkpoint names of an architecture, as patterns. ``{i}`` is the layer index."""
    embedding: str = "model.embed_tokens.weight"
    layer: str = "model.layers.{i}."
    mixer: str = "self_attn."
    feed_forward: str = "mlp."
    mixer_norm: str = "input_layernorm."
    feed_forward_norm: str = "post_attention_layernorm."
    final_norm: str = "model.norm."
    head: str = "lm_head.weight"


@dataclass(frozen=True)
class ModelSpec:
    """Everything the generic decoder needs: sizes, the layers, and the order they run in."""
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: Tuple[LayerSpec, ...]
    execution: Tuple[ExecStep, ...]
    final_norm: NormSpec
    tie_embeddings: bool
    max_positions: int
    names: TensorNames = field(default_factory=TensorNames)

    def __post_init__(self):
        seen = set()
        for step in self.execution:
            if not 0 <= step.layer < len(self.layers):
                raise ValueError(f"execution names layer {step.layer}, the model has {len(self.layers)}")
            if step.writes_cache:
                if step.cache in seen:
                    raise ValueError(f"cache entry {step.cache} has two writers in the run order")
                seen.add(step.cache)
            elif step.cache not in seen:
                raise ValueError(f"cache entry {step.cache} is read before any entry writes it")

    @property
    def num_cache_entries(self) -> int:
        return 1 + max((s.cache for s in self.execution), default=-1)


def default_execution(num_layers: int) -> Tuple[ExecStep, ...]:
    """Every layer once, in order, each with a cache entry of its own."""
    return tuple(ExecStep(layer=i, cache=i, writes_cache=True) for i in range(num_layers))
