"""Interfaces of the parts a decoder block is made of, and the registries that map a spec's
``kind`` to the class that runs it.

A part gets its sizes and constants from its spec, declares the tensors it wants by local name,
and is handed, at every step, the batch (``StepContext``) and, for mixers, a view of the cache
entry it works on. It never sees the model's configuration.

To add a part: write a spec dataclass with a ``kind`` field, a class deriving from ``Mixer``,
``FeedForward``, ``Norm`` or ``PositionEncoding``, and call the matching ``register_*``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part wants from the checkpoint.
    role 'matrix': kept in the compute dtype (bfloat16 or float32);
    role 'vector32': kept in float32 whatever the compute dtype (norm weights, biases of
    32-bit parts); role 'int': kept as int32."""
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"          # random-weights mode: 'normal' N(0, std) or 'ones_noise' 1 + N(0, 0.1)


@dataclass(frozen=True)
class CacheNeed:
    """Paged keys and values a mixer wants per token: ``num_kv_heads * head_dim`` for K and V
    each. ``window`` None: every key stays; n: only the last n positions are ever read, older
    pages may be given back."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size (for instance a recurrent state): one slot of ``shape``
    per live request, zeroed when the request is admitted."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    def __init__(self, spec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = device

    def tensors(self) -> Dict[str, TensorSpec]:
        """Local tensor names (e.g. 'q_proj.weight') and what they must look like."""
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receives exactly the tensors named by ``tensors()``, on the device, role applied."""


class Norm(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def forward_rows(self, x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """Norm of the selected rows only. Parts without a fused kernel may gather first."""
        return self.forward(x.index_select(0, rows.long()))

    def as_rms(self):
        """(weight float32 [size], eps) if this norm is y = weight * x * rsqrt(mean(x^2) + eps), so
        that the products around it may share it between them (``ops.linear``); None otherwise."""
        return None


class PositionEncoding(Part):
    """Owned by a mixer, to which it hands ``rotation()``: an ``ops.Rotation`` (which features are paired,
    and each pair's angle at every position, as inverse frequencies or as a table of cosines and sines)
    or None if positions are not used. The mixer passes it to the fused norm + rotation + append kernel
    without looking inside. A part that sets ``inv_freq`` (float32 [rotary_dim / 2]) and ``rotary_dim``
    gets the half-split rotation by position * inv_freq from the default below."""
    inv_freq = None
    rotary_dim = 0

    def rotation(self):
        if self.inv_freq is None:
            return None
        from .. import ops
        return ops.Rotation(self.rotary_dim, inv_freq=self.inv_freq)


class Mixer(Part):
    # True if forward() only launches kernels on the step's device tensors (no host reads, no
    # Python branching on the step's contents): such a step may be captured in a CUDA graph.
    graph_safe = False

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, x: torch.Tensor, step, cache) -> torch.Tensor:
        """x [T, hidden] (normed) -> [T, hidden]. ``step`` is the StepContext of the batch,
        ``cache`` the CacheView of the entry this run works on."""
        raise NotImplementedError

    def forward_residual(self, x, residual, step, cache) -> torch.Tensor:
        """residual + forward(x). Parts whose last kernel can add the residual override this."""
        from .. import ops
        return ops.add(residual, self.forward(x, step, cache))

    def forward_prenorm(self, x, norm: "Norm", link, next_norm: Optional["Norm"], step, cache):
        """x + forward(norm(x)) for ``x`` BEFORE its norm. ``link``: None, or what the part that made x
        left for this norm (an ``ops.NormLink``); ``next_norm``: the norm the result will pass through
        next, if known. Returns (result, link for that next norm or None). Parts whose products can
        share a norm between them override this; the default runs the norm on its own."""
        return self.forward_residual(norm.forward(x), x, step, cache), None


class FeedForward(Part):
    graph_safe = False      # as for a mixer: a feed-forward that picks its experts' rows on the host is not

    def forward(self, x: torch.Tensor, step) -> torch.Tensor:
        raise NotImplementedError

    def forward_residual(self, x, residual, step) -> torch.Tensor:
        from .. import ops
        return ops.add(residual, self.forward(x, step))

    def forward_prenorm(self, x, norm: "Norm", link, next_norm: Optional["Norm"], step):
        """As ``Mixer.forward_prenorm``, without a cache."""
        return self.forward_residual(norm.forward(x), x, step), None


class Block:
    """An arrangement of one mixer, one feed-forward and their norms."""

    def __init__(self, spec, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm,
                 feed_forward_norm: Norm):
        self.spec = spec
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm

    def forward(self, x, step, cache):
        raise NotImplementedError

    def forward_linked(self, x, link, next_norm: Optional[Norm], step, cache):
        """``forward`` that also takes what the block before left for this block's first norm and
        returns what this block leaves for ``next_norm`` (the first norm behind it): (x, link)."""
        return self.forward(x, step, cache), None


# ------------------------------------------------------------------ registries
_MIXERS: Dict[str, Callable] = {}
_FEED_FORWARDS: Dict[str, Callable] = {}
_NORMS: Dict[str, Callable] = {}
_POSITIONS: Dict[str, Callable] = {}
_BLOCKS: Dict[str, Callable] = {}


def _register(table, what):
    def register(kind: str, factory: Callable) -> None:
        table[kind] = factory
    register.__doc__ = f"Registers the class that runs {what} specs of this kind."
    return register


def _build(table, what):
    def build(spec, *args, **kwargs):
        kind = getattr(spec, "kind", None)
        if kind not in table:
            raise KeyError(f"no {what} registered for kind {kind!r}; known: {sorted(table)}")
        return table[kind](spec, *args, **kwargs)
    return build


register_mixer = _register(_MIXERS, "mixer")
register_feed_forward = _register(_FEED_FORWARDS, "feed-forward")
register_norm = _register(_NORMS, "norm")
register_position = _register(_POSITIONS, "position-encoding")
register_block = _register(_BLOCKS, "block arrangement")
build_mixer = _build(_MIXERS, "mixer")
build_feed_forward = _build(_FEED_FORWARDS, "feed-forward")
build_norm = _build(_NORMS, "norm")
build_position = _build(_POSITIONS, "position-encoding")


def build_block(spec, dtype, device) -> Block:
    if spec.arrangement not in _BLOCKS:
        raise KeyError(f"no block arrangement {spec.arrangement!r}; known: {sorted(_BLOCKS)}")
    return _BLOCKS[spec.arrangement](
        spec,
        build_mixer(spec.mixer, dtype, device),
        build_feed_forward(spec.feed_forward, dtype, device),
        build_norm(spec.mixer_norm, dtype, device),
        build_norm(spec.feed_forward_norm, dtype, device))
