"""Position encodings. The rotary part owns the float32 inverse frequencies
inv_freq[j] = theta ** (-2j / rotary_dim) (tinyinfer/layers/rotary_embedding.py:38-48 of the
reference, which also keeps them in float32 under a bfloat16 model, :51-70); the rotation itself
happens inside the mixer's fused norm + rotation + cache-append kernel."""
from __future__ import annotations

import torch

from .base import PositionEncoding, register_position


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {spec.rotary_dim}")
        exponent = torch.arange(0, spec.rotary_dim, 2, dtype=torch.float32) / spec.rotary_dim
        self.inv_freq = (1.0 / (spec.theta ** exponent)).to(device)
        self.rotary_dim = spec.rotary_dim


class NoPosition(PositionEncoding):
    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.inv_freq = None
        self.rotary_dim = 0


register_position("rope", RotaryEncoding)
register_position("none", NoPosition)
