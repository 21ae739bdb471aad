"""Block arrangements. 'pre_norm' is the reference's decoder layer
(tinyinfer/models/qwen3.py:192-221): x += mixer(norm(x)); x += feed_forward(norm(x)).
The residual sums are left to the parts' last kernels where they can fuse them."""
from __future__ import annotations

from .base import Block, register_block


class PreNormBlock(Block):
    def forward(self, x, step, cache):
        x = self.mixer.forward_residual(self.mixer_norm.forward(x), x, step, cache)
        x = self.feed_forward.forward_residual(self.feed_forward_norm.forward(x), x, step)
        return x


register_block("pre_norm", PreNormBlock)
