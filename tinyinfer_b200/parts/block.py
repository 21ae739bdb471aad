"""Block arrangements. 'pre_norm' is the reference's decoder layer
(tinyinfer/models/qwen3.py:192-221): x += mixer(norm(x)); x += feed_forward(norm(x)).
The residual sums are left to the parts' last kernels where they can fuse them."""
from __future__ import annotations

from .base import Block, register_block


class PreNormBlock(Block):
    def forward(self, x, step, cache):
        return self.forward_linked(x, None, None, step, cache)[0]

    def forward_linked(self, x, link, next_norm, step, cache):
        # each part gets its input before the norm, with the norm and with the norm that comes after it:
        # parts whose products can share a norm between them do so (a decode step saves the norm kernels)
        x, link = self.mixer.forward_prenorm(x, self.mixer_norm, link, self.feed_forward_norm, step, cache)
        x, link = self.feed_forward.forward_prenorm(x, self.feed_forward_norm, link, next_norm, step)
        return x, link


register_block("pre_norm", PreNormBlock)
