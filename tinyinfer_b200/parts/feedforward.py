"""Dense gated feed-forward (SwiGLU): down(silu(gate(x)) * up(x)), no bias
(tinyinfer/models/qwen3.py:148-150,170-175 of the reference). Gate and up are packed as one
[2I, H] matrix so that one matrix product feeds the activation, which acts on the float32
accumulators as the reference's kernel does (tinyinfer/csrc/mlp.cu:116-141)."""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorSpec, register_feed_forward


class GatedMLP(FeedForward):
    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} is not supported (silu only)")
        self.w_gate_up = self.w_down = None

    def tensors(self):
        s = self.spec
        return {
            "gate_proj.weight": TensorSpec((s.intermediate_size, s.hidden_size)),
            "up_proj.weight": TensorSpec((s.intermediate_size, s.hidden_size)),
            "down_proj.weight": TensorSpec((s.hidden_size, s.intermediate_size)),
        }

    def load(self, tensors):
        self.w_gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]],
                                   dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def forward(self, x, step=None):
        return ops.linear(ops.gated_linear(x, self.w_gate_up), self.w_down)

    def forward_residual(self, x, residual, step=None):
        return ops.linear(ops.gated_linear(x, self.w_gate_up), self.w_down, residual=residual)


register_feed_forward("gated_mlp", GatedMLP)
