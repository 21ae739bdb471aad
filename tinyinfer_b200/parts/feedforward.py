"""Dense gated feed-forward (SwiGLU): down(silu(gate(x)) * up(x)), no bias
(tinyinfer/models/qwen3.py:148-150,170-175 of the reference). Gate and up are packed as one
[2I, H] matrix so that one matrix product feeds the activation, which acts on the float32
accumulators as the reference's kernel does (tinyinfer/csrc/mlp.cu:116-141)."""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorSpec, register_feed_forward


class GatedMLP(FeedForward):
    graph_safe = True
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

    def forward_prenorm(self, x, norm, link, next_norm, step=None):
        rms = norm.as_rms()
        if rms is None or not ops.norm_link_ok(x):
            return super().forward_prenorm(x, norm, link, next_norm, step)
        if link is not None and link.weight is rms[0]:
            hidden = ops.gated_linear(link.scaled, self.w_gate_up, link=link, link_eps=rms[1])
        else:
            hidden = ops.gated_linear(norm.forward(x), self.w_gate_up)
        after = next_norm.as_rms() if next_norm is not None else None
        if after is None:
            return ops.linear(hidden, self.w_down, residual=x), None
        return ops.linear(hidden, self.w_down, residual=x, next_norm_weight=after[0])


register_feed_forward("gated_mlp", GatedMLP)
