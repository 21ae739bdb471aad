"""RMSNorm part (tinyinfer/layers/layernorm.py:7-25 of the reference; kernel formula
tinyinfer/csrc/rmsnorm.cu:22-50). The weight is kept in float32 because the norm is computed in
float32 whatever the compute dtype."""
from __future__ import annotations

from .. import ops
from .base import Norm, TensorSpec, register_norm


class RMSNorm(Norm):
    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.weight = None

    def tensors(self):
        return {"weight": TensorSpec((self.spec.size,), role="vector32", init="ones_noise")}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, x):
        return ops.rmsnorm(x, self.weight, self.spec.eps)

    def forward_rows(self, x, rows):
        return ops.rmsnorm(x, self.weight, self.spec.eps, rows=rows)

    def as_rms(self):
        return self.weight, self.spec.eps


register_norm("rmsnorm", RMSNorm)
