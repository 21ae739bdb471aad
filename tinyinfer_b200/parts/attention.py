"""Grouped-query attention mixer over the paged cache.

Order of operations as in the reference (tinyinfer/models/qwen3.py:106-132): packed q/k/v
projection, per-head RMSNorm of q and k, rotation, append of k and v to the cache, attention of
every token over its own request's keys, output projection. The q, k and v matrices are packed
row-wise as [q; k; v] like the reference's loader does (tinyinfer/utils/loader.py:52-96).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import CacheNeed, Mixer, TensorSpec, build_position, register_mixer


class Attention(Mixer):
    graph_safe = True

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.position = build_position(spec.position, dtype, device)
        self._rotation = self.position.rotation()      # opaque here: the kernel reads it
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None
        self.q_norm = self.k_norm = None

    def cache_need(self):
        return CacheNeed(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def tensors(self):
        s = self.spec
        t = {
            "q_proj.weight": TensorSpec((s.q_size, s.hidden_size)),
            "k_proj.weight": TensorSpec((s.kv_size, s.hidden_size)),
            "v_proj.weight": TensorSpec((s.kv_size, s.hidden_size)),
            "o_proj.weight": TensorSpec((s.hidden_size, s.q_size)),
        }
        if s.qk_norm is not None:
            t["q_norm.weight"] = TensorSpec((s.head_dim,), role="vector32", init="ones_noise")
            t["k_norm.weight"] = TensorSpec((s.head_dim,), role="vector32", init="ones_noise")
        if s.bias:
            t["q_proj.bias"] = TensorSpec((s.q_size,), role="vector32")
            t["k_proj.bias"] = TensorSpec((s.kv_size,), role="vector32")
            t["v_proj.bias"] = TensorSpec((s.kv_size,), role="vector32")
            t["o_proj.bias"] = TensorSpec((s.hidden_size,), role="vector32")
        return t

    def load(self, tensors):
        s = self.spec
        self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                                tensors["v_proj.weight"]], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].contiguous()
        if s.qk_norm is not None:
            self.q_norm = tensors["q_norm.weight"]
            self.k_norm = tensors["k_norm.weight"]
        if s.bias:
            self.b_qkv = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"],
                                    tensors["v_proj.bias"]]).contiguous()
            self.b_o = tensors["o_proj.bias"]

    def _attend(self, x, step, cache, link=None, link_eps=0.0):
        s = self.spec
        qkv = (ops.linear(x, self.w_qkv, bias=self.b_qkv) if link is None
               else ops.linear(x, self.w_qkv, bias=self.b_qkv, link=link, link_eps=link_eps))
        q = ops.qk_norm_rope_append(
            qkv, num_heads=s.num_heads, num_kv_heads=s.num_kv_heads, head_dim=s.head_dim,
            q_norm_weight=self.q_norm, k_norm_weight=self.k_norm,
            eps=s.qk_norm.eps if s.qk_norm is not None else 0.0,
            rotation=self._rotation, positions=step.positions, token_seq=step.token_seq,
            kv_cache=cache.kv if cache.writes else None, block_table=cache.block_table,
            status=step.status)
        return ops.paged_attention(q, cache.kv, positions=step.positions, token_seq=step.token_seq,
                                   block_table=cache.block_table, scale=s.scale, window=s.window,
                                   step=step, status=step.status)

    def forward(self, x, step, cache):
        return ops.linear(self._attend(x, step, cache), self.w_o, bias=self.b_o)

    def forward_residual(self, x, residual, step, cache):
        return ops.linear(self._attend(x, step, cache), self.w_o, bias=self.b_o, residual=residual)

    def forward_prenorm(self, x, norm, link, next_norm, step, cache):
        rms = norm.as_rms()
        if rms is None or not ops.norm_link_ok(x):
            return super().forward_prenorm(x, norm, link, next_norm, step, cache)
        # few tokens: the packed projection takes the norm's second half (if the product before left the
        # first), and the output projection leaves the first half of the norm that follows
        if link is not None and link.weight is rms[0]:
            attended = self._attend(link.scaled, step, cache, link=link, link_eps=rms[1])
        else:
            attended = self._attend(norm.forward(x), step, cache)
        after = next_norm.as_rms() if next_norm is not None else None
        if after is None:
            return ops.linear(attended, self.w_o, bias=self.b_o, residual=x), None
        return ops.linear(attended, self.w_o, bias=self.b_o, residual=x, next_norm_weight=after[0])


register_mixer("attention", Attention)
