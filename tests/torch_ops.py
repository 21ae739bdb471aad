"""Plain PyTorch statement of every kernel of ``tinyinfer_b200.ops``, with the same signatures.

Two uses: (1) the reference each CUDA kernel is compared with in the gpu tests; (2) a stand-in
for the extension in CPU tests of the engine's logic (cache, batching, scheduling), installed
by the ``cpu_ops`` fixture. It is test code: the package never imports it, and without the CUDA
extension the package itself fails loudly.

Arithmetic is float32 (or float64 when the inputs are), one rounding to the input dtype at the
end of each op, like the kernels.
"""
from __future__ import annotations

import math

import numpy as np
import torch

import plain_qwen3 as plain


def _acc(t):
    return t.to(torch.float64 if t.dtype == torch.float64 else torch.float32)


def embedding(token_ids, table):
    return table[token_ids.long()]


def rmsnorm(x, weight, eps, rows=None):
    if rows is not None:
        x = x[rows.long()]
    xf = _acc(x)
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (weight.to(xf.dtype) * xf * inv).to(x.dtype)


def add(a, b):
    return (_acc(a) + _acc(b)).to(a.dtype)


def linear(x, w, bias=None, residual=None, out_float32=False):
    y = _acc(x) @ _acc(w).T
    if bias is not None:
        y = y + bias.to(y.dtype)
    if residual is not None:
        y = y + _acc(residual)
    return y.to(torch.float32 if out_float32 else x.dtype)


def gated_linear(x, w_gate_up):
    inter = w_gate_up.shape[0] // 2
    g = _acc(x) @ _acc(w_gate_up[:inter]).T
    u = _acc(x) @ _acc(w_gate_up[inter:]).T
    return ((g / (1.0 + torch.exp(-g))) * u).to(x.dtype)


def qk_norm_rope_append(qkv, *, num_heads, num_kv_heads, head_dim, q_norm_weight, k_norm_weight, eps,
                        positions, token_seq, kv_cache, block_table, rotation=None, inv_freq=None, rotary_dim=0,
                        status=None):
    """``rotation``: an object with rotary_dim, inv_freq or cos_sin, interleaved (ops.Rotation);
    ``inv_freq`` + ``rotary_dim`` alone mean the half-split rotation by position * inv_freq."""
    interleaved, cos_sin = False, None
    if rotation is not None:
        inv_freq, rotary_dim = rotation.inv_freq, rotation.rotary_dim
        interleaved, cos_sin = rotation.interleaved, rotation.cos_sin
    t = qkv.shape[0]
    x = _acc(qkv).view(t, num_heads + 2 * num_kv_heads, head_dim)
    q, k, v = x[:, :num_heads], x[:, num_heads:num_heads + num_kv_heads], x[:, num_heads + num_kv_heads:]

    def norm(a, w):
        if w is None:
            return a
        return w.to(a.dtype) * a * torch.rsqrt(a.pow(2).mean(-1, keepdim=True) + eps)

    def rot(a):
        if inv_freq is None and cos_sin is None:
            return a
        half = rotary_dim // 2
        if cos_sin is not None:
            rows = cos_sin[positions.long()]
            cos, sin = rows[:, None, :half].to(a.dtype), rows[:, None, half:].to(a.dtype)
        else:
            ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]
            cos, sin = ang.cos().to(a.dtype)[:, None, :], ang.sin().to(a.dtype)[:, None, :]
        if interleaved:
            a1, a2 = a[..., 0:rotary_dim:2], a[..., 1:rotary_dim:2]
            turned = torch.stack((a1 * cos - a2 * sin, a2 * cos + a1 * sin), dim=-1).flatten(-2)
            return torch.cat((turned, a[..., rotary_dim:]), dim=-1)
        a1, a2 = a[..., :half], a[..., half:rotary_dim]
        return torch.cat((a1 * cos - a2 * sin, a2 * cos + a1 * sin, a[..., rotary_dim:]), dim=-1)

    q = rot(norm(q, q_norm_weight))
    k = rot(norm(k, k_norm_weight))
    if kv_cache is not None:
        page_size = kv_cache.shape[3]
        pos = positions.long()
        page = block_table[token_seq.long(), pos // page_size].long()
        assert bool((page >= 0).all()), "a token without a page"
        kv_cache[0, page, :, pos % page_size, :] = k.to(kv_cache.dtype)
        kv_cache[1, page, :, pos % page_size, :] = v.to(kv_cache.dtype)
    return q.to(qkv.dtype).contiguous()


def paged_attention(q, kv_cache, *, positions, token_seq, block_table, scale, window=None, step=None,
                    status=None):
    t, hq, d = q.shape
    _, _, hkv, page_size, _ = kv_cache.shape
    group = hq // hkv
    out = torch.empty((t, hq, d), dtype=q.dtype, device=q.device)
    for i in range(t):
        pos = int(positions[i])
        lo = max(0, pos - window + 1) if window else 0
        js = torch.arange(lo, pos + 1, device=q.device)
        pages = block_table[int(token_seq[i]), js // page_size].long()
        assert bool((pages >= 0).all()), "a visible key without a page"
        k = _acc(kv_cache[0, pages, :, js % page_size, :])         # [n, hkv, d]
        v = _acc(kv_cache[1, pages, :, js % page_size, :])
        qi = _acc(q[i]).view(hkv, group, d)
        s = torch.einsum("hgd,nhd->hgn", qi, k) * scale
        p = torch.softmax(s, dim=-1)
        out[i] = torch.einsum("hgn,nhd->hgd", p, v).reshape(hq, d).to(q.dtype)
    return out.view(t, hq * d)


def _with_extra(tokens, extra):
    """``extra``: words that ride behind the tokens (the kernels' status words)."""
    return tokens if extra is None else torch.cat((tokens, extra.to(tokens.device, torch.int32)))


def argmax(logits, extra=None):
    return _with_extra(torch.argmax(logits, dim=-1).to(torch.int32), extra)


def sample(logits, temperature, topk, greedy, seed, stream_id, step, extra=None):
    out = []
    for r in range(logits.shape[0]):
        out.append(plain.sample(logits[r].detach().cpu().numpy(), greedy=bool(greedy[r]),
                                temperature=float(temperature[r]), topk=int(topk[r]),
                                seed=int(seed[r]), stream=int(stream_id[r]), step=int(step[r])))
    return _with_extra(torch.tensor(out, dtype=torch.int32, device=logits.device), extra)


def token_nll(logits, tokens):
    x = logits.double()
    return (torch.logsumexp(x, dim=-1) - x.gather(1, tokens.long()[:, None])[:, 0]).float()


def feed_tokens(token_ids, dst_rows, src_rows, src):
    for d, r in zip(dst_rows.tolist(), src_rows.tolist()):
        if d >= 0:
            token_ids[d] = src[r]


def launch_count():
    return 0


ALL = ["embedding", "rmsnorm", "add", "linear", "gated_linear", "qk_norm_rope_append",
       "paged_attention", "argmax", "sample", "token_nll", "launch_count", "feed_tokens"]
