"""Plain, slow, whole-sequence Qwen3 dense model: the oracle of the test suite.

Every function below is written from the formulas of the reference project
(Jason-Young123/tinyInfer); the cited ``file:line`` are paths inside that project.
It runs on the CPU, takes a whole token sequence at once, keeps no cache, and shares
no code with ``tinyinfer_b200``: it parses ``config.json`` and reads
``model.safetensors`` by itself.

The sliding window has no counterpart in the reference (its attention is always
full causal, ``tinyinfer/layers/attention.py:236-265``); the rule used here is the
plain one: query ``i`` sees key ``j`` iff ``i - window < j <= i``.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import torch
from safetensors import safe_open


# --------------------------------------------------------------------------- folder
def read_model_folder(folder, dtype=torch.float64):
    """config.json as a dict and every tensor of the folder, upcast to ``dtype``."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    weights = {}
    for file in sorted(folder.glob("*.safetensors")):
        with safe_open(str(file), framework="pt", device="cpu") as f:
            for name in f.keys():
                weights[name] = f.get_tensor(name).to(dtype)
    return cfg, weights


def head_dim_of(cfg):
    # tinyinfer/models/qwen3.py:61 - head_dim falls back to hidden_size // heads
    return int(cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"])


def rope_theta_of(cfg):
    # tinyinfer/models/qwen3.py:39-48
    if "rope_theta" in cfg:
        return float(cfg["rope_theta"])
    scaling = cfg.get("rope_scaling")
    if scaling is not None:
        return float(scaling.get("rope_theta", 10000.0))
    return 10000.0


def layer_windows_of(cfg):
    """Per layer: the sliding window (int) or None. The rule follows the keys that a
    Qwen3 config.json carries: ``layer_types`` if present, else ``use_sliding_window``
    with ``max_window_layers`` (layers at or above that index slide)."""
    n = int(cfg["num_hidden_layers"])
    window = cfg.get("sliding_window")
    types = cfg.get("layer_types")
    if types is not None:
        return [int(window) if t == "sliding_attention" else None for t in types]
    if cfg.get("use_sliding_window") and window is not None:
        first = int(cfg.get("max_window_layers", n))
        return [int(window) if i >= first else None for i in range(n)]
    return [None] * n


# --------------------------------------------------------------------------- parts
def embedding(token_ids, table):
    # tinyinfer/models/qwen3.py:241 - a row lookup, no scaling
    return table[torch.as_tensor(token_ids, dtype=torch.long)]


def rmsnorm(x, weight, eps):
    # tinyinfer/csrc/rmsnorm.cu:22-50 - w * x * rsqrt(mean(x^2) + eps), mean over the last axis
    inv = torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return weight * x * inv


def rope(x, positions, theta, rotary_dim=None):
    """Half-split rotary embedding on x [T, heads, D].
    tinyinfer/layers/rotary_embedding.py:38-48 (inv_freq), :76-102 (rotation),
    tinyinfer/csrc/rope.cu:31-74 (angle = float32(position) * inv_freq)."""
    d = x.shape[-1]
    rot = d if rotary_dim is None else rotary_dim
    half = rot // 2
    # inv_freq and the angle are single precision in the reference
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    ang = torch.as_tensor(positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
    cos = ang.to(torch.float64).cos().to(x.dtype)[:, None, :]
    sin = ang.to(torch.float64).sin().to(x.dtype)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:rot]
    out = torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin, x[..., rot:]), dim=-1)
    return out


def attention(q, k, v, scale, window=None):
    """Causal grouped-query attention over one whole sequence.
    q [T, Hq, D], k and v [T, Hkv, D]; kv head of q head h is h // (Hq // Hkv)
    (tinyinfer/csrc/flash_decoding.cu:54-55); scores (q.k)*scale, keys j <= i kept
    (tinyinfer/layers/attention.py:236-265), softmax, weighted sum of v."""
    t, hq, d = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    kk = k.repeat_interleave(group, dim=1)
    vv = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, kk) * scale
    i = torch.arange(t)[:, None]
    j = torch.arange(t)[None, :]
    keep = j <= i
    if window is not None:
        keep = keep & (j > i - window)
    scores = scores.masked_fill(~keep[None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    return torch.einsum("hij,jhd->ihd", p, vv)


def swiglu(x, w_gate, w_up, w_down):
    # tinyinfer/csrc/mlp.cu:116-141 (silu(x.gate) * (x.up)), :246-266 (down);
    # silu(g) = g / (1 + exp(-g)), tinyinfer/csrc/utils.h:76-78
    g = x @ w_gate.T
    u = x @ w_up.T
    return ((g / (1.0 + torch.exp(-g))) * u) @ w_down.T


def attention_block(x, positions, w, prefix, cfg, window):
    """qkv projection, per-head QK RMSNorm, RoPE, attention, output projection.
    tinyinfer/models/qwen3.py:106-132."""
    hq = int(cfg["num_attention_heads"])
    hkv = int(cfg["num_key_value_heads"])
    d = head_dim_of(cfg)
    eps = float(cfg["rms_norm_eps"])
    t = x.shape[0]
    q = x @ w[prefix + "q_proj.weight"].T
    k = x @ w[prefix + "k_proj.weight"].T
    v = x @ w[prefix + "v_proj.weight"].T
    if cfg.get("attention_bias", False):
        q = q + w[prefix + "q_proj.bias"]
        k = k + w[prefix + "k_proj.bias"]
        v = v + w[prefix + "v_proj.bias"]
    q = q.view(t, hq, d)
    k = k.view(t, hkv, d)
    v = v.view(t, hkv, d)
    q = rmsnorm(q, w[prefix + "q_norm.weight"], eps)          # qwen3.py:116-117
    k = rmsnorm(k, w[prefix + "k_norm.weight"], eps)
    theta = rope_theta_of(cfg)
    q = rope(q, positions, theta)                              # qwen3.py:122
    k = rope(k, positions, theta)
    o = attention(q, k, v, d ** -0.5, window)                  # qwen3.py:87
    o = o.reshape(t, hq * d) @ w[prefix + "o_proj.weight"].T   # qwen3.py:132
    if cfg.get("attention_bias", False):
        o = o + w[prefix + "o_proj.bias"]
    return o


def decoder_layer(x, positions, w, i, cfg, window):
    # tinyinfer/models/qwen3.py:192-221 - pre-norm, two residual sums
    eps = float(cfg["rms_norm_eps"])
    p = f"model.layers.{i}."
    h = rmsnorm(x, w[p + "input_layernorm.weight"], eps)
    x = x + attention_block(h, positions, w, p + "self_attn.", cfg, window)
    h = rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
    x = x + swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                   w[p + "mlp.down_proj.weight"])
    return x


def forward(cfg, w, token_ids):
    """Logits [T, V] at every position of one whole sequence.
    tinyinfer/models/qwen3.py:239-248 (backbone), :283-288 (lm_head), :271-272 (tying)."""
    positions = list(range(len(token_ids)))
    x = embedding(token_ids, w["model.embed_tokens.weight"])
    windows = layer_windows_of(cfg)
    for i in range(int(cfg["num_hidden_layers"])):
        x = decoder_layer(x, positions, w, i, cfg, windows[i])
    x = rmsnorm(x, w["model.norm.weight"], float(cfg["rms_norm_eps"]))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) \
        else w["lm_head.weight"]
    return x @ head.T


# --------------------------------------------------------------------------- sampling
_PHILOX_M0, _PHILOX_M1 = 0xD2511F53, 0xCD9E8D57
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85


def philox4x32(counter, key, rounds=10):
    """Philox-4x32-10 on python ints (Salmon et al. 2011); counter 4 words, key 2 words."""
    c = list(counter)
    k = list(key)
    for _ in range(rounds):
        p0 = _PHILOX_M0 * c[0]
        p1 = _PHILOX_M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & 0xFFFFFFFF, p1 & 0xFFFFFFFF,
             ((p0 >> 32) ^ c[3] ^ k[1]) & 0xFFFFFFFF, p0 & 0xFFFFFFFF]
        k = [(k[0] + _PHILOX_W0) & 0xFFFFFFFF, (k[1] + _PHILOX_W1) & 0xFFFFFFFF]
    return c


def uniform_for(seed, stream, step, index):
    """The uniform in (0, 1) that token ``index`` of a row draws: word ``index % 4`` of the
    Philox block with counter (index // 4, step, stream, 0) and key (seed lo, seed hi)."""
    words = philox4x32([index // 4, step & 0xFFFFFFFF, stream & 0xFFFFFFFF, 0],
                       [seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF])
    return np.float32((words[index % 4] >> 9) + 0.5) * np.float32(1.0 / (1 << 23))


def sample(logits_row, *, greedy, temperature=1.0, topk=0, seed=0, stream=0, step=0):
    """One token from one row of logits.
    Greedy: argmax, first index wins ties (tinyinfer/layers/sampler.py:42-43).
    Else: scaled = logits / T in float32; values below the k-th largest become -inf, ties at
    the threshold stay (sampler.py:59-63); token = argmax(scaled + G), G = -log(-log(U))
    (sampler.py:69-72). U comes from ``uniform_for`` instead of the global generator."""
    row = np.asarray(logits_row, dtype=np.float32)
    if greedy:
        return int(np.argmax(row))
    scaled = (row / np.float32(temperature)).astype(np.float32)
    if topk and topk < row.shape[0]:
        kth = np.sort(scaled)[::-1][topk - 1]
        scaled = np.where(scaled < kth, -np.inf, scaled).astype(np.float32)
    best, best_v = -1, -math.inf
    for i in range(row.shape[0]):
        if scaled[i] == -np.inf:
            continue
        u = uniform_for(seed, stream, step, i)
        g = -np.log(-np.log(u, dtype=np.float32), dtype=np.float32)
        val = float(np.float32(scaled[i] + g))
        if val > best_v:
            best, best_v = i, val
    return best


def greedy_generate(cfg, w, prompt, num_new):
    """Greedy continuation by re-running the whole sequence for every new token."""
    ids = list(prompt)
    for _ in range(num_new):
        logits = forward(cfg, w, ids)
        ids.append(int(torch.argmax(logits[-1].float()).item()))
    return ids[len(prompt):]
