"""Makes tests/golden/ref_logits.npz: logits of the reference project's own Python model code
(Jason-Young123/tinyInfer, tinyinfer/models/qwen3.py) for a tiny random Qwen3 on the CPU.

The reference's model calls three functions of its CUDA extension unconditionally
(rmsnorm_forward, rope_forward, mlp_forward). No GPU is needed here because they are
replaced by the PyTorch formulas that the reference keeps beside each call as its own
"version1" (tinyinfer/layers/layernorm.py:16-21, tinyinfer/layers/rotary_embedding.py:114-133,
tinyinfer/models/qwen3.py:155-158). Everything else (packed QKV, QK-norm placement, the paged
cache, the causal offset, GQA mapping, tying) is the reference's code, run unchanged.

Usage:  python tests/golden/make_golden.py /path/to/tinyInfer
Weights come from numpy's RandomState, so that tests can rebuild them bit for bit.
"""
import sys
import types

import numpy as np
import torch

GOLDEN_CONFIG = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    vocab_size=96, hidden_size=48, num_hidden_layers=2, num_attention_heads=4,
    num_key_value_heads=2, head_dim=16, intermediate_size=80, rms_norm_eps=1e-5,
    rope_theta=50000.0, attention_bias=False, tie_word_embeddings=False,
    max_position_embeddings=64)
GOLDEN_TOKENS = [[5, 17, 3, 90, 41, 41, 0, 7, 63, 12, 95, 28, 1], [88, 2, 19]]
GOLDEN_SEED = 1234


def golden_weights(cfg=GOLDEN_CONFIG, seed=GOLDEN_SEED):
    """name -> float32 tensor, checkpoint names of a Qwen3 folder, fixed draw order."""
    rs = np.random.RandomState(seed)
    h, v, i = cfg["hidden_size"], cfg["vocab_size"], cfg["intermediate_size"]
    d, hq, hkv = cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"]

    def mat(*shape):
        return torch.from_numpy((rs.standard_normal(shape) * 0.05).astype(np.float32))

    def vec(n):
        return torch.from_numpy((1.0 + 0.1 * rs.standard_normal(n)).astype(np.float32))

    w = {"model.embed_tokens.weight": mat(v, h)}
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        w[p + "input_layernorm.weight"] = vec(h)
        w[p + "self_attn.q_proj.weight"] = mat(hq * d, h)
        w[p + "self_attn.k_proj.weight"] = mat(hkv * d, h)
        w[p + "self_attn.v_proj.weight"] = mat(hkv * d, h)
        w[p + "self_attn.q_norm.weight"] = vec(d)
        w[p + "self_attn.k_norm.weight"] = vec(d)
        w[p + "self_attn.o_proj.weight"] = mat(h, hq * d)
        w[p + "post_attention_layernorm.weight"] = vec(h)
        w[p + "mlp.gate_proj.weight"] = mat(i, h)
        w[p + "mlp.up_proj.weight"] = mat(i, h)
        w[p + "mlp.down_proj.weight"] = mat(h, i)
    w["model.norm.weight"] = vec(h)
    if not cfg["tie_word_embeddings"]:
        w["lm_head.weight"] = mat(v, h)
    return w


class _Shim:
    """The reference's own commented PyTorch formulas, standing in for its CUDA extension."""

    @staticmethod
    def rmsnorm_forward(input, weight, eps):
        x = input.float()
        var = x.pow(2).mean(dim=-1, keepdim=True)
        return weight * (x * torch.rsqrt(var + eps)).to(input.dtype)

    @staticmethod
    def rope_forward(q, k, positions, inv_freq):
        f = torch.outer(positions.float(), inv_freq.float())
        cos, sin = f.cos()[:, None, :], f.sin()[:, None, :]

        def rot(x):
            half = x.shape[-1] // 2
            x1, x2 = x[..., :half], x[..., half:]
            return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)
        return rot(q), rot(k)

    @staticmethod
    def mlp_forward(x, gate, up, down):
        return (torch.nn.functional.silu(x @ gate.T) * (x @ up.T)) @ down.T


def main(ref_root):
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref_root)
    import tinyinfer.layers.layernorm as ln
    import tinyinfer.layers.rotary_embedding as re_
    import tinyinfer.models.qwen3 as q3
    for m in (ln, re_, q3):
        m.load_extension = lambda: _Shim
    from tinyinfer.layers.attention import PagedKVCache
    from tinyinfer.utils.context import reset_context, set_context
    from tinyinfer.utils.loader import load_weights  # noqa: F401  (names checked below)

    cfg = dict(GOLDEN_CONFIG)
    page = 4
    ns = types.SimpleNamespace(**cfg, kvcache_block_size=page)
    model = q3.Qwen3ForCausalLM(ns, kv_cache=None, backend="torch").float().eval()
    w = golden_weights()
    # the reference's packing: rows of qkv_proj ordered q, k, v (tinyinfer/utils/loader.py:52-96)
    params = dict(model.named_parameters())
    with torch.no_grad():
        for name, t in w.items():
            if "_proj.weight" in name and any(s in name for s in (".q_proj", ".k_proj", ".v_proj")):
                continue
            params[name].copy_(t)
        for l in range(cfg["num_hidden_layers"]):
            p = f"model.layers.{l}.self_attn."
            params[p + "qkv_proj.weight"].copy_(torch.cat(
                [w[p + "q_proj.weight"], w[p + "k_proj.weight"], w[p + "v_proj.weight"]], dim=0))

    out = {}
    for r, tokens in enumerate(GOLDEN_TOKENS):
        n = len(tokens)
        nblk = (n + page - 1) // page
        cache = PagedKVCache(cfg["num_hidden_layers"], nblk + 3, page,
                             cfg["num_key_value_heads"], cfg["head_dim"],
                             dtype=torch.float32, device="cpu")
        model.set_kv_cache(cache)
        table = torch.tensor([[nblk + 2 - b for b in range(nblk)]], dtype=torch.int32)  # scattered pages
        # whole prompt in one step, then the same prompt again in two portions (cache read-back)
        for tag, cuts in (("whole", [n]), ("cut", [n // 2, n - n // 2])):
            rows = []
            start = 0
            for c in cuts:
                pos = torch.arange(start, start + c)
                slots = torch.tensor([int(table[0, p // page]) * page + p % page for p in pos.tolist()])
                set_context(context_lens=[start + c], cu_seqlens_q=[0, c], slot_mapping=slots,
                            block_tables=table)
                with torch.no_grad():
                    h, _ = model(torch.tensor(tokens[start:start + c]), pos)
                    rows.append(model.compute_logits(h))
                reset_context()
                start += c
            out[f"req{r}_{tag}"] = torch.cat(rows).numpy()
    np.savez(__file__.replace("make_golden.py", "ref_logits.npz"), **out)
    for k, v in out.items():
        print(k, v.shape, float(np.abs(v).max()))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/tinyInfer")
    main(sys.argv[1])
