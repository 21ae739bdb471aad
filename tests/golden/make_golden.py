"""Makes the golden logits of the reference project's own model code
(Jason-Young123/tinyInfer, tinyinfer/models/qwen3.py) for two tiny random Qwen3 models.

    python tests/golden/make_golden.py /path/to/tinyInfer
        -> tests/golden/ref_logits.npz, on the CPU. The reference's model calls three functions of its
        CUDA extension unconditionally (rmsnorm_forward, rope_forward, mlp_forward); here they are
        stand-ins that call the reference's own live Python layers where it has them
        (RotaryEmbedding._apply_rotary, tinyinfer/layers/rotary_embedding.py:77-102; SiluAndMul,
        tinyinfer/layers/activation.py:6-11) and, for the norm, the formula it keeps beside the call as
        "version1" (tinyinfer/layers/layernorm.py:16-21). Everything else (packed QKV, QK-norm
        placement, the paged cache, the causal offset, GQA mapping, tying) is the reference's code,
        run unchanged.

    python tests/golden/make_golden.py /path/to/installed/reference --gpu OUT.npz
        -> OUT.npz, on a GPU, in float32, with NO stand-in: the reference's built extension
        (tinyinfer._C: rmsnorm.cu, rope.cu, mlp.cu, flash_attention.cu, flash_decoding.cu) does the
        work, attention backend "flash". The committed copy is tests/golden/ref_logits_gpu.npz.

Both write, per model and request, the logits of the whole prompt in one step ("whole"), of the prompt
in two portions ("cut": the second reads the first back from the paged cache) and, on the GPU, of its
last tokens one by one ("decode": the FlashDecoding kernel). Weights come from numpy's RandomState, so
that tests can rebuild them bit for bit.
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
# A second model that differs in every size and ties its head to the embedding
# (tinyinfer/models/qwen3.py:271-272); the first has head_dim 16 where hidden / heads is 12.
GOLDEN_CONFIG_TIED = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    vocab_size=61, hidden_size=24, num_hidden_layers=3, num_attention_heads=3,
    num_key_value_heads=1, head_dim=8, intermediate_size=36, rms_norm_eps=1e-6,
    rope_theta=10000.0, attention_bias=False, tie_word_embeddings=True,
    max_position_embeddings=64)
GOLDEN_TOKENS_TIED = [[60, 0, 33, 33, 7, 21, 48, 5, 12], [9, 58, 30, 2, 44, 17, 6, 51, 23, 40, 1, 36, 19, 27, 3, 55, 11]]
GOLDEN_SEED_TIED = 4321
GOLDEN_MODELS = {"": (GOLDEN_CONFIG, GOLDEN_TOKENS, GOLDEN_SEED),
                 "tied_": (GOLDEN_CONFIG_TIED, GOLDEN_TOKENS_TIED, GOLDEN_SEED_TIED)}


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


def make_shim(rotary_module, activation_module):
    """Stand-ins for the three extension calls, made of the reference's own live Python layers."""
    apply_rotary = rotary_module.RotaryEmbedding._apply_rotary
    silu_and_mul = activation_module.SiluAndMul()

    class Shim:
        @staticmethod
        def rmsnorm_forward(input, weight, eps):
            # tinyinfer/layers/layernorm.py:16-21, the formula the reference keeps beside its kernel call
            x = input.float()
            var = x.pow(2).mean(dim=-1, keepdim=True)
            return weight * (x * torch.rsqrt(var + eps)).to(input.dtype)

        @staticmethod
        def rope_forward(q, k, positions, inv_freq):
            # angles as in tinyinfer/layers/rotary_embedding.py:125-128; the rotation is the reference's
            f = torch.outer(positions.float(), inv_freq.float())
            me = types.SimpleNamespace(rotary_dim=2 * inv_freq.numel())
            return apply_rotary(me, q, f.cos(), f.sin()), apply_rotary(me, k, f.cos(), f.sin())

        @staticmethod
        def mlp_forward(x, gate, up, down):
            # tinyinfer/models/qwen3.py:155-158 with the reference's SiluAndMul
            return silu_and_mul(torch.cat((x @ gate.T, x @ up.T), dim=-1)) @ down.T
    return Shim


def run_model(q3, PagedKVCache, set_context, reset_context, cfg, tokens_list, seed, device, backend, decode_tail):
    """Logits of the reference's Qwen3ForCausalLM for every request in the cuts described above."""
    page = 4
    ns = types.SimpleNamespace(**cfg, kvcache_block_size=page)
    model = q3.Qwen3ForCausalLM(ns, kv_cache=None, backend=backend).float().to(device).eval()
    w = golden_weights(cfg, seed)
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
    for r, tokens in enumerate(tokens_list):
        n = len(tokens)
        nblk = (n + page - 1) // page
        cache = PagedKVCache(cfg["num_hidden_layers"], nblk + 3, page,
                             cfg["num_key_value_heads"], cfg["head_dim"],
                             dtype=torch.float32, device=device)
        model.set_kv_cache(cache)
        table = torch.tensor([[nblk + 2 - b for b in range(nblk)]], dtype=torch.int32, device=device)  # scattered pages
        cuts = {"whole": [n], "cut": [n // 2, n - n // 2]}
        if decode_tail and n > 2:
            tail = min(decode_tail, n - 2)
            cuts["decode"] = [n - tail] + [1] * tail
        for tag, portions in cuts.items():
            rows = []
            start = 0
            for c in portions:
                pos = torch.arange(start, start + c, device=device)
                slots = torch.tensor([int(table[0, p // page]) * page + p % page for p in pos.tolist()], device=device)
                set_context(context_lens=[start + c], cu_seqlens_q=[0, c], slot_mapping=slots,
                            block_tables=table)
                with torch.no_grad():
                    h, _ = model(torch.tensor(tokens[start:start + c], device=device), pos)
                    rows.append(model.compute_logits(h).float().cpu())
                reset_context()
                start += c
            out[f"req{r}_{tag}"] = torch.cat(rows).numpy()
    return out


def main(ref_root, gpu_out=None):
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref_root)
    import tinyinfer.layers.activation as act
    import tinyinfer.layers.layernorm as ln
    import tinyinfer.layers.rotary_embedding as re_
    import tinyinfer.models.qwen3 as q3
    if gpu_out is None:
        shim = make_shim(re_, act)
        for m in (ln, re_, q3):
            m.load_extension = lambda: shim
    from tinyinfer.layers.attention import PagedKVCache
    from tinyinfer.utils.context import reset_context, set_context
    from tinyinfer.utils.loader import load_weights  # noqa: F401  (names checked below)

    out = {}
    for prefix, (cfg, tokens_list, seed) in GOLDEN_MODELS.items():
        got = run_model(q3, PagedKVCache, set_context, reset_context, dict(cfg), tokens_list, seed,
                        "cpu" if gpu_out is None else "cuda:0", "torch" if gpu_out is None else "flash",
                        decode_tail=0 if gpu_out is None else 6)
        out.update({prefix + k: v for k, v in got.items()})
    np.savez(gpu_out or __file__.replace("make_golden.py", "ref_logits.npz"), **out)
    for k, v in out.items():
        print(k, v.shape, float(np.abs(v).max()))


if __name__ == "__main__":
    if len(sys.argv) == 2:
        main(sys.argv[1])
    elif len(sys.argv) == 4 and sys.argv[2] == "--gpu":
        main(sys.argv[1], sys.argv[3])
    else:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/tinyInfer [--gpu OUT.npz]")
