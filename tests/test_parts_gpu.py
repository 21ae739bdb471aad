"""Each part of a block alone, built from its spec and fed by hand, against the plain function of
the same part: norm, rotary frequencies, attention mixer (with a window and with bias), gated
feed-forward, and their arrangement in a block."""
import pytest
import torch

import plain_qwen3 as plain
from tinyinfer_b200.config import AttentionSpec, GatedMLPSpec, LayerSpec, NormSpec, PositionSpec
from tinyinfer_b200.engine.batch import BatchBuffers, CacheView, StepEntry
from tinyinfer_b200.parts import build_block, build_feed_forward, build_mixer, build_norm, build_position

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float64) * std


def load_part(part, tensors64, dtype):
    given = {}
    for name, ts in part.tensors().items():
        t = tensors64[name]
        assert tuple(t.shape) == tuple(ts.shape)
        given[name] = t.to(dtype if ts.role == "matrix" else torch.float32).to(DEV)
    part.load(given)


def whole_step(n, hkv, d, page=8, dtype=torch.float32):
    """A StepContext for one request of n tokens run whole, with a fresh cache entry."""
    pages = (n + page - 1) // page + 2
    buffers = BatchBuffers(DEV, n, 1, pages, 1)
    table = list(reversed(range(pages)))[: (n + page - 1) // page]
    ctx = buffers.build([StepEntry("r", list(range(n)), [])], [0], [0], [[table]])
    kv = torch.full((2, pages, hkv, page, d), float("nan"), dtype=dtype, device=DEV)
    ctx.views[0] = CacheView(kv, ctx.block_tables[0], page, True, None)
    return ctx, ctx.views[0]


def test_norm_and_rotary_parts():
    spec = NormSpec(100, 1e-5)
    part = build_norm(spec, torch.float32, DEV)
    w = 1 + 0.1 * rnd(100, seed=1)
    load_part(part, {"weight": w}, torch.float32)
    x = rnd(9, 100, std=3.0)
    got = part.forward(x.float().to(DEV)).cpu().double()
    assert torch.allclose(got, plain.rmsnorm(x, w, 1e-5), atol=1e-5)
    rows = torch.tensor([8, 0], dtype=torch.int32, device=DEV)
    got = part.forward_rows(x.float().to(DEV), rows).cpu().double()
    assert torch.allclose(got, plain.rmsnorm(x[[8, 0]], w, 1e-5), atol=1e-5)
    pos = build_position(PositionSpec("rope", 1e6, 48), torch.bfloat16, DEV)
    want = 1.0 / (1e6 ** (torch.arange(0, 48, 2, dtype=torch.float32) / 48))
    assert pos.inv_freq.dtype == torch.float32 and torch.equal(pos.inv_freq.cpu(), want)
    assert build_position(PositionSpec("none"), torch.float32, DEV).inv_freq is None


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("hq,hkv,d,window,bias", [(4, 2, 16, None, False), (6, 2, 32, 7, True), (4, 1, 128, 30, False)])
def test_attention_part(dtype, tol, hq, hkv, d, window, bias):
    h, n, eps, theta = 72, 45, 1e-5, 50000.0
    spec = AttentionSpec(h, hq, hkv, d, d ** -0.5, PositionSpec("rope", theta, d), qk_norm=NormSpec(d, eps),
                         bias=bias, window=window)
    part = build_mixer(spec, dtype, DEV)
    assert part.cache_need().window == window and part.state_need() is None
    w = {"q_proj.weight": rnd(hq * d, h, seed=1, std=0.1), "k_proj.weight": rnd(hkv * d, h, seed=2, std=0.1),
         "v_proj.weight": rnd(hkv * d, h, seed=3, std=0.1), "o_proj.weight": rnd(h, hq * d, seed=4, std=0.1),
         "q_norm.weight": 1 + 0.1 * rnd(d, seed=5), "k_norm.weight": 1 + 0.1 * rnd(d, seed=6),
         "q_proj.bias": rnd(hq * d, seed=7, std=0.1), "k_proj.bias": rnd(hkv * d, seed=8, std=0.1),
         "v_proj.bias": rnd(hkv * d, seed=9, std=0.1), "o_proj.bias": rnd(h, seed=10, std=0.1)}
    if dtype == torch.bfloat16:      # both sides see the same rounded matrices
        w = {k: (v.to(dtype).double() if k.endswith("proj.weight") else v) for k, v in w.items()}
    load_part(part, w, dtype)
    x = rnd(n, h, seed=11)
    if dtype == torch.bfloat16:
        x = x.to(dtype).double()
    ctx, view = whole_step(n, hkv, d, dtype=dtype)
    got = part.forward(x.to(dtype).to(DEV), ctx, view).cpu().double()
    cfg = dict(num_attention_heads=hq, num_key_value_heads=hkv, head_dim=d, rms_norm_eps=eps, rope_theta=theta,
               attention_bias=bias)
    want = plain.attention_block(x, list(range(n)), w, "", cfg, window)
    assert (got - want).abs().max() <= tol * want.abs().max()
    res = rnd(n, h, seed=12)
    if dtype == torch.bfloat16:
        res = res.to(dtype).double()
    ctx, view = whole_step(n, hkv, d, dtype=dtype)
    got = part.forward_residual(x.to(dtype).to(DEV), res.to(dtype).to(DEV), ctx, view).cpu().double()
    assert (got - (want + res)).abs().max() <= tol * (want + res).abs().max()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
def test_feed_forward_part_and_block(dtype, tol):
    h, inter, n, eps = 72, 200, 33, 1e-6
    ffn_spec = GatedMLPSpec(h, inter)
    w = {"gate_proj.weight": rnd(inter, h, seed=1, std=0.1), "up_proj.weight": rnd(inter, h, seed=2, std=0.1),
         "down_proj.weight": rnd(h, inter, seed=3, std=0.1)}
    if dtype == torch.bfloat16:
        w = {k: v.to(dtype).double() for k, v in w.items()}
    part = build_feed_forward(ffn_spec, dtype, DEV)
    load_part(part, w, dtype)
    x = rnd(n, h, seed=4).to(dtype).double()
    got = part.forward(x.to(dtype).to(DEV)).cpu().double()
    want = plain.swiglu(x, w["gate_proj.weight"], w["up_proj.weight"], w["down_proj.weight"])
    assert (got - want).abs().max() <= tol * want.abs().max()

    hq, hkv, d, theta = 4, 2, 16, 10000.0
    attn_spec = AttentionSpec(h, hq, hkv, d, d ** -0.5, PositionSpec("rope", theta, d), qk_norm=NormSpec(d, eps))
    block = build_block(LayerSpec(attn_spec, ffn_spec, NormSpec(h, eps), NormSpec(h, eps)), dtype, DEV)
    pw = {"model.layers.0.self_attn.q_proj.weight": rnd(hq * d, h, seed=5, std=0.1),
          "model.layers.0.self_attn.k_proj.weight": rnd(hkv * d, h, seed=6, std=0.1),
          "model.layers.0.self_attn.v_proj.weight": rnd(hkv * d, h, seed=7, std=0.1),
          "model.layers.0.self_attn.o_proj.weight": rnd(h, hq * d, seed=8, std=0.1),
          "model.layers.0.self_attn.q_norm.weight": 1 + 0.1 * rnd(d, seed=9),
          "model.layers.0.self_attn.k_norm.weight": 1 + 0.1 * rnd(d, seed=10),
          "model.layers.0.input_layernorm.weight": 1 + 0.1 * rnd(h, seed=11),
          "model.layers.0.post_attention_layernorm.weight": 1 + 0.1 * rnd(h, seed=12)}
    pw.update({"model.layers.0.mlp." + k: v for k, v in w.items()})
    if dtype == torch.bfloat16:
        pw = {k: (v.to(dtype).double() if "proj" in k else v) for k, v in pw.items()}
    for prefix, p in (("self_attn.", block.mixer), ("mlp.", block.feed_forward),
                      ("input_layernorm.", block.mixer_norm), ("post_attention_layernorm.", block.feed_forward_norm)):
        load_part(p, {k[len("model.layers.0." + prefix):]: v for k, v in pw.items()
                      if k.startswith("model.layers.0." + prefix)}, dtype)
    ctx, view = whole_step(n, hkv, d, dtype=dtype)
    got = block.forward(x.to(dtype).to(DEV), ctx, view).cpu().double()
    cfg = dict(num_attention_heads=hq, num_key_value_heads=hkv, head_dim=d, rms_norm_eps=eps, rope_theta=theta)
    want = plain.decoder_layer(x, list(range(n)), pw, 0, cfg, None)
    assert (got - want).abs().max() <= tol * want.abs().max()
