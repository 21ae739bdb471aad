"""Each CUDA kernel alone beside its plain PyTorch statement (tests/torch_ops.py), at sizes other
than the engine's: odd widths, head sizes in steps of 16, every page size, windows, groups."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import torch_ops as ref

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def dev():
    return torch.device("cuda:0")


def tol(dtype):
    return dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def close(a, b, dtype, scale=1.0):
    t = tol(dtype)
    torch.testing.assert_close(a.double(), b.double(), rtol=t["rtol"], atol=t["atol"] * scale)


def rnd(*shape, dtype, seed=0, std=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype).to(dev())


@pytest.fixture(scope="module")
def ops():
    from tinyinfer_b200 import ops
    return ops


def test_extension_is_loaded_and_cpu_is_refused(ops):
    from tinyinfer_b200.ops import library
    x = torch.ones(4, 8)
    with pytest.raises(ops.KernelError):
        ops.rmsnorm(x, torch.ones(8), 1e-6)
    ops.add(rnd(3, dtype=torch.float32), rnd(3, dtype=torch.float32))
    assert "core" in library.loaded_libraries() and ops.launch_count() > 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("t,h,v", [(1, 64, 256), (7, 100, 389), (33, 4096, 1000), (5, 5120, 77)])
def test_embedding(ops, dtype, t, h, v):
    table = rnd(v, h, dtype=dtype)
    ids = torch.randint(0, v, (t,), dtype=torch.int32, device=dev())
    assert torch.equal(ops.embedding(ids, table), ref.embedding(ids, table))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,size,eps", [(1, 16, 1e-6), (9, 96, 1e-5), (5, 100, 1e-6), (3, 4096, 1e-6),
                                           (2, 5120, 1e-5), (300, 128, 1e-6)])
def test_rmsnorm(ops, dtype, rows, size, eps):
    x = rnd(rows, size, dtype=dtype, std=3.0)
    w = 1.0 + 0.1 * rnd(size, dtype=torch.float32, seed=1)
    close(ops.rmsnorm(x, w, eps), ref.rmsnorm(x, w, eps), dtype)
    pick = torch.tensor([rows - 1, 0, rows // 2], dtype=torch.int32, device=dev())
    close(ops.rmsnorm(x, w, eps, rows=pick), ref.rmsnorm(x, w, eps, rows=pick), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_add(ops, dtype):
    a, b = rnd(37, 100, dtype=dtype), rnd(37, 100, dtype=dtype, seed=1)
    assert torch.equal(ops.add(a, b), ref.add(a, b))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (5, 100, 96), (64, 64, 16), (65, 130, 50), (130, 389, 320),
                                   (2, 1000, 4096), (300, 96, 176)])
def test_linear(ops, dtype, m, n, k):
    x, w = rnd(m, k, dtype=dtype), rnd(n, k, dtype=dtype, seed=1, std=k ** -0.5)
    bias = rnd(n, dtype=torch.float32, seed=2)
    res = rnd(m, n, dtype=dtype, seed=3)
    close(ops.linear(x, w), ref.linear(x, w), dtype)
    close(ops.linear(x, w, bias=bias, residual=res), ref.linear(x, w, bias=bias, residual=res), dtype)
    out32 = ops.linear(x, w, out_float32=True)
    assert out32.dtype == torch.float32
    close(out32, ref.linear(x, w, out_float32=True), torch.float32, scale=10.0 if dtype == torch.bfloat16 else 1.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,inter,k", [(1, 128, 64), (7, 176, 96), (70, 448, 320), (33, 100, 50)])
def test_gated_linear(ops, dtype, m, inter, k):
    x, w = rnd(m, k, dtype=dtype), rnd(2 * inter, k, dtype=dtype, seed=1, std=k ** -0.5)
    close(ops.gated_linear(x, w), ref.gated_linear(x, w), dtype)


def linear_rows_do_not_depend_on_the_batch(ops, dtype):
    x, w = rnd(130, 96, dtype=dtype), rnd(100, 96, dtype=dtype, seed=1)
    whole = ops.linear(x, w)
    assert torch.equal(whole[77:78], ops.linear(x[77:80].contiguous(), w)[:1])
    assert torch.equal(whole[:70], ops.linear(x[:70].contiguous(), w))
    # one row alone takes the small-batch kernel: the same sum, at most another rounding
    close(whole[77:78], ops.linear(x[77:78].contiguous(), w), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_rows_do_not_depend_on_the_batch(ops, dtype):
    linear_rows_do_not_depend_on_the_batch(ops, dtype)


# the tensor-core path: tiles that wrap the pipeline, many tiles per CTA, every small-batch width
TC_SHAPES = [(1, 4096, 4096), (8, 6144, 4096), (16, 1000, 512), (17, 520, 264), (33, 4096, 1024), (64, 389, 320),
             (65, 256, 128), (128, 128, 64), (200, 1000, 4096), (2048, 4096, 512), (777, 1032, 1096), (3, 40, 8),
             # 65..128 tokens with the weights on the accumulator lanes and a cut k loop; 256 x 256 tiles
             # with ragged edges in every direction
             (100, 4096, 4096), (128, 1000, 2048), (1500, 5000, 136), (3100, 2600, 72),
             # 16 tokens and more: the units of a cut k loop add up together (9 and 12 cuts)
             (16, 4096, 4096), (48, 2048, 12288), (64, 4096, 4096),
             # 149 to 295 tiles of 128 outputs: more than half the CTA slots, fewer than all
             (8, 25600, 1024), (40, 30000, 520), (1, 19200, 4096)]


@pytest.fixture
def one_cta_form(ops):
    """The products of many tokens stay with the one-CTA kernel (the library would hand some to the pair form)."""
    ops.set_pair_form(False)
    yield
    ops.set_pair_form(True)


@pytest.mark.parametrize("m,n,k", TC_SHAPES)
def test_linear_tensor_cores(ops, one_cta_form, m, n, k):
    dtype = torch.bfloat16
    x, w = rnd(m, k, dtype=dtype), rnd(n, k, dtype=dtype, seed=1, std=k ** -0.5)
    bias = rnd(n, dtype=torch.float32, seed=2)
    res = rnd(m, n, dtype=dtype, seed=3)
    close(ops.linear(x, w), ref.linear(x, w), dtype)
    close(ops.linear(x, w, bias=bias, residual=res), ref.linear(x, w, bias=bias, residual=res), dtype)
    close(ops.linear(x, w, out_float32=True), ref.linear(x, w, out_float32=True), torch.float32, scale=100.0)
    ops.check_kernel_status()


# the pair form (two CTAs a 256 x 256 tile): one tile, many tiles per cluster, ragged edges in every direction,
# k loops shorter and longer than the ring of stages, fewer tiles than clusters
PAIR_SHAPES = [(256, 256, 64), (2048, 4096, 512), (777, 1032, 1096), (1500, 5000, 136), (3100, 2600, 72), (130, 300, 4096),
               (4096, 6144, 4096), (1, 256, 128), (513, 12288, 256)]


@pytest.mark.parametrize("m,n,k", PAIR_SHAPES)
def test_linear_pair_form(ops, monkeypatch, m, n, k):
    monkeypatch.setattr(ops, "PAIR_MIN_TOKENS", 1)
    dtype = torch.bfloat16
    x, w = rnd(m, k, dtype=dtype), rnd(n, k, dtype=dtype, seed=1, std=k ** -0.5)
    bias = rnd(n, dtype=torch.float32, seed=2)
    res = rnd(m, n, dtype=dtype, seed=3)
    close(ops.linear(x, w), ref.linear(x, w), dtype)
    close(ops.linear(x, w, bias=bias, residual=res), ref.linear(x, w, bias=bias, residual=res), dtype)
    close(ops.linear(x, w, out_float32=True), ref.linear(x, w, out_float32=True), torch.float32, scale=100.0)
    ops.check_kernel_status()


def test_products_of_many_tokens_choose_their_form(ops):
    """Left alone, the library sends a product of 2,048 tokens to the pair form and one of 300 to the one-CTA
    form; both give what the plain product gives."""
    dtype = torch.bfloat16
    for m in (2048, 300):
        x, w = rnd(m, 512, dtype=dtype), rnd(4096, 512, dtype=dtype, seed=1, std=512 ** -0.5)
        res = rnd(m, 4096, dtype=dtype, seed=3)
        close(ops.linear(x, w, residual=res), ref.linear(x, w, residual=res), dtype)
        wg = rnd(2 * 1536, 512, dtype=dtype, seed=4, std=512 ** -0.5)
        close(ops.gated_linear(x, wg), ref.gated_linear(x, wg), dtype)
    ops.check_kernel_status()


@pytest.mark.parametrize("m,inter,k", [(256, 128, 64), (300, 448, 320), (2048, 1024, 256), (130, 136, 40), (1500, 2500, 136),
                                       (3100, 1300, 72), (2048, 12288, 512)])
def test_gated_linear_pair_form(ops, monkeypatch, m, inter, k):
    monkeypatch.setattr(ops, "PAIR_MIN_TOKENS", 1)
    dtype = torch.bfloat16
    x, w = rnd(m, k, dtype=dtype), rnd(2 * inter, k, dtype=dtype, seed=1, std=k ** -0.5)
    close(ops.gated_linear(x, w), ref.gated_linear(x, w), dtype)
    ops.check_kernel_status()


@pytest.mark.parametrize("m,k0,h,inter,eps", [(1, 512, 1024, 768, 1e-6), (8, 4096, 4096, 1536, 1e-6),
                                            (33, 1024, 520, 200, 1e-5), (64, 1024, 2048, 1000, 1e-6)])
def test_rmsnorm_shared_between_two_products(ops, m, k0, h, inter, eps):
    """For few tokens the product that makes a residual stream x also leaves x * g and the sums of squares
    of x's rows; the products behind the norm read x * g and scale their rows by 1 / rms: the same
    results as product, norm kernel, product."""
    dtype = torch.bfloat16
    a, w0 = rnd(m, k0, dtype=dtype), rnd(h, k0, dtype=dtype, seed=1, std=k0 ** -0.5)
    res = rnd(m, h, dtype=dtype, seed=2)
    g = (1 + 0.1 * rnd(h, dtype=torch.float32, seed=3)).contiguous()
    x, link = ops.linear(a, w0, residual=res, next_norm_weight=g)
    close(x, ref.linear(a, w0, residual=res), dtype)
    assert link is not None, "this shape was expected to cut its k loop and leave a link"
    torch.testing.assert_close(link.sums[:link.parts].sum(dim=0), (x.float() ** 2).sum(dim=1), rtol=1e-4, atol=1e-4)
    close(link.scaled, (x.float() * g).to(dtype), dtype)
    # the plain statement with the norm's result NOT rounded to bfloat16 in between: the shared norm rounds
    # x * g where the norm kernel rounds x * g / rms, so either differs from this by one rounding of the input
    normed = ref.rmsnorm(x.float(), g, eps)
    w1 = rnd(inter, h, dtype=dtype, seed=4, std=h ** -0.5)
    bias = rnd(inter, dtype=torch.float32, seed=5)
    close(ops.linear(link.scaled, w1, bias=bias, link=link, link_eps=eps),
          ref.linear(normed, w1.float(), bias=bias).to(dtype), dtype)
    res2 = rnd(m, inter, dtype=dtype, seed=7)
    close(ops.linear(link.scaled, w1, residual=res2, link=link, link_eps=eps),
          ref.linear(normed, w1.float(), residual=res2.float()).to(dtype), dtype)
    w2 = rnd(2 * inter, h, dtype=dtype, seed=6, std=h ** -0.5)
    close(ops.gated_linear(link.scaled, w2, link=link, link_eps=eps), ref.gated_linear(normed, w2.float()).to(dtype), dtype)
    # more tokens than a link takes: no link, the plain product
    big, none = ops.linear(rnd(65, k0, dtype=dtype), w0, next_norm_weight=g)
    assert none is None and big.shape == (65, h)
    ops.check_kernel_status()


@pytest.mark.parametrize("m,inter,k", [(1, 12288, 4096), (8, 1000, 512), (20, 448, 320), (64, 100, 96), (65, 176, 96),
                                       # few tiles and a long k: the k loops are cut, from 16 tokens on the units add up together
                                       (32, 6144, 2048), (64, 1000, 1024), (17, 3000, 768), (8, 6144, 2048), (16, 1028, 4096),
                                       # more tiles (of 64 outputs) than half the CTA slots and fewer than all: not cut
                                       (8, 12288, 4096), (1, 12288, 1024), (64, 12288, 512), (33, 9700, 2056), (16, 18000, 640),
                                       (300, 448, 320), (2048, 1024, 256), (130, 72, 40), (1500, 2500, 136), (3100, 1300, 72)])
def test_gated_linear_tensor_cores(ops, one_cta_form, m, inter, k):
    dtype = torch.bfloat16
    x, w = rnd(m, k, dtype=dtype), rnd(2 * inter, k, dtype=dtype, seed=1, std=k ** -0.5)
    close(ops.gated_linear(x, w), ref.gated_linear(x, w), dtype)
    ops.check_kernel_status()


def paged_setup(dtype, lens, hq, hkv, d, page, seed=0, extra_pages=3):
    """Random q/k/v for requests of the given lengths, laid into scattered pages."""
    g = torch.Generator().manual_seed(seed)
    total_pages = sum((n + page - 1) // page for n in lens) + extra_pages
    perm = torch.randperm(total_pages, generator=g).tolist()
    tables, nxt = [], 0
    for n in lens:
        nb = (n + page - 1) // page
        tables.append(perm[nxt:nxt + nb])
        nxt += nb
    width = max(len(t) for t in tables)
    bt = torch.tensor([t + [-1] * (width - len(t)) for t in tables], dtype=torch.int32, device=dev())
    kv = torch.full((2, total_pages, hkv, page, d), float("nan"), dtype=dtype, device=dev())
    return bt, kv


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page,rot,norm", [
    (4, 2, 16, 4, 16, True), (6, 2, 32, 8, 32, True), (8, 2, 64, 16, 64, True), (4, 1, 128, 64, 128, True),
    (3, 3, 48, 5, 24, False), (2, 1, 256, 32, 256, True), (5, 5, 80, 16, 0, True)])
def test_qk_norm_rope_append(ops, dtype, hq, hkv, d, page, rot, norm):
    lens = [9, 1, 23]
    starts = [3, 0, 40]                       # tokens already held: this step appends lens[i] more
    bt, kv = paged_setup(dtype, [s + n for s, n in zip(starts, lens)], hq, hkv, d, page)
    t = sum(lens)
    qkv = rnd(t, (hq + 2 * hkv) * d, dtype=dtype, std=2.0)
    pos = torch.tensor([p for s, n in zip(starts, lens) for p in range(s, s + n)], dtype=torch.int32, device=dev())
    seq = torch.tensor([i for i, n in enumerate(lens) for _ in range(n)], dtype=torch.int32, device=dev())
    qw = (1 + 0.1 * rnd(d, dtype=torch.float32, seed=5)) if norm else None
    kw = (1 + 0.1 * rnd(d, dtype=torch.float32, seed=6)) if norm else None
    inv = None
    if rot:
        inv = (1.0 / (1e6 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(dev())
    kv_ref = kv.clone()
    args = dict(num_heads=hq, num_kv_heads=hkv, head_dim=d, q_norm_weight=qw, k_norm_weight=kw, eps=1e-6,
                inv_freq=inv, rotary_dim=rot, positions=pos, token_seq=seq, block_table=bt)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    q = ops.qk_norm_rope_append(qkv, kv_cache=kv, status=status, **args)
    q_ref = ref.qk_norm_rope_append(qkv, kv_cache=kv_ref, **args)
    assert int(status.item()) == 0
    close(q, q_ref, dtype, scale=4.0)
    written = ~torch.isnan(kv_ref.float())
    assert torch.equal(written, ~torch.isnan(kv.float())), "wrote to other slots than the reference"
    close(kv[written], kv_ref[written], dtype, scale=4.0)
    # an entry that only reads the cache gets q and leaves the pages alone
    kv2 = kv.clone()
    q2 = ops.qk_norm_rope_append(qkv, kv_cache=None, **args)
    assert torch.equal(q2, q) and torch.equal(torch.nan_to_num(kv2.float()), torch.nan_to_num(kv.float()))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page,rot", [(4, 2, 16, 4, 16), (3, 1, 64, 16, 64), (4, 1, 128, 64, 128),
                                                (3, 3, 48, 5, 24), (2, 2, 80, 16, 40)])
@pytest.mark.parametrize("interleaved,table", [(True, False), (False, True), (True, True)])
def test_rotation_by_table_and_in_interleaved_pairs(ops, dtype, hq, hkv, d, page, rot, interleaved, table):
    """The other forms of the rotation: pairs (2j, 2j + 1) instead of (j, j + rot / 2), and angles from a
    table of cosines and sines per position instead of position * inv_freq (here: angles that no
    inv_freq gives, a square-root law)."""
    lens, starts = [9, 1, 23], [3, 0, 40]
    bt, kv = paged_setup(dtype, [s + n for s, n in zip(starts, lens)], hq, hkv, d, page)
    t = sum(lens)
    qkv = rnd(t, (hq + 2 * hkv) * d, dtype=dtype, std=2.0)
    pos = torch.tensor([p for s, n in zip(starts, lens) for p in range(s, s + n)], dtype=torch.int32, device=dev())
    seq = torch.tensor([i for i, n in enumerate(lens) for _ in range(n)], dtype=torch.int32, device=dev())
    qw = 1 + 0.1 * rnd(d, dtype=torch.float32, seed=5)
    kw = 1 + 0.1 * rnd(d, dtype=torch.float32, seed=6)
    inv = (1.0 / (1e4 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(dev())
    if table:
        ang = torch.sqrt(torch.arange(70, dtype=torch.float32, device=dev()))[:, None] * inv[None, :] * 3.0
        rotation = ops.Rotation(rot, cos_sin=torch.cat((ang.cos(), ang.sin()), dim=1).contiguous(), interleaved=interleaved)
    else:
        rotation = ops.Rotation(rot, inv_freq=inv, interleaved=interleaved)
    args = dict(num_heads=hq, num_kv_heads=hkv, head_dim=d, q_norm_weight=qw, k_norm_weight=kw, eps=1e-6,
                rotation=rotation, positions=pos, token_seq=seq, block_table=bt)
    kv_ref = kv.clone()
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    q = ops.qk_norm_rope_append(qkv, kv_cache=kv, status=status, **args)
    q_ref = ref.qk_norm_rope_append(qkv, kv_cache=kv_ref, **args)
    assert int(status.item()) == 0
    close(q, q_ref, dtype, scale=4.0)
    written = ~torch.isnan(kv_ref.float())
    assert torch.equal(written, ~torch.isnan(kv.float()))
    close(kv[written], kv_ref[written], dtype, scale=4.0)
    if table:                                   # a position the table does not reach: said, and nothing written
        short = ops.Rotation(rot, cos_sin=rotation.cos_sin[:50].contiguous(), interleaved=interleaved)
        kv3 = torch.full_like(kv, float("nan"))
        ops.qk_norm_rope_append(qkv, kv_cache=kv3, status=status, **dict(args, rotation=short))
        assert int(status.item()) == 4
        beyond = (pos >= 50).nonzero().flatten().tolist()
        for row in beyond:
            pg = int(bt[int(seq[row]), int(pos[row]) // page])
            assert torch.isnan(kv3[0, pg, :, int(pos[row]) % page].float()).all()


def test_a_position_beyond_the_block_table_is_a_token_without_a_page(ops):
    """A table narrower than a token's position needs: the kernels say so through the status word and
    neither read the next request's row nor write into its pages."""
    hq, hkv, d, page = 4, 2, 64, 16
    for dtype in DTYPES:
        bt = torch.tensor([[0], [1]], dtype=torch.int32, device=dev())          # one page each
        kv = torch.full((2, 3, hkv, page, d), float("nan"), dtype=dtype, device=dev())
        qkv = rnd(2, (hq + 2 * hkv) * d, dtype=dtype)
        pos = torch.tensor([16, 3], dtype=torch.int32, device=dev())            # request 0 would need a second page
        seq = torch.tensor([0, 1], dtype=torch.int32, device=dev())
        status = torch.zeros(1, dtype=torch.int32, device=dev())
        ops.qk_norm_rope_append(qkv, num_heads=hq, num_kv_heads=hkv, head_dim=d, q_norm_weight=None,
                                k_norm_weight=None, eps=1e-6, positions=pos, token_seq=seq, kv_cache=kv,
                                block_table=bt, status=status)
        assert int(status.item()) == 1
        assert torch.isnan(kv[:, 0].float()).all() and torch.isnan(kv[:, 2].float()).all()
        assert not torch.isnan(kv[:, 1, :, 3].float()).any() and torch.isnan(kv[:, 1, :, 0].float()).all()
        # the generic attention kernel: the key it cannot find counts as missing, the others still count
        kv[:, 0] = 0.5
        kv[:, 1] = 0.25
        status.zero_()
        q = rnd(2, hq, d, dtype=dtype, seed=3)
        import tinyinfer_b200.ops as real_ops
        out = torch.empty((2, hq * d), dtype=dtype, device=dev())
        real_ops._run("core", "ti_attention_generic", out.data_ptr(), q.data_ptr(), kv.data_ptr(), pos.data_ptr(),
                      seq.data_ptr(), bt.data_ptr(), 1, 2, hq, hkv, d, page, 3, d ** -0.5, 0, status.data_ptr(),
                      real_ops._dtype_code(q), real_ops._stream())
        assert int(status.item()) == 2
        close(out[0], torch.full_like(out[0], 0.5), dtype)
        close(out[1], torch.full_like(out[1], 0.25), dtype)


def test_decode_attention_scratch_is_checked_and_fully_written(ops):
    """The exported decode entry point takes its scratch from the caller: with as many floats as the library
    asks for, every word the merge reads has been written (the scratch starts as NaN); with one float less
    the call is refused with a message and nothing runs."""
    from tinyinfer_b200.ops import library
    hq, hkv, d, page = 8, 2, 128, 64
    lens = [700, 300]
    dtype = torch.bfloat16
    bt, kv = paged_setup(dtype, lens, hq, hkv, d, page, seed=2)
    fill_cache(kv, bt, lens, hkv, d, page, dtype)
    pos = torch.tensor([c - 1 for c in lens], dtype=torch.int32, device=dev())
    seq = torch.arange(2, dtype=torch.int32, device=dev())
    rows = torch.arange(2, dtype=torch.int32, device=dev())
    q = rnd(2, hq, d, dtype=dtype, seed=8)
    fn = ops._fn("sm100", "ti_attention_decode_bf16")
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    want = ref.paged_attention(q, kv, positions=pos, token_seq=seq, block_table=bt, scale=d ** -0.5)
    need = ops.decode_scratch_floats(2, hq, hkv, d, max(lens), 0)
    assert 0 < need < 1 << 20
    for given, fine in ((need, True), (need - 1, False)):
        scratch = torch.full((need,), float("nan"), dtype=torch.float32, device=dev())
        out = torch.zeros((2, hq * d), dtype=dtype, device=dev())
        rc = fn(out.data_ptr(), q.data_ptr(), kv.data_ptr(), scratch.data_ptr(), given, rows.data_ptr(), 2,
                pos.data_ptr(), seq.data_ptr(), bt.data_ptr(), bt.shape[1], hq, hkv, d, page, kv.shape[1], d ** -0.5,
                0, max(lens), status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        message = library.load("sm100").ti_last_error().decode()
        assert int(status.item()) == 0
        if fine:
            assert rc == 0, message
            assert torch.isfinite(out.float()).all()
            close(out, want, dtype)
        else:
            assert rc != 0 and "floats of scratch" in message
            assert not out.any()


def fill_cache(kv, bt, lens, hkv, d, page, dtype, seed=0):
    """Writes random keys and values for positions 0..len-1 of every request; returns them."""
    ks, vs = [], []
    for i, n in enumerate(lens):
        k = rnd(n, hkv, d, dtype=dtype, seed=seed + 10 * i)
        v = rnd(n, hkv, d, dtype=dtype, seed=seed + 10 * i + 1)
        for p in range(n):
            pg = int(bt[i, p // page])
            kv[0, pg, :, p % page] = k[p]
            kv[1, pg, :, p % page] = v[p]
        ks.append(k)
        vs.append(v)
    return ks, vs


ATTN_SHAPES = [
    # hq, hkv, d, page, window, [(context, q_len)]
    (4, 2, 16, 4, None, [(9, 9), (37, 1), (20, 5)]),
    (6, 2, 32, 8, 11, [(50, 50), (33, 1), (64, 7)]),
    (8, 2, 64, 16, None, [(130, 130), (129, 1), (200, 2)]),
    (4, 1, 128, 64, 40, [(300, 44), (65, 1), (64, 1), (1, 1)]),
    (3, 3, 48, 5, None, [(17, 17), (31, 1)]),
    (2, 1, 256, 32, None, [(70, 3), (33, 1)]),
    (32, 8, 128, 64, None, [(257, 257), (512, 1), (511, 1)]),
    # the tensor-core kernels: many decode splits, windows, cached prefixes, every page size, groups 1..16
    (8, 8, 128, 16, None, [(1500, 1), (1, 1), (256, 1), (257, 1), (1024, 1)]),
    (16, 1, 64, 32, None, [(700, 1), (300, 100), (65, 64)]),
    (8, 2, 128, 128, 300, [(1000, 1), (900, 130), (299, 1), (300, 1), (301, 1)]),
    (4, 4, 64, 64, 70, [(500, 200), (129, 2), (64, 64), (1, 1)]),
    (12, 3, 128, 64, None, [(450, 61), (63, 63), (2, 2), (1100, 17)]),
    # portions of several tiles of 256 rows behind a prefix, their ends of 129 and 128 rows and less
    (8, 2, 128, 64, None, [(1300, 897), (700, 513), (640, 384), (1, 1)]),
    (4, 2, 64, 32, 200, [(1500, 1000), (420, 385)]),
]


@pytest.mark.parametrize("pair_min_ctas", [0, 1 << 30])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page,window,work", ATTN_SHAPES)
def test_paged_attention(ops, monkeypatch, dtype, hq, hkv, d, page, window, work, pair_min_ctas):
    """pair_min_ctas: 0 sends every tile of more than 128 rows to the kernel with two query tiles a CTA,
    the large value sends its halves to the kernel with one (what the product does with few tiles)."""
    if pair_min_ctas and (dtype != torch.bfloat16 or d not in (64, 128)):
        pytest.skip("one path only")
    monkeypatch.setattr(ops, "PAIR_MIN_CTAS", pair_min_ctas)
    lens = [c for c, _ in work]
    bt, kv = paged_setup(dtype, lens, hq, hkv, d, page, seed=1)
    fill_cache(kv, bt, lens, hkv, d, page, dtype)
    pos = torch.tensor([p for c, n in work for p in range(c - n, c)], dtype=torch.int32, device=dev())
    seq = torch.tensor([i for i, (c, n) in enumerate(work) for _ in range(n)], dtype=torch.int32, device=dev())
    q = rnd(pos.shape[0], hq, d, dtype=dtype, seed=7)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    args = dict(positions=pos, token_seq=seq, block_table=bt, scale=d ** -0.5, window=window)
    out = ops.paged_attention(q, kv, status=status, **args)
    assert int(status.item()) == 0
    want = ref.paged_attention(q, kv, **args)
    assert torch.isfinite(out.float()).all()
    close(out, want, dtype)


@pytest.mark.parametrize("hq,hkv,d,page,window,lens", [
    (32, 8, 128, 64, None, [4096, 3000, 1, 257, 513, 4000, 2048, 1025]),
    (8, 8, 64, 16, None, [9000, 8193, 700, 8192]),
    (8, 4, 128, 128, 2500, [6000, 2501, 2500, 5121, 40, 4608, 3000, 5632, 5633, 6000, 2600, 4097, 777, 5120]),
    # many short requests: a CTA's run of four key tiles crosses kv heads and requests
    (6, 3, 128, 32, None, [1, 64, 65, 130, 7, 200, 63, 129, 2, 300, 64, 64, 1, 191, 192, 193] * 3),
    (4, 1, 64, 16, 100, [1, 99, 100, 101, 164, 165, 230, 700, 3, 64] * 7),
    # 8 and 9 query heads a kv head at head size 128: the merge of a CTA's four warps through the smaller buffer;
    # 12 and 16: one CTA an SM with a ring of six stages
    (64, 8, 128, 64, None, [4096, 3000, 1, 257, 513, 4000, 2048, 1025, 64, 65]),
    (18, 2, 128, 64, 1500, [5000, 1499, 1500, 1501, 1, 2900, 700, 64, 63, 4097, 333, 2048]),
    (24, 2, 128, 32, None, [2600, 1, 129, 4000, 512, 77, 1024, 3001]),
    (32, 2, 128, 128, None, [6000, 1, 64, 1300, 2049, 257, 4500])])
def test_decode_attention_shares_the_keys_out_evenly(ops, hq, hkv, d, page, window, lens):
    """Long contexts are cut where a CTA's run ends, not at fixed positions, and short ones share a CTA: the
    same results wherever the cuts fall (inside a request, at its last key, across kv heads and requests, a
    window that starts inside a run)."""
    dtype = torch.bfloat16
    bt, kv = paged_setup(dtype, lens, hq, hkv, d, page, seed=5)
    fill_cache(kv, bt, lens, hkv, d, page, dtype)
    pos = torch.tensor([c - 1 for c in lens], dtype=torch.int32, device=dev())
    seq = torch.arange(len(lens), dtype=torch.int32, device=dev())
    q = rnd(len(lens), hq, d, dtype=dtype, seed=8)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    args = dict(positions=pos, token_seq=seq, block_table=bt, scale=d ** -0.5, window=window)
    out = ops.paged_attention(q, kv, status=status, **args)
    assert int(status.item()) == 0
    close(out, ref.paged_attention(q, kv, **args), dtype)
    # rows in another order and fewer of them: other cuts, the same results
    keep = list(range(len(lens) - 1, -1, -2))
    sub = ops.paged_attention(q[keep].contiguous(), kv, positions=pos[keep].contiguous(),
                              token_seq=seq[keep].contiguous(), block_table=bt, scale=d ** -0.5, window=window)
    close(sub, out[keep], dtype)
    ops.check_kernel_status()


def test_attention_at_random_sizes(ops):
    """Thirty batches drawn at random (a fixed seed): head counts and groups, head size, page size, windows,
    contexts from one key to a few thousand, single decoded tokens next to prompt portions of every length, more
    decoded rows than the decode kernel has threads: every one against the plain attention."""
    import random
    rng = random.Random(20)
    dtype = torch.bfloat16
    for case in range(30):
        d = rng.choice([64, 128])
        hkv = rng.choice([1, 2, 3, 8])
        group = rng.choice([1, 2, 4, 5, 8, 16])
        hq = hkv * group
        page = rng.choice([16, 32, 64, 128])
        window = rng.choice([None, None, rng.randrange(1, 700)])
        work = []
        if case % 5 == 0:                                   # many decoded rows
            work += [(rng.randrange(1, 400), 1) for _ in range(rng.choice([170, 200, 330]))]
        else:
            for _ in range(rng.randrange(1, 7)):
                ctx = rng.choice([1, 2, 63, 64, 65, 127, 128, 129, 255, 256, 257, rng.randrange(1, 3000)])
                n = rng.choice([1, 1, 1, ctx, min(ctx, 2), min(ctx, 128), min(ctx, 129), min(ctx, 256), min(ctx, 257),
                                rng.randrange(1, ctx + 1)])
                work.append((ctx, n))
        lens = [c for c, _ in work]
        bt, kv = paged_setup(dtype, lens, hq, hkv, d, page, seed=case)
        fill_cache(kv, bt, lens, hkv, d, page, dtype)
        pos = torch.tensor([p for c, n in work for p in range(c - n, c)], dtype=torch.int32, device=dev())
        seq = torch.tensor([i for i, (c, n) in enumerate(work) for _ in range(n)], dtype=torch.int32, device=dev())
        q = rnd(pos.shape[0], hq, d, dtype=dtype, seed=100 + case)
        args = dict(positions=pos, token_seq=seq, block_table=bt, scale=d ** -0.5, window=window)
        for pair_min in (0, 148):
            ops.PAIR_MIN_CTAS = pair_min
            try:
                out = ops.paged_attention(q, kv, **args)
            finally:
                ops.PAIR_MIN_CTAS = 148
            assert torch.isfinite(out.float()).all(), (case, work[:6], hq, hkv, d, page, window)
            want = ref.paged_attention(q, kv, **args)
            err = (out.float() - want.float()).abs().max().item()
            assert err < 3e-2, (case, err, work[:6], hq, hkv, d, page, window, pair_min)
    ops.check_kernel_status()


def test_products_at_random_sizes(ops):
    """Forty products drawn at random (a fixed seed), plain and gated, with and without bias and residual, in
    whichever form the library chooses and in the pair form: against the plain product."""
    import random
    rng = random.Random(21)
    dtype = torch.bfloat16
    for case in range(40):
        m = rng.choice([1, 7, 16, 33, 64, 65, 100, 128, 129, 300, 511, 512, 513, 700, 1024, 1300, 2050])
        n = rng.choice([128, 136, 256, 264, 520, 1000, 1024, 2048, 3080])
        k = rng.choice([8, 64, 72, 136, 512, 1096])
        gated = case % 3 == 0
        x = rnd(m, k, dtype=dtype, seed=case)
        w = rnd(2 * n if gated else n, k, dtype=dtype, seed=1000 + case, std=k ** -0.5)
        for force_pair in (False, True):
            if force_pair and (2 * n if gated else n) < 256:
                continue
            ops.PAIR_MIN_TOKENS = 1 if force_pair else 1 << 30
            try:
                if gated:
                    got, want = ops.gated_linear(x, w), ref.gated_linear(x, w)
                else:
                    bias = rnd(n, dtype=torch.float32, seed=2) if case % 2 else None
                    res = rnd(m, n, dtype=dtype, seed=3) if case % 4 < 2 else None
                    got, want = ops.linear(x, w, bias=bias, residual=res), ref.linear(x, w, bias=bias, residual=res)
            finally:
                ops.PAIR_MIN_TOKENS = 1 << 30
            close(got, want, dtype)
    ops.check_kernel_status()


@pytest.mark.parametrize("hq,hkv,d,page,window,work", [
    (4, 2, 128, 64, None, [(5000, 200), (2300, 129)]),          # halves of a 200-row tile and a 129-row tile, shares of 1,024+ keys
    (2, 1, 64, 16, None, [(9000, 100)]),                         # one tile of 100 rows on 2 CTAs: many shares
    (4, 4, 128, 128, 3000, [(8000, 256), (4100, 60), (2049, 128)]),   # a window: the first shares hold no visible key
    (8, 2, 128, 64, None, [(4096, 128), (2048, 2048)])])
def test_prompt_portions_behind_long_prefixes_share_the_keys_out(ops, monkeypatch, hq, hkv, d, page, window, work):
    """Few query tiles behind thousands of keys: the keys are split over CTAs and merged. The same results as the
    plain attention, and as the kernel without the split."""
    dtype = torch.bfloat16
    lens = [c for c, _ in work]
    bt, kv = paged_setup(dtype, lens, hq, hkv, d, page, seed=3)
    fill_cache(kv, bt, lens, hkv, d, page, dtype)
    pos = torch.tensor([p for c, n in work for p in range(c - n, c)], dtype=torch.int32, device=dev())
    seq = torch.tensor([i for i, (c, n) in enumerate(work) for _ in range(n)], dtype=torch.int32, device=dev())
    q = rnd(pos.shape[0], hq, d, dtype=dtype, seed=7)
    args = dict(positions=pos, token_seq=seq, block_table=bt, scale=d ** -0.5, window=window)
    monkeypatch.setattr(ops, "PAIR_MIN_CTAS", 1 << 30)           # the one-tile kernel takes everything
    split = ops.paged_attention(q, kv, **args)
    monkeypatch.setattr(ops, "KEY_SPLIT_MAX_CTAS", 0)
    whole = ops.paged_attention(q, kv, **args)
    assert torch.isfinite(split.float()).all()
    close(split, ref.paged_attention(q, kv, **args), dtype)
    close(split, whole, dtype)
    ops.check_kernel_status()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,page,window,ctx,far", [(64, 16, None, 700, 3), (128, 64, None, 900, 64),
                                                   (32, 8, 100, 500, 400), (128, 64, 256, 1000, 744),
                                                   (16, 4, None, 333, 0)])
def test_attention_finds_one_far_key(ops, dtype, d, page, window, ctx, far):
    """One key among hundreds is made to dominate: the output must be its value, wherever in the
    pages it lies (first key, a page's edge, the first key inside the window)."""
    hq, hkv = 4, 2
    bt, kv = paged_setup(dtype, [ctx], hq, hkv, d, page, seed=2)
    ks, vs = fill_cache(kv, bt, [ctx], hkv, d, page, dtype)
    q = rnd(1, hq, d, dtype=dtype, seed=3)
    pg = int(bt[0, far // page])
    for h in range(hkv):                                # key `far` points along q of its group's first head
        kv[0, pg, h, far % page] = (q[0, h * 2].float() * 40.0).to(dtype)
    pos = torch.tensor([ctx - 1], dtype=torch.int32, device=dev())
    seq = torch.zeros(1, dtype=torch.int32, device=dev())
    out = ops.paged_attention(q, kv, positions=pos, token_seq=seq, block_table=bt, scale=d ** -0.5,
                              window=window).view(hq, d)
    for h in range(hkv):
        close(out[h * 2], vs[0][far, h], dtype)
    if window is not None:                              # one key further back is outside: no trace of it
        out_far = far - 1
        assert ctx - 1 - out_far >= window
        pg = int(bt[0, out_far // page])
        kv[0, pg, :, out_far % page] = (q[0, 0].float() * 400.0).to(dtype)
        again = ops.paged_attention(q, kv, positions=pos, token_seq=seq, block_table=bt, scale=d ** -0.5,
                                    window=window).view(hq, d)
        assert torch.equal(again, out)


def test_argmax_and_ties(ops):
    x = rnd(9, 1000, dtype=torch.float32)
    x[3, 17] = x[3, 500] = 50.0
    x[4, 999] = 60.0
    got = ops.argmax(x)
    assert got.tolist() == torch.argmax(x, dim=-1).tolist()
    assert got[3].item() == 17 and got[4].item() == 999


def test_sampling_matches_plain(ops):
    n, v = 12, 389
    logits = rnd(n, v, dtype=torch.float32, std=2.0)
    temp = torch.tensor([1.0, 0.7, 1.3, 1.0] * 3, device=dev())
    topk = torch.tensor([0, 5, 100, 1, 389, 400, 2, 0, 50, 0, 7, 0], dtype=torch.int32, device=dev())
    greedy = torch.tensor([0, 0, 0, 0, 0, 0, 1, 0, 0, 1, 0, 0], dtype=torch.int32, device=dev())
    seed = torch.tensor([11, 11, 11, 2 ** 40 + 5] * 3, dtype=torch.int64, device=dev())
    stream = torch.arange(n, dtype=torch.int32, device=dev())
    step = torch.tensor([0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11], dtype=torch.int32, device=dev())
    got = ops.sample(logits, temp, topk, greedy, seed, stream, step).tolist()
    want = ref.sample(logits.cpu(), temp.cpu(), topk.cpu(), greedy.cpu(), seed.cpu(), stream.cpu(), step.cpu()).tolist()
    assert got == want
    # the same row in another batch, at another place, draws the same token
    again = ops.sample(logits[5:6].contiguous(), temp[5:6], topk[5:6], greedy[5:6], seed[5:6], stream[5:6], step[5:6])
    assert again.item() == got[5]


@pytest.mark.parametrize("v", [151936, 50001])
def test_sampling_of_long_rows_matches_plain(ops, v):
    """A row is shared out over several blocks: top-k through the slices' own candidates (k up to 256), through
    a scan of the whole row (larger k; hundreds of equal logits at the top), no top-k, greedy: the token is the
    one the plain sampler draws from the whole row."""
    ks = [0, 1, 100, 256, 257, 5000, 0, 50, 50, 7, 300, 3]
    n = len(ks)
    logits = rnd(n, v, dtype=torch.float32, std=2.5)
    logits[7, 1000:3500] = 9.0            # 2,500 equal logits above all others: more candidates than a slice may leave
    logits[8, ::977] = 9.0                # equal logits at the top spread over the slices: ties at the threshold are kept
    logits[9, 6] = float("-inf")
    temp = torch.tensor([1.0, 0.7, 1.3, 0.9] * 3, device=dev())
    topk = torch.tensor(ks, dtype=torch.int32, device=dev())
    greedy = torch.tensor([0, 0, 0, 0, 0, 0, 1, 0, 0, 0, 0, 1], dtype=torch.int32, device=dev())
    seed = torch.tensor([7, 2 ** 33 + 1, 99] * 4, dtype=torch.int64, device=dev())
    stream = torch.arange(n, dtype=torch.int32, device=dev())
    for first_step in (0, 40):
        step = torch.arange(first_step, first_step + n, dtype=torch.int32, device=dev())
        got = ops.sample(logits, temp, topk, greedy, seed, stream, step).tolist()
        want = ref.sample(logits.cpu(), temp.cpu(), topk.cpu(), greedy.cpu(), seed.cpu(), stream.cpu(), step.cpu()).tolist()
        assert got == want


def test_sampling_distribution_and_topk(ops):
    v, n = 64, 4000
    row = rnd(1, v, dtype=torch.float32, std=1.5)
    logits = row.expand(n, v).contiguous()
    temp = torch.full((n,), 0.8, device=dev())
    zeros = torch.zeros(n, dtype=torch.int32, device=dev())
    seed = torch.full((n,), 99, dtype=torch.int64, device=dev())
    step = torch.arange(n, dtype=torch.int32, device=dev())
    draws = ops.sample(logits, temp, zeros, zeros, seed, zeros, step).cpu().numpy()
    p = torch.softmax(row[0].cpu().double() / 0.8, dim=-1).numpy()
    freq = np.bincount(draws, minlength=v) / n
    assert np.abs(freq - p).max() < 4.0 * math.sqrt(p.max() / n) + 0.01
    k = 5
    topk = torch.full((n,), k, dtype=torch.int32, device=dev())
    draws = ops.sample(logits, temp, topk, zeros, seed, zeros, step).cpu().numpy()
    allowed = set(torch.topk(row[0], k).indices.tolist())
    assert set(draws.tolist()) <= allowed and len(set(draws.tolist())) == k


def test_token_nll(ops):
    logits = rnd(7, 1003, dtype=torch.float32, std=3.0)
    tokens = torch.tensor([0, 1002, 5, 500, 77, 3, 999], dtype=torch.int32, device=dev())
    torch.testing.assert_close(ops.token_nll(logits, tokens), ref.token_nll(logits, tokens), rtol=1e-5, atol=1e-5)
