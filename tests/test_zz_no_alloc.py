"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some callers of the kernels may not allocate device memory (code inside another runtime's capture
region, an engine that has handed all free memory to its cache). For them the library exports
``ti_attention_decode_bf16_noalloc``, which keeps the split partials in an array built into the
library. This test calls that symbol with ctypes, twice in a row with different inputs, and checks
each result against the ordinary entry point (which takes a scratch buffer from the caller) and
against the plain PyTorch statement of paged attention, within the tolerance the other kernel tests
use (contexts that end exactly on a split of 256 keys and one key past it, and a sliding window among
them); it also checks that the call allocates nothing and that a call beyond the built-in capacity is
refused with a message. It is collected last so that a run
that stops at the first failure has already run every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

c_int, c_float, c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p


def make_case(seed, contexts, hq=8, hkv=2, d=128, page=64):
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(seed)
    n = len(contexts)
    pages_per = [(c + page - 1) // page for c in contexts]
    total = sum(pages_per) + 2
    perm = torch.randperm(total, generator=g).tolist()
    width = max(pages_per)
    table, nxt = [], 0
    for k in pages_per:
        table.append(perm[nxt:nxt + k] + [-1] * (width - k))
        nxt += k
    kv = (torch.randn(2, total, hkv, page, d, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    q = torch.randn(n, hq, d, generator=g).to(torch.bfloat16).to(dev)
    return dict(
        q=q, kv=kv, block_table=torch.tensor(table, dtype=torch.int32, device=dev),
        positions=torch.tensor([c - 1 for c in contexts], dtype=torch.int32, device=dev),
        token_seq=torch.arange(n, dtype=torch.int32, device=dev),
        rows=torch.arange(n, dtype=torch.int32, device=dev), hq=hq, hkv=hkv, d=d, page=page, pages=total,
        max_context=max(contexts))


def test_noalloc_entry_point_matches_the_ordinary_one_twice():
    from tinyinfer_b200 import ops
    from tinyinfer_b200.ops import library
    lib = library.load("sm100")
    fn = lib.ti_attention_decode_bf16_noalloc
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                   c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p]
    lib.ti_attention_decode_noalloc_capacity.restype = ctypes.c_longlong
    capacity = lib.ti_attention_decode_noalloc_capacity()
    assert capacity == 2 * 1024 * 1024
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")

    def call(case, out, num_rows=None, window=0):
        return fn(out.data_ptr(), case["q"].data_ptr(), case["kv"].data_ptr(), case["rows"].data_ptr(),
                  num_rows or case["rows"].shape[0], case["positions"].data_ptr(), case["token_seq"].data_ptr(),
                  case["block_table"].data_ptr(), case["block_table"].shape[1], case["hq"], case["hkv"], case["d"],
                  case["page"], case["pages"], float(case["d"]) ** -0.5, window, case["max_context"],
                  status.data_ptr(), stream)

    import torch_ops
    # calls in a row, each with fewer or shorter requests than the one before: what a call left in the
    # shared array must not show in the next
    for seed, contexts, window in ((1, [700, 1, 256, 257, 1030], 0), (2, [90, 300], 0), (3, [512, 513, 40], 300)):
        case = make_case(seed, contexts)
        args = dict(positions=case["positions"], token_seq=case["token_seq"], block_table=case["block_table"],
                    scale=float(case["d"]) ** -0.5, window=window or None)
        want = ops.paged_attention(case["q"], case["kv"], **args)
        plain = torch_ops.paged_attention(case["q"], case["kv"], **args)
        out = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        assert call(case, out, window=window) == 0, lib.ti_last_error().decode()
        torch.cuda.synchronize()
        assert (torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]) == before, "the call allocated"
        assert torch.isfinite(out.float()).all()
        torch.testing.assert_close(out.float(), want.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(out.float(), plain.float(), rtol=2e-2, atol=2e-2)
    assert int(status.item()) == 0
    ops.check_kernel_status()

    # beyond the built-in scratch: refused before anything is read or launched, with a message that says why
    # (the call claims more rows than the scratch has slots for; it never looks at them)
    case = make_case(3, [40])
    out = torch.zeros(1, case["hq"] * case["d"], dtype=torch.bfloat16, device="cuda:0")
    too_many = capacity // (case["hq"] * (case["d"] + 2)) + 1
    assert call(case, out, num_rows=too_many) != 0
    assert b"built-in scratch" in lib.ti_last_error()
    assert not out.any()
