"""Python face of the CUDA kernels: one function per kernel family.

Every function checks shapes and dtypes, allocates its output with torch, and calls an
``extern "C"`` launcher of ``tinyinfer_b200/csrc`` on the current CUDA stream. There is no CPU
path and no library attention or model code behind these names: a tensor that is not on a CUDA
device, or a library that cannot be built, raises.

Conventions: activations and matrices are bfloat16 or float32 (the model's compute dtype),
norm weights, biases and logits are float32, indices are int32, and everything is contiguous.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import library

c_int, c_float, c_void_p, c_ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong


class KernelError(RuntimeError):
    pass


_SIGNATURES = {
    "core": {
        "ti_embedding": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "ti_feed_tokens": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
        "ti_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
        "ti_add": [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p],
        "ti_qk_norm_rope_append": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float,
                                   c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                   c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
        "ti_attention_generic": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                 c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                 c_void_p, c_int, c_void_p],
        "ti_gemm_simt": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                         c_int, c_int, c_int, c_void_p],
        "ti_sample": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                      c_void_p, c_int, c_void_p],
        "ti_argmax": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
        "ti_token_nll": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "ti_sample_parts": [],
        "ti_sample_candidates": [],
    },
}
_SIGNATURES["sm100"] = {
    "ti_gemm_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                     c_void_p, c_ll, c_void_p, c_int, c_void_p, c_void_p],
    "ti_gemm_bf16_linked": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                            c_void_p, c_ll, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_void_p, c_void_p],
}
_SIGNATURES["sm100"]["ti_gemm_set_pair_form"] = [c_int]
_SIGNATURES["sm100"]["ti_gemm_pair_bf16"] = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                             c_int, c_void_p, c_void_p]
NORM_LINK_MAX_TOKENS = 64   # up to here two products can share an RMSNorm between them (see linear)
PAIR_MIN_TOKENS = 1 << 30   # tests and measurements: from this many tokens on a product is sent to the pair form (two
                            # CTAs a 256 x 256 tile) whatever the library would choose; it chooses by itself from 512 on


def set_pair_form(allowed: bool) -> None:
    """Measurements: whether the library may run products of many tokens in the pair form (default: yes)."""
    _fn("sm100", "ti_gemm_set_pair_form")(1 if allowed else 0)
_SIGNATURES["sm100"]["ti_attention_decode_bf16"] = [
    c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
    c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p]
_SIGNATURES["sm100"]["ti_attention_decode_scratch_floats"] = [c_int, c_int, c_int, c_int, c_int, c_int]
_SIGNATURES["sm100"]["ti_attention_prefill_pair_bf16"] = [
    c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
    c_float, c_int, c_void_p, c_void_p]
_SIGNATURES["sm100"]["ti_attention_prefill_tc_bf16"] = [
    c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
    c_float, c_int, c_int, c_int, c_int, c_void_p, c_ll, c_void_p, c_void_p]
PREFILL_TILE = 256        # most query rows per CTA of the prefill attention kernels (two tiles of 128)
PAIR_MIN_CTAS = 148       # fewer CTAs than this of the two-tile kernel: its tiles run as halves, one a CTA
KEY_SPLIT_MAX_CTAS = 148  # at most half as many CTAs of the one-tile kernel: the keys are shared out over CTAs as well
_bound = {}
_status = {}


def status_words(device) -> torch.Tensor:
    """The two int32 device words through which kernels report what they could not do:
    [0] a bounded wait that ran out (the number of the wait), [1] a token or key whose request holds no
    page for it, or a context longer than the splits it was given. Zero means all is well."""
    key = torch.device(device)
    t = _status.get(key)
    if t is None:
        t = _status[key] = torch.zeros(2, dtype=torch.int32, device=key)
    return t


def kernel_status(device) -> torch.Tensor:
    """The word that kernels with bounded waits set when a wait runs out."""
    return status_words(device)[0:1]


def page_status(device) -> torch.Tensor:
    """The word that kernels set when they meet a token or a key without a page."""
    return status_words(device)[1:2]


def status_message(wait_code: int, page_code: int) -> Optional[str]:
    """What two status words say, or None if both are zero."""
    said = []
    if wait_code == 23:
        said.append("a decode step has more key tiles than its attention kernel counts (2^31: about 137 G keys); "
                    "the step's results are not to be used")
    elif wait_code:
        said.append(f"a kernel gave up waiting on a barrier (status {wait_code}); the step's results are not to be used")
    if page_code:
        said.append(f"a kernel met a token or key without a page (status {page_code})")
    return "; ".join(said) or None


def raise_on_status(device, wait_code: int, page_code: int) -> None:
    """Raises KernelError (and clears the words) if either code, read from ``device``, is set."""
    msg = status_message(wait_code, page_code)
    if msg is not None:
        status_words(device).zero_()
        raise KernelError(msg)


def check_kernel_status() -> None:
    """Raises if any kernel reported a wait that ran out or a missing page (synchronises)."""
    for device, t in list(_status.items()):
        wait_code, page_code = t.tolist()
        raise_on_status(device, wait_code, page_code)


_WORKSPACE_FLOATS = 12 * 1024 * 1024     # 48 MB of float32 partial tiles for the stream-k cuts of matrix products
_NUM_COUNTERS = 16384
_workspace = {}


def _gemm_scratch(device):
    """(partials, counters) shared by all tensor-core matrix products on this device; safe because
    they are ordered on one stream and every launch leaves the counters at zero."""
    key = torch.device(device)
    pair = _workspace.get(key)
    if pair is None:
        pair = _workspace[key] = (torch.empty(_WORKSPACE_FLOATS, dtype=torch.float32, device=key),
                                  torch.zeros(_NUM_COUNTERS, dtype=torch.int32, device=key))
    return pair


def _tensor_core_ok(x: torch.Tensor, w: torch.Tensor, *others) -> bool:
    """The tcgen05 kernels take bfloat16 operands whose rows start on 16-byte boundaries."""
    if x.dtype != torch.bfloat16 or x.shape[1] % 8:
        return False
    return all(t is None or t.data_ptr() % 16 == 0 for t in (x, w) + others)


def _fn(lib_name: str, name: str):
    key = (lib_name, name)
    fn = _bound.get(key)
    if fn is None:
        lib = library.load(lib_name)
        fn = getattr(lib, name)
        fn.argtypes = _SIGNATURES[lib_name][name]
        fn.restype = c_int
        _bound[key] = fn
    return fn


def _run(lib_name: str, name: str, *args) -> None:
    rc = _fn(lib_name, name)(*args)
    if rc != 0:
        msg = library.load(lib_name).ti_last_error().decode(errors="replace")
        raise KernelError(f"{name} failed ({rc}): {msg}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle (the raw query is an order of magnitude cheaper than
    torch.cuda.current_stream(), and this runs once per kernel launch)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"compute dtype must be float32 or bfloat16, got {t.dtype}")


def _check(t: torch.Tensor, name: str, dtype=None, ndim: Optional[int] = None) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor: tinyinfer_b200 has no CPU path")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} must have {ndim} dimensions, got shape {tuple(t.shape)}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    return t


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# ---------------------------------------------------------------------- elementwise
def embedding(token_ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """rows of ``table`` [V, H] at ``token_ids`` int32 [T] -> [T, H]."""
    _check(token_ids, "token_ids", torch.int32, 1)
    _check(table, "table", None, 2)
    out = torch.empty((token_ids.shape[0], table.shape[1]), dtype=table.dtype, device=table.device)
    _run("core", "ti_embedding", out.data_ptr(), table.data_ptr(), token_ids.data_ptr(),
         token_ids.shape[0], table.shape[1], table.shape[0], _dtype_code(table), _stream())
    return out


def feed_tokens(token_ids: torch.Tensor, dst_rows: torch.Tensor, src_rows: torch.Tensor, src: torch.Tensor) -> None:
    """token_ids[dst_rows[i]] = src[src_rows[i]] wherever dst_rows[i] >= 0 (all int32, on the device): tokens
    that a step sampled become inputs of the next step without a trip to the host."""
    _check(token_ids, "token_ids", torch.int32, 1)
    _check(dst_rows, "dst_rows", torch.int32, 1)
    _check(src_rows, "src_rows", torch.int32, 1)
    _check(src, "src", torch.int32, 1)
    if src_rows.shape[0] != dst_rows.shape[0]:
        raise KernelError("feed_tokens: one source row per destination row")
    _run("core", "ti_feed_tokens", token_ids.data_ptr(), dst_rows.data_ptr(), src_rows.data_ptr(), src.data_ptr(),
         dst_rows.shape[0], _stream())


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """w * x * rsqrt(mean(x^2) + eps) over the last axis; ``rows`` int32 [N] picks input rows."""
    _check(x, "x")
    _check(weight, "weight", torch.float32, 1)
    size = x.shape[-1]
    if weight.shape[0] != size:
        raise KernelError(f"norm weight has {weight.shape[0]} entries, rows have {size}")
    if rows is None:
        out = torch.empty_like(x)
        n = x.numel() // size
    else:
        _check(rows, "rows", torch.int32, 1)
        if x.dim() != 2:
            raise KernelError("row selection needs a 2-D input")
        n = rows.shape[0]
        out = torch.empty((n, size), dtype=x.dtype, device=x.device)
    _run("core", "ti_rmsnorm", out.data_ptr(), x.data_ptr(), weight.data_ptr(), _ptr(rows), n, size,
         float(eps), _dtype_code(x), _stream())
    return out


def add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a + b, summed in float32 and rounded once."""
    _check(a, "a")
    _check(b, "b", a.dtype)
    if a.shape != b.shape:
        raise KernelError(f"add: shapes differ {tuple(a.shape)} vs {tuple(b.shape)}")
    out = torch.empty_like(a)
    _run("core", "ti_add", out.data_ptr(), a.data_ptr(), b.data_ptr(), a.numel(), _dtype_code(a), _stream())
    return out


# ---------------------------------------------------------------------- matrix products
class NormLink:
    """What a product leaves for the RMSNorm behind it, when that norm is spread over the two products
    around it: ``scaled`` = x * g in x's dtype (x: the product's output as rounded, g: the norm's weight),
    ``sums`` float32 [parts, M]: per token, partial sums of squares of x; ``weight`` is g itself (kept to
    tell which norm the link was made for), ``size`` the length of a row of x."""

    def __init__(self, scaled, sums, parts, weight, size):
        self.scaled, self.sums, self.parts, self.weight, self.size = scaled, sums, parts, weight, size


def norm_link_ok(x: torch.Tensor) -> bool:
    """True if the products around an RMSNorm of ``x`` can share it (bfloat16 on the tensor cores, at
    most 64 rows): the norm kernel between them, a hop of a decode step, is then left out."""
    return x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] <= NORM_LINK_MAX_TOKENS


def _gemm_linked(out, x, w, bias, residual, m, n, k, gated, scale, emit_weight):
    ws, counters = _gemm_scratch(x.device)
    scaled = sums = None
    if emit_weight is not None:
        scaled = torch.empty((m, n), dtype=x.dtype, device=x.device)
        sums = torch.empty(((n + 127) // 128, m), dtype=torch.float32, device=x.device)
    written = ctypes.c_int(0)
    _run("sm100", "ti_gemm_bf16_linked", out.data_ptr(), x.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(residual),
         m, n, k, gated, ws.data_ptr(), ws.numel(), counters.data_ptr(), counters.numel(),
         scale[0].sums.data_ptr() if scale else None, scale[0].parts if scale else 0,
         scale[0].size if scale else 0, float(scale[1]) if scale else 0.0,
         _ptr(emit_weight), _ptr(scaled), _ptr(sums), ctypes.addressof(written),
         kernel_status(x.device).data_ptr(), _stream())
    if emit_weight is None or written.value == 0:
        return None
    return NormLink(scaled, sums, written.value, emit_weight, n)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           residual: Optional[torch.Tensor] = None, out_float32: bool = False, *,
           link: Optional[NormLink] = None, link_eps: float = 0.0,
           next_norm_weight: Optional[torch.Tensor] = None):
    """x [M, K] . w [N, K]^T (+ bias [N]) (+ residual [M, N]), float32 accumulation.
    ``out_float32`` stores the accumulator unrounded (logits).

    An RMSNorm between two products of at most 64 tokens can be spread over them.
    ``next_norm_weight`` (float32 [N]): the weight of the norm that follows THIS product; the result is
    then (out, NormLink or None): the link, if the kernel could make it, holds out * weight and the
    sums of squares of out's rows. ``link`` (with ``link_eps``): x is ``link.scaled`` of the norm BEFORE
    this product, and every output row is multiplied by rsqrt(mean(x_before^2) + eps) here."""
    _check(x, "x", None, 2)
    _check(w, "w", x.dtype, 2)
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"linear: x has {k} columns, w has {w.shape[1]}")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
    if residual is not None:
        _check(residual, "residual", x.dtype, 2)
        if tuple(residual.shape) != (m, n):
            raise KernelError("linear: residual shape differs from the output's")
    out = torch.empty((m, n), dtype=torch.float32 if out_float32 else x.dtype, device=x.device)
    wants_link = next_norm_weight is not None
    if link is not None or wants_link:
        if out_float32 or not (_tensor_core_ok(x, w) and norm_link_ok(x)):
            if link is not None:
                raise KernelError("linear: a norm link needs the tensor-core product of at most 64 rows")
        else:
            made = _gemm_linked(out, x, w, bias, residual, m, n, k, 0, (link, link_eps) if link else None,
                                next_norm_weight)
            return (out, made) if wants_link else out
    if _tensor_core_ok(x, w) and m >= PAIR_MIN_TOKENS and n >= 256:
        _run("sm100", "ti_gemm_pair_bf16", out.data_ptr(), x.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(residual),
             m, n, k, 0, int(out_float32), kernel_status(x.device).data_ptr(), _stream())
        return (out, None) if wants_link else out
    if _tensor_core_ok(x, w):
        ws, counters = _gemm_scratch(x.device)
        _run("sm100", "ti_gemm_bf16", out.data_ptr(), x.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(residual),
             m, n, k, 0, int(out_float32), ws.data_ptr(), ws.numel(), counters.data_ptr(), counters.numel(),
             kernel_status(x.device).data_ptr(), _stream())
        return (out, None) if wants_link else out
    _run("core", "ti_gemm_simt", out.data_ptr(), x.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(residual),
         m, n, k, 0, int(out_float32 and x.dtype != torch.float32), _dtype_code(x), _stream())
    return (out, None) if wants_link else out


def gated_linear(x: torch.Tensor, w_gate_up: torch.Tensor, *, link: Optional[NormLink] = None,
                 link_eps: float = 0.0) -> torch.Tensor:
    """silu(x.Wg^T) * (x.Wu^T) with ``w_gate_up`` = [Wg; Wu] of shape [2I, K] -> [M, I]; the
    activation and the product act on the float32 accumulators, one rounding. ``link``: as in
    ``linear`` (both halves are scaled before the activation)."""
    _check(x, "x", None, 2)
    _check(w_gate_up, "w_gate_up", x.dtype, 2)
    m, k = x.shape
    if w_gate_up.shape[1] != k or w_gate_up.shape[0] % 2:
        raise KernelError("gated_linear: weight must be [2I, K]")
    inter = w_gate_up.shape[0] // 2
    out = torch.empty((m, inter), dtype=x.dtype, device=x.device)
    if link is not None:
        if not (_tensor_core_ok(x, w_gate_up) and norm_link_ok(x)):
            raise KernelError("gated_linear: a norm link needs the tensor-core product of at most 64 rows")
        _gemm_linked(out, x, w_gate_up, None, None, m, inter, k, 1, (link, link_eps), None)
        return out
    if _tensor_core_ok(x, w_gate_up) and m >= PAIR_MIN_TOKENS and inter >= 128:
        _run("sm100", "ti_gemm_pair_bf16", out.data_ptr(), x.data_ptr(), w_gate_up.data_ptr(), None, None,
             m, inter, k, 1, 0, kernel_status(x.device).data_ptr(), _stream())
        return out
    if _tensor_core_ok(x, w_gate_up):
        ws, counters = _gemm_scratch(x.device)
        _run("sm100", "ti_gemm_bf16", out.data_ptr(), x.data_ptr(), w_gate_up.data_ptr(), None, None,
             m, inter, k, 1, 0, ws.data_ptr(), ws.numel(), counters.data_ptr(), counters.numel(),
             kernel_status(x.device).data_ptr(), _stream())
        return out
    _run("core", "ti_gemm_simt", out.data_ptr(), x.data_ptr(), w_gate_up.data_ptr(), None, None,
         m, inter, k, 1, 0, _dtype_code(x), _stream())
    return out


# ---------------------------------------------------------------------- attention
class Rotation:
    """How a position turns the features of a head: what a position-encoding part hands to a mixer, which
    passes it on to ``qk_norm_rope_append`` unread. The first ``rotary_dim`` features of every head are
    rotated in pairs, (j, j + rotary_dim / 2) or, ``interleaved``, (2j, 2j + 1), pair j of position p by
    the angle p * inv_freq[j] (``inv_freq`` float32 [rotary_dim / 2]) or by the angle whose cosine and
    sine stand in ``cos_sin`` (float32 [positions, rotary_dim]: a row holds the rotary_dim / 2 cosines,
    then the sines; any encoding whose angles depend on the position alone). Exactly one of the two."""

    def __init__(self, rotary_dim: int, inv_freq: Optional[torch.Tensor] = None,
                 cos_sin: Optional[torch.Tensor] = None, interleaved: bool = False):
        if (inv_freq is None) == (cos_sin is None):
            raise KernelError("a rotation needs inverse frequencies or a table of cosines and sines, one of them")
        if rotary_dim <= 0 or rotary_dim % 2:
            raise KernelError(f"rotary_dim must be positive and even, got {rotary_dim}")
        if inv_freq is not None:
            if inv_freq.dtype != torch.float32 or tuple(inv_freq.shape) != (rotary_dim // 2,):
                raise KernelError("inv_freq must be float32 with rotary_dim / 2 entries")
        elif cos_sin.dtype != torch.float32 or cos_sin.dim() != 2 or cos_sin.shape[1] != rotary_dim:
            raise KernelError("cos_sin must be float32 [positions, rotary_dim]")
        self.rotary_dim, self.inv_freq, self.cos_sin, self.interleaved = rotary_dim, inv_freq, cos_sin, bool(interleaved)


def qk_norm_rope_append(qkv: torch.Tensor, *, num_heads: int, num_kv_heads: int, head_dim: int,
                        q_norm_weight: Optional[torch.Tensor], k_norm_weight: Optional[torch.Tensor],
                        eps: float, positions: torch.Tensor, token_seq: torch.Tensor,
                        kv_cache: Optional[torch.Tensor], block_table: torch.Tensor,
                        rotation: Optional[Rotation] = None,
                        inv_freq: Optional[torch.Tensor] = None, rotary_dim: int = 0,
                        status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Splits ``qkv`` [T, (Hq + 2 Hkv) D] by heads; norms q and k per head, rotates them by
    their positions, returns q [T, Hq, D] and writes k and v into the pages of
    ``kv_cache`` [2, pages, Hkv, page, D] (None: the entry only reads the cache).
    ``rotation``: a ``Rotation`` or None (positions are not used); ``inv_freq`` with ``rotary_dim``
    is short for the half-split rotation by position * inv_freq."""
    _check(qkv, "qkv", None, 2)
    t = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError("qk_norm_rope_append: qkv width does not match the head counts")
    _check(positions, "positions", torch.int32, 1)
    _check(token_seq, "token_seq", torch.int32, 1)
    _check(block_table, "block_table", torch.int32, 2)
    for name, w in (("q_norm_weight", q_norm_weight), ("k_norm_weight", k_norm_weight)):
        if w is not None:
            _check(w, name, torch.float32, 1)
            if w.shape[0] != head_dim:
                raise KernelError(f"{name} must have head_dim entries")
    if rotation is None and inv_freq is not None:
        rotation = Rotation(rotary_dim, inv_freq=inv_freq)
    if rotation is not None:
        if rotation.rotary_dim > head_dim:
            raise KernelError(f"rotary_dim {rotation.rotary_dim} exceeds head_dim {head_dim}")
        _check(rotation.inv_freq if rotation.inv_freq is not None else rotation.cos_sin, "the rotation's tensor")
    page_size = num_pages = 1
    if kv_cache is not None:
        _check(kv_cache, "kv_cache", qkv.dtype, 5)
        if kv_cache.shape[0] != 2 or kv_cache.shape[2] != num_kv_heads or kv_cache.shape[4] != head_dim:
            raise KernelError(f"kv_cache shape {tuple(kv_cache.shape)} is not [2, pages, Hkv, page, D]")
        num_pages, page_size = kv_cache.shape[1], kv_cache.shape[3]
    q = torch.empty((t, num_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    rot = rotation
    _run("core", "ti_qk_norm_rope_append", q.data_ptr(), qkv.data_ptr(), _ptr(kv_cache),
         _ptr(q_norm_weight), _ptr(k_norm_weight), float(eps),
         _ptr(rot.inv_freq) if rot else None, _ptr(rot.cos_sin) if rot else None,
         rot.cos_sin.shape[0] if rot and rot.cos_sin is not None else 0, int(rot.interleaved) if rot else 0,
         rot.rotary_dim if rot else 0, positions.data_ptr(), token_seq.data_ptr(),
         block_table.data_ptr(), block_table.shape[1], t, num_heads, num_kv_heads, head_dim,
         page_size, num_pages, _ptr(status), _dtype_code(qkv), _stream())
    return q


def plan_attention(q_lens, starts):
    """Splits a step's entries into single decoded tokens and portions of prompts.
    Returns (decode_rows, tiles, num_pair_tiles): flat rows of entries that bring one token, and for the
    others tiles [entry, first flat row, rows, first position]. A portion is cut into tiles of
    PREFILL_TILE = 256 query rows for the kernel that runs two query tiles a CTA; what is left at its end,
    if it is at most 128 rows, is a tile for the kernel with one. The first ``num_pair_tiles`` tiles are
    the former, the rest the latter; each kind longest key range first."""
    decode_rows, pairs, singles = [], [], []
    row = 0
    for i, (n, start) in enumerate(zip(q_lens, starts)):
        if n == 1:
            decode_rows.append(row)
        else:
            off = 0
            while n - off > PREFILL_TILE // 2:
                rows = min(PREFILL_TILE, n - off)
                pairs.append((i, row + off, rows, start + off))
                off += rows
            if off < n:
                singles.append((i, row + off, n - off, start + off))
        row += n
    pairs.sort(key=lambda t: -(t[3] + t[2]))
    singles.sort(key=lambda t: -(t[3] + t[2]))
    return decode_rows, [x for t in pairs + singles for x in t], len(pairs)


def attention_tensor_cores_ok(q: torch.Tensor, kv_cache: torch.Tensor) -> bool:
    """The tensor-core attention kernels take bfloat16, head sizes 64 and 128, up to 16 query heads
    per kv head, and pages of 16, 32 or a multiple of 64 tokens."""
    _, hq, d = q.shape
    hkv, page = kv_cache.shape[2], kv_cache.shape[3]
    return (q.dtype == torch.bfloat16 and d in (64, 128) and hq % hkv == 0 and hq // hkv <= 16
            and (page in (16, 32) or page % 64 == 0))


_generic_warned = set()


def _warn_generic_attention(hq: int, hkv: int, d: int, page_size: int) -> None:
    """Says once per shape that a bfloat16 model runs its attention on the generic float32-arithmetic
    kernel: right, but many times slower than the tensor-core kernels."""
    key = (hq, hkv, d, page_size)
    if key in _generic_warned:
        return
    _generic_warned.add(key)
    import warnings
    warnings.warn(f"tinyinfer_b200: attention with {hq} query heads over {hkv} kv heads, head_dim {d}, pages of "
                  f"{page_size} runs on the generic kernel (the tensor-core kernels take head_dim 64 or 128, at most "
                  f"16 query heads per kv head, pages of 16, 32 or a multiple of 64): correct, but far slower",
                  RuntimeWarning, stacklevel=3)


_attn_scratch = {}
_attn_scratch_outgrown = []     # kept alive: captured graphs may still write their partials there


def _decode_scratch(device, floats: int) -> torch.Tensor:
    key = torch.device(device)
    t = _attn_scratch.get(key)
    if t is None or t.numel() < floats:
        if t is not None:
            _attn_scratch_outgrown.append(t)
        t = _attn_scratch[key] = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=key)
    return t


_scratch_floats = {}


def decode_scratch_floats(num_rows: int, hq: int, hkv: int, head_dim: int, max_context: int, window: int = 0) -> int:
    """Floats of scratch the decode attention kernel needs for this batch (a slot for every CTA's and every
    (request, kv head)'s partial result), as the library says. A function of its arguments alone."""
    key = (num_rows, hq, hkv, head_dim, max_context, window)
    n = _scratch_floats.get(key)
    if n is None:
        fn = _fn("sm100", "ti_attention_decode_scratch_floats")
        fn.restype = ctypes.c_longlong
        n = _scratch_floats[key] = int(fn(*key))
    return n


def release_scratch(device) -> None:
    """Drops the scratch buffers kept for ``device`` (they are made again when next needed). Only when no
    captured graph that uses them will be replayed again."""
    key = torch.device(device)
    _attn_scratch.pop(key, None)
    _attn_scratch_outgrown.clear()
    _workspace.pop(key, None)
    _argmax_scratch.pop(key, None)
    _sample_scratch.pop(key, None)


def paged_attention(q: torch.Tensor, kv_cache: torch.Tensor, *, positions: torch.Tensor,
                    token_seq: torch.Tensor, block_table: torch.Tensor, scale: float,
                    window: Optional[int] = None, step=None,
                    status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of q [T, Hq, D] over the pages of each token's own request.
    Token t sees keys max(0, pos - window + 1) .. pos of request ``token_seq[t]``.
    Returns [T, Hq * D]. ``step`` (the StepContext of the batch) carries the split of the batch
    into decoded tokens and prompt portions; without it the split is derived here (a device read)."""
    _check(q, "q", None, 3)
    _check(kv_cache, "kv_cache", q.dtype, 5)
    _check(positions, "positions", torch.int32, 1)
    _check(token_seq, "token_seq", torch.int32, 1)
    _check(block_table, "block_table", torch.int32, 2)
    t, hq, d = q.shape
    _, num_pages, hkv, page_size, d2 = kv_cache.shape
    if d2 != d or kv_cache.shape[0] != 2:
        raise KernelError("paged_attention: kv_cache does not match q")
    out = torch.empty((t, hq * d), dtype=q.dtype, device=q.device)
    if t == 0:
        return out
    if not attention_tensor_cores_ok(q, kv_cache):
        if q.dtype == torch.bfloat16:
            _warn_generic_attention(hq, hkv, d, page_size)
        _run("core", "ti_attention_generic", out.data_ptr(), q.data_ptr(), kv_cache.data_ptr(),
             positions.data_ptr(), token_seq.data_ptr(), block_table.data_ptr(), block_table.shape[1],
             t, hq, hkv, d, page_size, num_pages, float(scale), int(window or 0), _ptr(status),
             _dtype_code(q), _stream())
        return out
    if step is not None:
        decode_rows, num_decode = step.decode_rows, step.num_decode
        tiles, num_tiles, max_context = step.prefill_tiles, step.num_prefill_tiles, step.max_context
        num_pairs = step.num_pair_tiles
    else:
        pos_h, seq_h = positions.tolist(), token_seq.tolist()
        q_lens, starts = [], []
        for i, (p_, s_) in enumerate(zip(pos_h, seq_h)):
            if i and seq_h[i - 1] == s_ and pos_h[i - 1] + 1 == p_:
                q_lens[-1] += 1
            else:
                q_lens.append(1)
                starts.append(p_)
        # entries here are runs of consecutive positions; their request index comes from token_seq
        rows_l, tiles_l, num_pairs = plan_attention(q_lens, starts)
        firsts, r = [], 0
        for n in q_lens:
            firsts.append(seq_h[r])
            r += n
        for k in range(0, len(tiles_l), 4):
            tiles_l[k] = firsts[tiles_l[k]]
        decode_rows = torch.tensor(rows_l or [0], dtype=torch.int32, device=q.device)
        tiles = torch.tensor(tiles_l or [0, 0, 0, 0], dtype=torch.int32, device=q.device)
        num_decode, num_tiles, max_context = len(rows_l), len(tiles_l) // 4, max(pos_h) + 1
    kstatus = kernel_status(q.device).data_ptr()
    if num_decode:
        scratch = _decode_scratch(q.device, decode_scratch_floats(num_decode, hq, hkv, d, max_context, int(window or 0)))
        _run("sm100", "ti_attention_decode_bf16", out.data_ptr(), q.data_ptr(), kv_cache.data_ptr(),
             scratch.data_ptr(), scratch.numel(), decode_rows.data_ptr(), num_decode, positions.data_ptr(),
             token_seq.data_ptr(), block_table.data_ptr(), block_table.shape[1], hq, hkv, d, page_size,
             num_pages, float(scale), int(window or 0), int(max_context), kstatus, _stream())
    def one_tile_kernel(first: int, count: int, halves: int) -> None:
        # Few query tiles behind a long prefix: the keys are shared out over CTAs too (at least 1,024 to a CTA),
        # so that most SMs have a CTA; their partial results meet in a merge kernel.
        ctas = count * (2 if halves else 1) * hq
        splits = 1
        if ctas * 2 <= KEY_SPLIT_MAX_CTAS and max_context >= 2048:
            splits = max(1, min(KEY_SPLIT_MAX_CTAS // ctas, int(max_context) // 1024))
        split_keys = -(-(-(-int(max_context) // splits)) // 128) * 128 if splits > 1 else 0
        scratch_ptr, scratch_floats = None, 0
        if splits > 1:
            scratch = _decode_scratch(q.device, count * (2 if halves else 1) * splits * hq * 128 * (d + 2))
            scratch_ptr, scratch_floats = scratch.data_ptr(), scratch.numel()
        _run("sm100", "ti_attention_prefill_tc_bf16", out.data_ptr(), q.data_ptr(), kv_cache.data_ptr(),
             tiles.data_ptr() + 16 * first, count, t, block_table.data_ptr(), block_table.shape[1], hq, hkv, d, page_size,
             num_pages, float(scale), int(window or 0), halves, splits, split_keys, scratch_ptr, scratch_floats, kstatus,
             _stream())

    if num_pairs * hq >= PAIR_MIN_CTAS:             # two query tiles a CTA
        _run("sm100", "ti_attention_prefill_pair_bf16", out.data_ptr(), q.data_ptr(), kv_cache.data_ptr(),
             tiles.data_ptr(), num_pairs, t, block_table.data_ptr(), block_table.shape[1], hq, hkv, d, page_size,
             num_pages, float(scale), int(window or 0), kstatus, _stream())
    elif num_pairs:                                 # too few of them to fill the machine: one query tile a CTA
        one_tile_kernel(0, num_pairs, 1)
    if num_tiles > num_pairs:                       # ends of portions of at most 128 rows
        one_tile_kernel(num_pairs, num_tiles - num_pairs, 0)
    return out


# ---------------------------------------------------------------------- sampling
_ARGMAX_PARTS = 32
_argmax_scratch = {}
_sample_scratch = {}


def argmax(logits: torch.Tensor, extra: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Index of the largest logit of every row (first index on ties), int32 [N]. ``extra``: int32 device
    words (at most 32) that the kernel copies behind the tokens, so that one copy to the host brings both;
    the result then has N + len(extra) entries."""
    _check(logits, "logits", torch.float32, 2)
    n = logits.shape[0]
    num_extra = _check_extra(extra)
    out = torch.empty((n + num_extra,), dtype=torch.int32, device=logits.device)
    key = torch.device(logits.device)
    scratch = _argmax_scratch.get(key)
    if scratch is None or scratch[2].numel() < n:
        rows = max(256, n)
        scratch = _argmax_scratch[key] = (
            torch.empty(rows * _ARGMAX_PARTS, dtype=torch.float32, device=key),
            torch.empty(rows * _ARGMAX_PARTS, dtype=torch.int32, device=key),
            torch.zeros(rows, dtype=torch.int32, device=key))
    _run("core", "ti_argmax", out.data_ptr(), logits.data_ptr(), n, logits.shape[1], scratch[0].data_ptr(),
         scratch[1].data_ptr(), scratch[2].data_ptr(), _ptr(extra), num_extra, _stream())
    return out


def _check_extra(extra: Optional[torch.Tensor]) -> int:
    if extra is None:
        return 0
    _check(extra, "extra", torch.int32, 1)
    if extra.shape[0] > 32:
        raise KernelError("at most 32 extra words travel with the tokens")
    return extra.shape[0]


def sample(logits: torch.Tensor, temperature: torch.Tensor, topk: torch.Tensor, greedy: torch.Tensor,
           seed: torch.Tensor, stream_id: torch.Tensor, step: torch.Tensor,
           extra: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 logits [N, V]. Per row: ``greedy`` (int32 0/1),
    ``temperature`` (float32 > 0), ``topk`` (int32, 0 = off), and the random stream
    (``seed`` int64, ``stream_id`` int32, ``step`` int32). ``extra``: as in ``argmax``."""
    _check(logits, "logits", torch.float32, 2)
    n = logits.shape[0]
    for name, t, dt in (("temperature", temperature, torch.float32), ("topk", topk, torch.int32),
                        ("greedy", greedy, torch.int32), ("seed", seed, torch.int64),
                        ("stream_id", stream_id, torch.int32), ("step", step, torch.int32)):
        _check(t, name, dt, 1)
        if t.shape[0] != n:
            raise KernelError(f"{name} must have one entry per row")
    num_extra = _check_extra(extra)
    out = torch.empty((n + num_extra,), dtype=torch.int32, device=logits.device)
    key = torch.device(logits.device)
    scratch = _sample_scratch.get(key)
    if scratch is None or scratch[5].numel() < n:
        # a row is shared out over several blocks: their best, and for top-k their candidates, meet here
        rows = max(64, n)
        parts = int(_fn("core", "ti_sample_parts")())
        cap = int(_fn("core", "ti_sample_candidates")())
        scratch = _sample_scratch[key] = (
            torch.empty(rows * parts, dtype=torch.float32, device=key),
            torch.empty(rows * parts, dtype=torch.int32, device=key),
            torch.empty(rows * parts * cap, dtype=torch.int32, device=key),
            torch.empty(rows * parts * cap, dtype=torch.int32, device=key),
            torch.empty(rows * parts, dtype=torch.int32, device=key),
            torch.zeros(rows, dtype=torch.int32, device=key))
    _run("core", "ti_sample", out.data_ptr(), logits.data_ptr(), n, logits.shape[1],
         temperature.data_ptr(), topk.data_ptr(), greedy.data_ptr(), seed.data_ptr(),
         stream_id.data_ptr(), step.data_ptr(), *(t.data_ptr() for t in scratch), _ptr(extra), num_extra, _stream())
    return out


def token_nll(logits: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """logsumexp(logits[row]) - logits[row, tokens[row]] in float32, [N]."""
    _check(logits, "logits", torch.float32, 2)
    _check(tokens, "tokens", torch.int32, 1)
    if tokens.shape[0] != logits.shape[0]:
        raise KernelError("token_nll: one token per row")
    out = torch.empty((logits.shape[0],), dtype=torch.float32, device=logits.device)
    _run("core", "ti_token_nll", out.data_ptr(), logits.data_ptr(), tokens.data_ptr(), logits.shape[0],
         logits.shape[1], _stream())
    return out


def launch_count() -> int:
    return library.launch_count()
