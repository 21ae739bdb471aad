"""The plain implementation against logits of the reference project's own model code.

``tests/golden/ref_logits.npz`` was written by ``tests/golden/make_golden.py``, which runs
tinyinfer/models/qwen3.py of the reference on the CPU (its three extension calls replaced by
stand-ins made of the reference's own live Python layers); ``tests/golden/ref_logits_gpu.npz`` by the
same script on a B200 with no stand-in: there the reference's CUDA kernels (norm, rotation,
feed-forward, FlashAttention and FlashDecoding) computed every number, in float32."""
from pathlib import Path

import numpy as np
import torch

import plain_qwen3 as plain
from golden.make_golden import GOLDEN_CONFIG, GOLDEN_MODELS, GOLDEN_TOKENS, golden_weights

GOLDEN = Path(__file__).parent / "golden" / "ref_logits.npz"
GOLDEN_GPU = Path(__file__).parent / "golden" / "ref_logits_gpu.npz"


def test_plain_matches_reference_model_code():
    """Two models (untied with head_dim != hidden / heads; tied), each request whole and in two portions."""
    ref = np.load(GOLDEN)
    for prefix, (cfg, tokens_list, seed) in GOLDEN_MODELS.items():
        w32 = golden_weights(cfg, seed)
        for dtype, tol in ((torch.float32, 2e-5), (torch.float64, 2e-5)):
            w = {k: v.to(dtype) for k, v in w32.items()}
            for r, tokens in enumerate(tokens_list):
                got = plain.forward(cfg, w, tokens).to(torch.float64).numpy()
                for tag in ("whole", "cut"):
                    want = ref[f"{prefix}req{r}_{tag}"].astype(np.float64)
                    assert got.shape == want.shape
                    assert np.abs(got - want).max() < tol, (prefix, dtype, r, tag)


def test_plain_matches_the_reference_kernels():
    """The same models through the reference's own CUDA kernels on a B200 (float32): whole prompts and
    portions through its FlashAttention kernel, the last tokens one by one through its FlashDecoding
    kernel. The tolerance is the one the engine's 32-bit path is held to."""
    ref = np.load(GOLDEN_GPU)
    checked = 0
    for prefix, (cfg, tokens_list, seed) in GOLDEN_MODELS.items():
        w = {k: v.double() for k, v in golden_weights(cfg, seed).items()}
        for r, tokens in enumerate(tokens_list):
            got = plain.forward(cfg, w, tokens).numpy()
            for tag in ("whole", "cut", "decode"):
                key = f"{prefix}req{r}_{tag}"
                if key not in ref.files:
                    continue
                want = ref[key].astype(np.float64)
                assert got.shape == want.shape
                assert np.abs(got - want).max() <= 5e-5 * np.abs(got).max(), (key, np.abs(got - want).max())
                checked += 1
    assert checked >= 11


def test_plain_window_equals_full_when_window_covers_everything():
    w = {k: v.double() for k, v in golden_weights().items()}
    tokens = GOLDEN_TOKENS[0]
    full = plain.forward(GOLDEN_CONFIG, w, tokens)
    cfg = dict(GOLDEN_CONFIG, sliding_window=len(tokens), layer_types=["sliding_attention"] * 2)
    assert torch.equal(full, plain.forward(cfg, w, tokens))
    cfg = dict(GOLDEN_CONFIG, sliding_window=3, layer_types=["full_attention", "sliding_attention"])
    cut = plain.forward(cfg, w, tokens)
    assert torch.allclose(cut[:3], full[:3])          # the window has not bitten yet
    assert not torch.allclose(cut[5:], full[5:])


def test_plain_parts():
    torch.manual_seed(0)
    x = torch.randn(5, 3, 8, dtype=torch.float64)
    # position 0 is the identity of the rotation
    assert torch.allclose(plain.rope(x[:1], [0], 10000.0), x[:1])
    # a rotation keeps the norm of every (j, j + half) pair
    y = plain.rope(x, [3, 9, 27, 81, 243], 1e6)
    assert torch.allclose(x[..., :4] ** 2 + x[..., 4:] ** 2, y[..., :4] ** 2 + y[..., 4:] ** 2)
    # RMSNorm of a row gives unit mean square before the weight
    n = plain.rmsnorm(x, torch.ones(8, dtype=torch.float64), 0.0)
    assert torch.allclose(n.pow(2).mean(-1), torch.ones(5, 3, dtype=torch.float64))
    # one query, one key: attention returns v
    q = torch.randn(1, 4, 8, dtype=torch.float64)
    kv = torch.randn(1, 2, 8, dtype=torch.float64)
    o = plain.attention(q, kv, kv, 0.3)
    assert torch.allclose(o[0, 0], kv[0, 0]) and torch.allclose(o[0, 3], kv[0, 1])


def test_plain_sampler():
    row = np.array([0.1, 2.0, -1.0, 2.0, 0.5], dtype=np.float32)
    assert plain.sample(row, greedy=True) == 1            # first index wins the tie
    # top-k 1 at any temperature is the argmax as well (ties at the threshold stay: 1 or 3)
    assert plain.sample(row, greedy=False, temperature=0.7, topk=1, seed=3) in (1, 3)
    draws = [plain.sample(row, greedy=False, temperature=1.0, topk=0, seed=7, stream=2, step=s)
             for s in range(200)]
    assert draws == [plain.sample(row, greedy=False, temperature=1.0, topk=0, seed=7, stream=2, step=s)
                     for s in range(200)]
    freq = np.bincount(draws, minlength=5) / 200.0
    p = np.exp(row) / np.exp(row).sum()
    assert np.abs(freq - p).max() < 0.12
    u = [plain.uniform_for(1, 0, 0, i) for i in range(64)]
    assert 0.0 < min(u) and max(u) < 1.0
