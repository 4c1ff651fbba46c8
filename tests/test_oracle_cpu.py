"""The C oracle against two independent restatements and against the committed fixtures."""
import math
import os

import numpy as np
import pytest
import torch

from oracle.oracle import attention_f64, gemm_f64

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(1, 128, 128, 2, 64), (2, 96, 160, 3, 32), (1, 257, 257, 1, 128)])
def test_attention_matches_numpy_f64(oracle, shape, causal):
    B, Sq, Skv, H, D = shape
    rng = np.random.default_rng(7)
    q = rng.standard_normal((B, Sq, H, D), dtype=np.float32)
    k = rng.standard_normal((B, Skv, H, D), dtype=np.float32)
    v = rng.standard_normal((B, Skv, H, D), dtype=np.float32)
    scale = 1.0 / math.sqrt(D)
    got = oracle.attention(q, k, v, scale, causal)
    ref = attention_f64(q, k, v, scale, causal)
    assert np.abs(got["o"] - ref["o"]).max() < 2e-5
    assert np.abs(got["lse"] - ref["lse"]).max() < 2e-5
    assert np.abs(got["row_max"] - ref["row_max"]).max() < 2e-5
    assert np.abs(got["inv_sum"] / ref["inv_sum"] - 1).max() < 2e-5


def test_attention_matches_torch_sdpa(oracle):
    B, S, H, D = 2, 192, 4, 64
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(B, S, H, D, generator=g) for _ in range(3))
    for causal in (False, True):
        ref = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal).transpose(1, 2)
        got = oracle.attention(q.numpy(), k.numpy(), v.numpy(), 1.0 / math.sqrt(D), causal)["o"]
        assert np.abs(got - ref.numpy()).max() < 2e-5


def test_attention_head_and_batch_ranges(oracle):
    rng = np.random.default_rng(0)
    q, k, v = (rng.standard_normal((2, 64, 4, 32), dtype=np.float32) for _ in range(3))
    full = oracle.attention(q, k, v, 0.2)["o"]
    part = oracle.attention(q, k, v, 0.2, b_range=(1, 2), h_range=(1, 3))["o"]
    assert np.array_equal(part[1, :, 1:3], full[1, :, 1:3])
    assert not part[0].any() and not part[1, :, 0].any() and not part[1, :, 3].any()


@pytest.mark.parametrize("col_major", [True, False])
def test_gemm_matches_numpy_f64(oracle, col_major):
    rng = np.random.default_rng(5)
    a = rng.uniform(-1, 1, (70, 96)).astype(np.float32)
    b = rng.uniform(-1, 1, (50, 96)).astype(np.float32)
    c0 = rng.uniform(-1, 1, (70, 50)).astype(np.float32)
    got = oracle.gemm(a, b, alpha=0.5, beta=2.0, c_in=c0, c_col_major=col_major)
    assert np.abs(got - gemm_f64(a, b, 0.5, 2.0, c0)).max() < 1e-4


@pytest.mark.parametrize("name,tdt", [("fp16", torch.float16), ("bf16", torch.bfloat16), ("e4m3", torch.float8_e4m3fn)])
def test_conversions_bit_exact_with_torch(oracle, name, tdt):
    rng = np.random.default_rng(11)
    x = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * 3,
        rng.standard_normal(20000).astype(np.float32) * 1e-3,
        rng.uniform(-500, 500, 20000).astype(np.float32),
        np.array([0.0, -0.0, 1.0, -1.0, 448.0, 447.9, 464.0, 1e-9, 2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -11,
                  65504.0, 65519.0, 6.1e-5, 5.96e-8, 2.98e-8, 2.99e-8], np.float32)])
    if name == "e4m3":
        x = np.clip(x, -448, 448)        # torch's cast does not saturate; the oracle's does (tested below)
    raw = oracle.quantize(x, name)
    t = torch.from_numpy(x).to(tdt)
    view = t.view(torch.uint8 if name == "e4m3" else torch.int16).numpy().astype(raw.dtype)
    assert np.array_equal(raw, view)
    back = oracle.dequantize(raw, name)
    assert np.array_equal(back, t.float().numpy())


def test_e4m3_saturates(oracle):
    raw = oracle.quantize(np.array([1e6, -1e6, 449.0, 480.0], np.float32), "e4m3")
    assert np.array_equal(oracle.dequantize(raw, "e4m3"), np.array([448, -448, 448, 448], np.float32))


def test_compare_rule(oracle):
    ref = np.array([1.0, 1.0, 0.001, 2.0, 0.0], np.float32)
    got = np.array([1.004, 1.2, 0.0061, 2.0, 0.0], np.float32)     # only elements 1 and 2 break abs AND rel
    r = oracle.compare(got, ref)
    assert r["mismatch_pct"] == pytest.approx(40.0)
    assert r["max_abs"] == pytest.approx(0.2, rel=1e-5) and r["argmax"] == 1
    r = oracle.compare(np.array([np.nan, 1.0], np.float32), np.array([1.0, 1.0], np.float32))
    assert r["nonfinite"] == 1 and r["mismatch_pct"] == pytest.approx(50.0)


def test_fill_is_index_keyed(oracle):
    whole = oracle.fill((1000,), seed=3081, kind="normal")
    part = oracle.fill((300,), seed=3081, kind="normal", first_index=200)
    assert np.array_equal(whole[200:500], part)
    big = oracle.fill((200000,), seed=1, kind="normal")
    assert abs(big.mean()) < 0.01 and abs(big.std() - 1) < 0.01
    u = oracle.fill((200000,), seed=2, kind="uniform")
    assert u.min() >= -1 and u.max() <= 1 and abs(u.mean()) < 0.01


def test_golden_fixtures(oracle):
    data = np.load(os.path.join(GOLDEN, "attention_small.npz"))
    for tag in ("c1", "causal", "ragged", "causal64", "ragged64"):
        q, k, v = data[f"{tag}_q"], data[f"{tag}_k"], data[f"{tag}_v"]
        causal = bool(data[f"{tag}_causal"])
        got = oracle.attention(q, k, v, float(data[f"{tag}_scale"]), causal)
        assert np.abs(got["o"] - data[f"{tag}_o"]).max() < 2e-5
        assert np.abs(got["lse"] - data[f"{tag}_lse"]).max() < 2e-5
    data = np.load(os.path.join(GOLDEN, "attention_d128.npz"))
    for tag in ("causal128", "offset128"):
        q, k, v = data[f"{tag}_q"], data[f"{tag}_k"], data[f"{tag}_v"]
        got = oracle.attention(q, k, v, float(data[f"{tag}_scale"]), bool(data[f"{tag}_causal"]))
        assert np.abs(got["o"] - data[f"{tag}_o"]).max() < 2e-5
        assert np.abs(got["lse"] - data[f"{tag}_lse"]).max() < 2e-5
    g = np.load(os.path.join(GOLDEN, "gemm_small.npz"))
    got = oracle.gemm(g["a"], g["b"], alpha=float(g["alpha"]), beta=float(g["beta"]), c_in=g["c_in"])
    assert np.abs(got - g["c"]).max() < 1e-4
