"""The persistent one-tile-per-CTA FMHA kernel (CFK_TUNE_FMHA_KERNEL = 2) through the C ABI against the CPU oracle.

Same tolerances as test_fmha_gpu.py.  Every case runs with three grid sizes: one CTA per SM (the default), one CTA
per work item (no CTA ever takes a second item) and three CTAs (every CTA walks many items, so the hand-over between
items - Q buffers, the O tile of the previous item still draining, barrier phases that run on - is exercised)."""
import math

import numpy as np
import pytest
import torch

from helpers import make_qkv, run_fmha
from test_fmha_gpu import check

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[0, 3, 1 << 20], ids=["per_sm", "3ctas", "per_item"])
def persist_lib(lib, request):
    from cfk_b200 import TUNE_FMHA_GRID, TUNE_FMHA_KERNEL
    lib.set_tunable(TUNE_FMHA_KERNEL, 2)
    lib.set_tunable(TUNE_FMHA_GRID, request.param)
    yield lib
    lib.set_tunable(TUNE_FMHA_KERNEL, -1)
    lib.set_tunable(TUNE_FMHA_GRID, -1)


# (dtype, B, Sq, Skv, H, D, causal)
CASES = [
    (0, 1, 128, 128, 2, 64, False),      # config 1 of the baseline
    (0, 1, 256, 256, 1, 128, False),
    (0, 2, 1024, 1024, 3, 128, False),
    (0, 1, 1024, 1024, 2, 64, False),
    (0, 1, 1024, 1024, 2, 128, True),
    (0, 1, 1024, 1024, 2, 64, True),
    (0, 1, 384, 640, 2, 128, False),     # Sq != Skv, odd tile counts
    (0, 1, 384, 640, 2, 128, True),      # causal with an offset diagonal
    (1, 1, 1024, 1024, 2, 128, False),
    (1, 1, 2048, 2048, 2, 128, True),    # bf16: two-term P in the first blocks, plain P after
    (1, 1, 512, 512, 2, 64, True),
    (2, 1, 1024, 1024, 2, 128, False),
    (2, 1, 1024, 1024, 2, 128, True),
    (2, 1, 1024, 1024, 2, 64, False),    # e4m3 at head dimension 64: 64-byte rows, 64-byte swizzle
    (2, 2, 333, 500, 3, 64, True),
    (0, 2, 333, 333, 2, 128, True),      # ragged
    (0, 2, 1, 77, 2, 128, False),
    (1, 2, 100, 100, 2, 128, True),
    (2, 2, 200, 333, 2, 128, False),
    (0, 2, 129, 257, 2, 128, True),
    (0, 3, 640, 640, 5, 128, True),      # many items of different lengths per CTA
]


@pytest.mark.parametrize("dtype,B,Sq,Skv,H,D,causal", CASES)
def test_fmha_persist_matches_oracle(persist_lib, oracle, cuda, dtype, B, Sq, Skv, H, D, causal):
    low, f32, scales = make_qkv(dtype, B, Sq, Skv, H, D, seed=5081 + Sq + D)
    got, stats = run_fmha(persist_lib, low, scales, dtype, causal)
    check(oracle, got, stats, f32, 1.0 / math.sqrt(D), causal, dtype)


@pytest.mark.parametrize("causal", [False, True])
def test_fmha_persist_large_logits_trigger_rescale(persist_lib, oracle, cuda, causal):
    """Keys whose norm grows along the sequence move the running maximum past the lazy threshold again and again:
    each time the owner of the key tile waits for the previous P V and rescales the row of O, and the other
    warpgroup picks the new reference maximum up from the chain and rescales its partial row sum."""
    B, S, H, D = 1, 2048, 2, 128
    g = torch.Generator().manual_seed(3)
    q = torch.randn(B, S, H, D, generator=g)
    k = torch.randn(B, S, H, D, generator=g) * torch.linspace(0.2, 6.0, S).view(1, S, 1, 1)
    v = torch.randn(B, S, H, D, generator=g)
    low = [x.half() for x in (q, k, v)]
    f32 = [x.float().numpy() for x in low]
    got, stats = run_fmha(persist_lib, low, [1, 1, 1], 0, causal)
    check(oracle, got, stats, f32, 1.0 / math.sqrt(D), causal, 0, max_abs=4e-3)


def test_fmha_persist_agrees_with_two_tile_kernel(lib, cuda):
    from cfk_b200 import TUNE_FMHA_KERNEL
    low, _, scales = make_qkv(0, 2, 1024, 1024, 4, 128, seed=5)
    o1, s1 = run_fmha(lib, low, scales, 0, True)
    lib.set_tunable(TUNE_FMHA_KERNEL, 2)
    try:
        o2, s2 = run_fmha(lib, low, scales, 0, True)
    finally:
        lib.set_tunable(TUNE_FMHA_KERNEL, -1)
    assert np.abs(o1 - o2).max() <= 1e-3
    assert np.abs(s1["lse"] - s2["lse"]).max() <= 1e-4


@pytest.mark.parametrize("dtype,D,causal", [(0, 128, False), (1, 128, True), (0, 64, True)])
def test_fmha_persist_score_dump(persist_lib, cuda, dtype, D, causal):
    """Raw Q K^T before scale and mask, [B][H][Sq][Skv] (the COPYOUTMM0 output of the reference, fmha_consumer.h:31-42)."""
    B, Sq, Skv, H = 1, 300, 424, 2
    low, f32, scales = make_qkv(dtype, B, Sq, Skv, H, D, seed=11)
    q, k, v = (x.cuda() for x in low)
    o = torch.empty(B, Sq, H, D, device="cuda", dtype=torch.float16)
    dump = torch.full((B, H, Sq, Skv), -77.0, device="cuda", dtype=q.dtype)
    persist_lib.fmha_forward(q, k, v, o, dtype=dtype, batch=B, heads=H, seqlen_q=Sq, seqlen_kv=Skv, head_dim=D,
                           softmax_scale=1.0 / math.sqrt(D), causal=causal, s_dump=dump)
    persist_lib.check_device()
    ref = np.einsum("bihd,bjhd->bhij", f32[0].astype(np.float64), f32[1].astype(np.float64))
    got = dump.float().cpu().numpy()
    written = got != -77.0
    i = np.arange(Sq)[:, None]
    j = np.arange(Skv)[None, :]
    visible = (j <= i + (Skv - Sq)) if causal else np.ones((Sq, Skv), bool)
    assert written[0, 0][visible].all()
    tol = np.abs(ref) * 2.0 ** (-10 if dtype == 0 else -7) + 1e-3
    assert (np.abs(got - ref)[written] <= tol[written]).all()


@pytest.mark.parametrize("B,Sq,Skv,H,D,causal", [(1, 1024, 1024, 2, 128, False), (1, 333, 500, 1, 64, True)])
def test_fmha_persist_hybrid_e4m3_qk_fp16_v(persist_lib, oracle, cuda, B, Sq, Skv, H, D, causal):
    low8, f32_8, scales = make_qkv(2, B, Sq, Skv, H, D, seed=21 + Sq)
    low16, f32_16, _ = make_qkv(0, B, Sq, Skv, H, D, seed=21 + Sq)
    q, k, v = low8[0].cuda(), low8[1].cuda(), low16[2].cuda()
    o = torch.full((B, Sq, H, D), -1.0, device="cuda", dtype=torch.float16)
    lse = torch.zeros(B, H, Sq, device="cuda", dtype=torch.float32)
    persist_lib.fmha_forward(q, k, v, o, dtype=2, batch=B, heads=H, seqlen_q=Sq, seqlen_kv=Skv, head_dim=D,
                           softmax_scale=1.0 / math.sqrt(D), causal=causal, q_descale=scales[0], k_descale=scales[1],
                           v_descale=1.0, lse=lse, v_fp16=True)
    persist_lib.check_device()
    ref = oracle.attention(f32_8[0], f32_8[1], f32_16[2], 1.0 / math.sqrt(D), causal)
    cmp = oracle.compare(o.float().cpu().numpy(), ref["o"])
    assert cmp["nonfinite"] == 0 and cmp["max_abs"] <= 2e-3, cmp
    assert np.abs(lse.cpu().numpy() - ref["lse"]).max() <= 2e-3
