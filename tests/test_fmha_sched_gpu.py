"""The two tensor-memory schedules of the two-tile FMHA kernel at head dimension 128 (CFK_TUNE_FMHA_SCHED): probabilities
written over the scores (0), or one score buffer shared by the two query tiles with the probabilities in buffers of
their own (1).  The default picks by input type, so every case here runs under both, against the CPU oracle, and the
two must agree bit for bit: they issue the same tensor-core instructions on the same operands in a different order
in time."""
import math

import numpy as np
import pytest
import torch

from helpers import make_qkv, run_fmha
from test_fmha_gpu import check

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[0, 1], ids=["p_over_s", "shared_s"])
def sched_lib(lib, request):
    from cfk_b200 import TUNE_FMHA_SCHED
    lib.set_tunable(TUNE_FMHA_SCHED, request.param)
    yield lib
    lib.set_tunable(TUNE_FMHA_SCHED, -1)


# (dtype, B, Sq, Skv, H, D, causal)
CASES = [
    (0, 1, 256, 256, 1, 128, False),
    (0, 2, 1024, 1024, 3, 128, False),
    (0, 1, 1024, 1024, 2, 128, True),     # the two tiles of a CTA see different numbers of key tiles
    (0, 1, 384, 640, 2, 128, False),      # Sq != Skv; the last query block has one tile only
    (0, 1, 384, 640, 2, 128, True),
    (1, 1, 1024, 1024, 2, 128, False),    # bf16, two-term P everywhere: stays on schedule 0
    (1, 1, 2048, 2048, 2, 128, True),     # bf16: two-term P in the first blocks, plain P after
    (2, 1, 1024, 1024, 2, 128, False),
    (2, 1, 1024, 1024, 2, 128, True),
    (0, 2, 333, 333, 2, 128, True),       # ragged
    (0, 2, 1, 77, 2, 128, False),
    (1, 2, 100, 100, 2, 128, True),
    (2, 2, 200, 333, 2, 128, False),
    (0, 2, 129, 257, 2, 128, True),
    (0, 1, 128, 2048, 2, 128, False),     # one query tile, sixteen key tiles
    (0, 1, 2048, 128, 2, 128, False),     # one key tile
]


@pytest.mark.parametrize("dtype,B,Sq,Skv,H,D,causal", CASES)
def test_fmha_schedule_matches_oracle(sched_lib, oracle, cuda, dtype, B, Sq, Skv, H, D, causal):
    low, f32, scales = make_qkv(dtype, B, Sq, Skv, H, D, seed=6081 + Sq + Skv)
    got, stats = run_fmha(sched_lib, low, scales, dtype, causal)
    check(oracle, got, stats, f32, 1.0 / math.sqrt(D), causal, dtype)


@pytest.mark.parametrize("causal", [False, True])
def test_fmha_schedule_hybrid_matches_oracle(sched_lib, oracle, cuda, causal):
    """e4m3 Q and K with fp16 V and P (the first GEMM at the 8-bit rate, the second at the 16-bit rate)."""
    B, Sq, Skv, H, D = 2, 512, 768, 2, 128
    low8, f32_8, scales = make_qkv(2, B, Sq, Skv, H, D, seed=6500)
    low16, f32_16, _ = make_qkv(0, B, Sq, Skv, H, D, seed=6500)          # same draws, rounded to fp16
    q, k, v = low8[0].cuda(), low8[1].cuda(), low16[2].cuda()
    o = torch.full((B, Sq, H, D), -1.0, device="cuda", dtype=torch.float16)
    sched_lib.fmha_forward(q, k, v, o, dtype=2, batch=B, heads=H, seqlen_q=Sq, seqlen_kv=Skv, head_dim=D,
                           softmax_scale=1.0 / math.sqrt(D), causal=causal, q_descale=scales[0], k_descale=scales[1],
                           v_descale=1.0, v_fp16=True)
    sched_lib.check_device()
    ref = oracle.attention(f32_8[0], f32_8[1], f32_16[2], 1.0 / math.sqrt(D), causal)
    cmp = oracle.compare(o.float().cpu().numpy(), ref["o"])
    assert cmp["nonfinite"] == 0 and cmp["max_abs"] <= 2e-3, cmp


@pytest.mark.parametrize("causal", [False, True])
def test_fmha_schedule_large_logits_trigger_rescale(sched_lib, oracle, cuda, causal):
    """Keys whose norm grows along the sequence move the running maximum past the lazy threshold again and again; with
    the probabilities in their own buffers the rescale of O has to wait for the previous P V by a barrier of its own."""
    B, S, H, D = 1, 2048, 2, 128
    g = torch.Generator().manual_seed(3)
    q = torch.randn(B, S, H, D, generator=g)
    k = torch.randn(B, S, H, D, generator=g) * torch.linspace(0.2, 6.0, S).view(1, S, 1, 1)
    v = torch.randn(B, S, H, D, generator=g)
    low = [x.half() for x in (q, k, v)]
    f32 = [x.float().numpy() for x in low]
    got, stats = run_fmha(sched_lib, low, [1, 1, 1], 0, causal)
    check(oracle, got, stats, f32, 1.0 / math.sqrt(D), causal, 0, max_abs=4e-3)


@pytest.mark.parametrize("dtype,causal", [(0, False), (0, True), (1, True), (2, False), (2, True)])
def test_fmha_schedules_agree_bit_for_bit(lib, cuda, dtype, causal):
    from cfk_b200 import TUNE_FMHA_EXP_EMU, TUNE_FMHA_SCHED
    low, _, scales = make_qkv(dtype, 2, 1536, 1536, 4, 128, seed=77)
    outs = []
    try:
        lib.set_tunable(TUNE_FMHA_EXP_EMU, 1)      # its default depends on the schedule; the arithmetic must not
        for sched in (0, 1):
            lib.set_tunable(TUNE_FMHA_SCHED, sched)
            o, stats = run_fmha(lib, low, scales, dtype, causal)
            outs.append((o, stats))
    finally:
        lib.set_tunable(TUNE_FMHA_SCHED, -1)
        lib.set_tunable(TUNE_FMHA_EXP_EMU, -1)
    assert np.array_equal(outs[0][0], outs[1][0])
    for name in outs[0][1]:
        assert np.array_equal(outs[0][1][name], outs[1][1][name]), name
