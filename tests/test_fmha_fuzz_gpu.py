"""Seeded random shapes through the C ABI against the CPU oracle: ragged query and key lengths, batch and head counts
that leave the last (batch, head) group of a causal launch short, both head dimensions of the two-tile kernel and every
input type.  The shapes are small enough for the oracle; what varies is which tiles of a CTA exist and how many key
tiles each sees, which is what the tensor-memory schedules differ in."""
import math
import random

import pytest

from helpers import make_qkv, run_fmha
from test_fmha_gpu import check

pytestmark = pytest.mark.gpu


def _cases():
    rnd = random.Random(20250)
    out = []
    for i in range(36):
        dtype = i % 3
        D = 64 if (i // 3) % 2 else 128
        B = rnd.choice([1, 2, 3])
        H = rnd.choice([1, 2, 5])
        Sq = rnd.choice([1, 64, 127, 128, 129, 255, 256, 257, 384, 500, 777, 1025])
        Skv = rnd.choice([Sq, Sq, rnd.choice([1, 100, 128, 129, 640, 1300])])
        causal = rnd.random() < 0.5 and Skv >= Sq      # the library refuses a causal mask that leaves rows without keys
        out.append((dtype, B, Sq, Skv, H, D, causal))
    return out


@pytest.mark.parametrize("dtype,B,Sq,Skv,H,D,causal", _cases())
def test_fmha_random_shape_matches_oracle(lib, oracle, cuda, dtype, B, Sq, Skv, H, D, causal):
    low, f32, scales = make_qkv(dtype, B, Sq, Skv, H, D, seed=9000 + 7 * Sq + Skv + D)
    got, stats = run_fmha(lib, low, scales, dtype, causal)
    check(oracle, got, stats, f32, 1.0 / math.sqrt(D), causal, dtype)


@pytest.mark.parametrize("dtype,B,Sq,Skv,H,D,causal", _cases()[:18])
def test_fmha_random_shape_other_schedule(lib, oracle, cuda, dtype, B, Sq, Skv, H, D, causal):
    """The same shapes with the schedule the default does not pick for the type (head dimension 128 only)."""
    from cfk_b200 import TUNE_FMHA_SCHED
    if D != 128:
        pytest.skip("one schedule at this head dimension")
    low, f32, scales = make_qkv(dtype, B, Sq, Skv, H, D, seed=9000 + 7 * Sq + Skv + D)
    lib.set_tunable(TUNE_FMHA_SCHED, 0 if dtype == 2 else 1)
    try:
        got, stats = run_fmha(lib, low, scales, dtype, causal)
    finally:
        lib.set_tunable(TUNE_FMHA_SCHED, -1)
    check(oracle, got, stats, f32, 1.0 / math.sqrt(D), causal, dtype)
