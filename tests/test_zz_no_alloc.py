"""cfk_fmha_forward_static: the forward pass for callers that may not allocate device memory (servers
whose own pool owns all of HBM, latency-bound loops, hosts that forbid allocation after start-up).  It must
give what cfk_fmha_forward gives, call after call, although its scratch is one shared array that keeps
the previous call's contents.  Collected last on purpose: a stop-at-first-failure run has then already
been through every other test."""
import math

import numpy as np
import pytest
import torch

from helpers import make_qkv

pytestmark = pytest.mark.gpu


def _args(lib, low, o, scales, dtype, causal, iterations=1):
    q, k, v = low
    B, S, H, D = q.shape
    return lib.fmha_args(q, k, v, o, dtype=dtype, batch=B, heads=H, seqlen_q=S, seqlen_kv=k.shape[1], head_dim=D,
                         softmax_scale=1.0 / math.sqrt(D), causal=causal, q_descale=scales[0], k_descale=scales[1],
                         v_descale=scales[2], iterations=iterations)


@pytest.mark.parametrize("dtype,causal,D", [(0, True, 128), (1, False, 128), (2, False, 128), (1, True, 256), (2, True, 64)])
def test_static_entry_point_matches_the_allocating_one_twice(lib, cuda, dtype, causal, D):
    low, _, scales = make_qkv(dtype, 2, 1024, 1024, 3, D, seed=31 + dtype)
    low = [x.cuda() for x in low]
    want = torch.full((2, 1024, 3, D), -1.0, device="cuda", dtype=torch.float16)
    assert lib.fmha_forward_raw(_args(lib, low, want, scales, dtype, causal)) == 0
    lib.check_device()
    for call in range(2):     # the second call finds the scratch as the first one left it
        got = torch.full_like(want, -2.0)
        assert lib.fmha_forward_static_raw(_args(lib, low, got, scales, dtype, causal)) == 0
        # iterations == 0: wait for the stream and report the status word of the call before
        assert lib.fmha_forward_static_raw(_args(lib, low, got, scales, dtype, causal, iterations=0)) == 0
        # same kernels, same inputs: the tolerance of the other tests (2e-3) is met with zero difference
        diff = (got.float() - want.float()).abs().max().item()
        assert diff <= 2e-3, (call, diff)
        assert torch.equal(got, want), call


def test_static_entry_point_rejects_what_the_other_rejects(lib, cuda):
    low, _, scales = make_qkv(0, 1, 128, 128, 1, 64, seed=1)
    low = [x.cuda() for x in low]
    o = torch.zeros(1, 128, 1, 64, device="cuda", dtype=torch.float16)
    a = _args(lib, low, o, scales, 0, False)
    a.head_dim = 96
    assert lib.fmha_forward_static_raw(a) == 2
    a = _args(lib, low, o, scales, 0, False)
    a.o = None
    assert lib.fmha_forward_static_raw(a) == 1


def test_static_entry_point_allocates_no_device_memory(lib, cuda):
    """The property the entry point is named for: after one warm-up call (which looks the array's address up), the
    free device memory the driver reports does not move across further calls, whatever the shape."""
    shapes = [(0, 2, 1024, 3, 128, True), (2, 1, 2048, 2, 128, False), (1, 1, 512, 2, 64, True), (0, 1, 640, 1, 256, False)]
    prepared = []
    for (dtype, B, S, H, D, causal) in shapes:
        low, _, scales = make_qkv(dtype, B, S, S, H, D, seed=7 + S)
        low = [x.cuda() for x in low]
        o = torch.empty(B, S, H, D, device="cuda", dtype=torch.float16)
        prepared.append((low, o, scales, dtype, causal))
    assert lib.fmha_forward_static_raw(_args(lib, *prepared[0])) == 0       # warm-up: address lookup, module load
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for rep in range(3):
        for pr in prepared:
            assert lib.fmha_forward_static_raw(_args(lib, *pr)) == 0
            assert lib.fmha_forward_static_raw(_args(lib, *pr, iterations=0)) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before


def test_static_entry_point_reports_a_wait_that_gave_up_and_the_next_call_clears_it(lib, cuda):
    """The entry point's own failure path, without a failure: the bounded-wait self-test (one warp, 50 ms, a barrier
    nothing arrives on) reports into the fixed array.  The status query then says DEVICE_WAIT; the allocated status
    block of the other entry point knows nothing of it; the next static call clears the word, computes correctly,
    and the query is clean again."""
    low, _, scales = make_qkv(0, 1, 512, 512, 2, 128, seed=3)
    low = [x.cuda() for x in low]
    want = torch.empty(1, 512, 2, 128, device="cuda", dtype=torch.float16)
    assert lib.fmha_forward_raw(_args(lib, low, want, scales, 0, True)) == 0
    lib.check_device()
    got = torch.full_like(want, -2.0)
    assert lib.fmha_forward_static_raw(_args(lib, low, got, scales, 0, True)) == 0
    assert lib.fmha_forward_static_raw(_args(lib, low, got, scales, 0, True, iterations=0)) == 0
    assert lib.selftest_wait_gives_up_static(0) == 1                        # limits outside 1..1000 ms are refused
    assert lib.selftest_wait_gives_up_static(50) == 0
    assert lib.fmha_forward_static_raw(_args(lib, low, got, scales, 0, True, iterations=0)) == 6    # CFK_ERR_DEVICE_WAIT
    assert lib.device_status() == (0, 0)                                    # the allocated block is a different word
    # the query does not clear the word; the next call does, on its stream, before its launches
    assert lib.fmha_forward_static_raw(_args(lib, low, got, scales, 0, True, iterations=0)) == 6
    got.fill_(-2.0)
    assert lib.fmha_forward_static_raw(_args(lib, low, got, scales, 0, True)) == 0
    assert lib.fmha_forward_static_raw(_args(lib, low, got, scales, 0, True, iterations=0)) == 0
    assert torch.equal(got, want)
