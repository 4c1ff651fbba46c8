"""The failure path of the kernels' bounded waits, exercised without faulting anything: a self-test warp waits, with
a short limit, on a barrier that nothing arrives on.  The wait gives up, the status word says which one, launches
enqueued while the word is set do nothing, and after the word has been read the library works as before.  (The
reference's kernels wait on their barriers without a limit; a lost arrival there hangs the GPU.)"""
import math
import time

import numpy as np
import pytest
import torch

from helpers import make_qkv, run_fmha

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_leaves_the_library_usable(lib, oracle, cuda):
    lib.check_device()                                   # starts clean
    assert lib.selftest_wait_gives_up(0) == 1 and lib.selftest_wait_gives_up(5000) == 1   # limits outside 1..1000 ms
    t0 = time.monotonic()
    assert lib.selftest_wait_gives_up(50) == 0
    # an FMHA call enqueued behind it finds the status word set and must not touch its output
    low, f32, scales = make_qkv(0, 1, 256, 256, 2, 128, seed=1)
    q, k, v = (x.cuda() for x in low)
    o = torch.full((1, 256, 2, 128), -1.0, device="cuda", dtype=torch.float16)
    lib.fmha_forward(q, k, v, o, dtype=0, batch=1, heads=2, seqlen_q=256, seqlen_kv=256, head_dim=128,
                     softmax_scale=1.0 / math.sqrt(128), causal=False)
    rc, code = lib.device_status()
    elapsed = time.monotonic() - t0
    assert rc == 6 and code == 901                       # CFK_ERR_DEVICE_WAIT, the self-test's wait
    assert 0.04 <= elapsed < 2.0                         # it waited for its limit, not for the kernels' 2 s
    assert bool((o == -1.0).all())
    # the word was cleared by the read; the same call now runs and is correct
    assert lib.device_status() == (0, 0)
    got, _ = run_fmha(lib, low, scales, 0, False, want_stats=False)
    ref = oracle.attention(f32[0], f32[1], f32[2], 1.0 / math.sqrt(128), False)["o"]
    assert np.abs(got - ref).max() <= 2e-3
