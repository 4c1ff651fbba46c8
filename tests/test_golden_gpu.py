"""The CUDA path on the committed fixtures (tests/golden/*.npz, made by tests/golden/make_golden.py from the float64
restatement of the reference's checker): the cases whose head dimension the kernels are built for (64 in attention_small.npz, 128 in attention_d128.npz), and
the GEMM case.
Same inputs, bit for bit, as the CPU test of the oracle on these files (test_oracle_cpu.py)."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("tag", ["c1", "causal64", "ragged64"])
@pytest.mark.parametrize("kernel", [0, 2])
def test_fmha_on_the_golden_vectors(lib, cuda, tag, kernel):
    from cfk_b200 import TUNE_FMHA_KERNEL
    data = np.load(os.path.join(GOLDEN, "attention_small.npz"))
    q, k, v = (torch.from_numpy(data[f"{tag}_{n}"]).cuda() for n in "qkv")        # fp16, as stored
    B, Sq, H, D = q.shape
    Skv = k.shape[1]
    o = torch.full((B, Sq, H, D), -1.0, device="cuda", dtype=torch.float16)
    lse = torch.full((B, H, Sq), -1.0, device="cuda", dtype=torch.float32)
    lib.set_tunable(TUNE_FMHA_KERNEL, kernel)
    try:
        lib.fmha_forward(q, k, v, o, dtype=0, batch=B, heads=H, seqlen_q=Sq, seqlen_kv=Skv, head_dim=D,
                         softmax_scale=float(data[f"{tag}_scale"]), causal=bool(data[f"{tag}_causal"]), lse=lse)
        lib.check_device()
    finally:
        lib.set_tunable(TUNE_FMHA_KERNEL, -1)
    assert np.abs(o.float().cpu().numpy() - data[f"{tag}_o"]).max() <= 2e-3        # the stated 16-bit bound
    assert np.abs(lse.cpu().numpy() - data[f"{tag}_lse"]).max() <= 2e-3


@pytest.mark.parametrize("tag", ["causal128", "offset128"])
@pytest.mark.parametrize("kernel,sched", [(0, 0), (0, 1), (2, -1)])
def test_fmha_on_the_golden_vectors_at_head_dimension_128(lib, cuda, tag, kernel, sched):
    """The benchmark's head dimension: the two-tile kernel under both tensor-memory schedules and the persistent one."""
    from cfk_b200 import TUNE_FMHA_KERNEL, TUNE_FMHA_SCHED
    data = np.load(os.path.join(GOLDEN, "attention_d128.npz"))
    q, k, v = (torch.from_numpy(data[f"{tag}_{n}"]).cuda() for n in "qkv")        # fp16, as stored
    B, Sq, H, D = q.shape
    Skv = k.shape[1]
    o = torch.full((B, Sq, H, D), -1.0, device="cuda", dtype=torch.float16)
    lse = torch.full((B, H, Sq), -1.0, device="cuda", dtype=torch.float32)
    lib.set_tunable(TUNE_FMHA_KERNEL, kernel)
    lib.set_tunable(TUNE_FMHA_SCHED, sched)
    try:
        lib.fmha_forward(q, k, v, o, dtype=0, batch=B, heads=H, seqlen_q=Sq, seqlen_kv=Skv, head_dim=D,
                         softmax_scale=float(data[f"{tag}_scale"]), causal=bool(data[f"{tag}_causal"]), lse=lse)
        lib.check_device()
    finally:
        lib.set_tunable(TUNE_FMHA_KERNEL, -1)
        lib.set_tunable(TUNE_FMHA_SCHED, -1)
    assert np.abs(o.float().cpu().numpy() - data[f"{tag}_o"]).max() <= 2e-3
    assert np.abs(lse.cpu().numpy() - data[f"{tag}_lse"]).max() <= 2e-3


def test_gemm_on_the_golden_vectors(lib, cuda):
    g = np.load(os.path.join(GOLDEN, "gemm_small.npz"))
    a, b, c_in = (torch.from_numpy(g[n]).half().cuda() for n in ("a", "b", "c_in"))  # values are fp16-representable
    M, K = a.shape
    N = b.shape[0]
    for row_major in (False, True):
        c = (c_in if row_major else c_in.t()).contiguous().clone()
        lib.gemm(a, b, c, dtype=0, m=M, n=N, k=K, alpha=float(g["alpha"]), beta=float(g["beta"]), c_row_major=row_major)
        lib.check_device()
        got = c.float().cpu().numpy()
        got = got if row_major else got.T
        tol = 2.0 ** -10 * np.maximum(np.abs(g["c"]), 1.0) + 1e-4                    # fp16 rounding of the result
        assert (np.abs(got - g["c"]) <= tol).all()
