"""GEMM through the C ABI against the CPU oracle (fp32 accumulation of the same 16-bit operands)."""
import numpy as np
import pytest
import torch

from helpers import TORCH_DT

pytestmark = pytest.mark.gpu


def run(lib, oracle, M, N, K, dtype=0, row_major=False, alpha=1.0, beta=0.0, L=1, seed=0):
    g = torch.Generator().manual_seed(seed)
    dt = TORCH_DT[dtype]
    a = (torch.rand(L, M, K, generator=g) * 2 - 1).to(dt)
    b = (torch.rand(L, N, K, generator=g) * 2 - 1).to(dt)
    c0 = (torch.rand(L, M, N, generator=g) * 2 - 1).to(dt)
    c_store = (c0 if row_major else c0.transpose(1, 2)).contiguous().cuda()
    lib.gemm(a.cuda(), b.cuda(), c_store, dtype=dtype, m=M, n=N, k=K, l=L, alpha=alpha, beta=beta,
             c_row_major=row_major)
    lib.check_device()
    got = c_store.float().cpu()
    got = got if row_major else got.transpose(1, 2)
    for l in range(L):
        ref = oracle.gemm(a[l].float().numpy(), b[l].float().numpy(), alpha=alpha, beta=beta,
                          c_in=c0[l].float().numpy() if beta else None)
        # output rounding to the 16-bit type: half an ulp of the result, plus fp32 summation-order noise
        ulp = 2.0 ** (-10 if dtype == 0 else -7)
        tol = ulp * np.maximum(np.abs(ref), 1.0) + 1e-4
        err = np.abs(got[l].numpy() - ref)
        assert (err <= tol).all(), (err.max(), np.abs(ref).max())


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (1024, 1024, 1024), (2048, 768, 4096)])
@pytest.mark.parametrize("row_major", [False, True])
def test_gemm_matches_oracle(lib, oracle, cuda, M, N, K, row_major):
    run(lib, oracle, M, N, K, row_major=row_major)


def test_gemm_alpha_beta_bf16_ragged(lib, oracle, cuda):
    run(lib, oracle, 1000, 776, 264, dtype=1, alpha=0.5, beta=2.0)
    run(lib, oracle, 1000, 776, 264, dtype=0, alpha=-1.25, beta=0.5, row_major=True)


def test_gemm_batched(lib, oracle, cuda):
    run(lib, oracle, 384, 512, 320, L=3)


def test_gemm_linearity_at_full_size(lib, oracle, cuda):
    """8192^3 (the baseline's GEMM config): C(alpha=2) == 2 * C(alpha=1) in fp16 (power-of-two scaling
    commutes with rounding while nothing overflows or is subnormal); a sampled set of entries equals an
    fp64 dot product of the same operands to fp16 rounding; and one full band of 256 rows and one full band of 256
    columns of the result (each crossing every tile of the other direction) equal the oracle's."""
    n = 8192
    torch.manual_seed(1)
    a = (torch.rand(n, n, device="cuda") * 2 - 1).half()
    b = (torch.rand(n, n, device="cuda") * 2 - 1).half()
    c1 = torch.empty(n, n, device="cuda", dtype=torch.float16)
    c2 = torch.empty_like(c1)
    lib.gemm(a, b, c1, dtype=0, m=n, n=n, k=n)
    lib.gemm(a, b, c2, dtype=0, m=n, n=n, k=n, alpha=2.0)
    lib.check_device()
    # exact except where the result is an fp16 subnormal (fixed spacing 2^-24 there)
    assert (c2.float() - 2 * c1.float()).abs().max().item() <= 2.0 ** -23
    idx = torch.randint(0, n, (64, 2))
    for m, nn in idx.tolist():
        ref = float(a[m].double() @ b[nn].double())
        assert abs(float(c1[nn, m]) - ref) <= 2.0 ** -10 * max(1.0, abs(ref)) + 2e-3   # column-major C
    af, bf = a.float().cpu().numpy(), b.float().cpu().numpy()
    m0, n0 = 3 * 256 + 128, 29 * 256                     # the row band straddles two 256-row tiles
    rows = oracle.gemm(af, bf, m_range=(m0, m0 + 256))[m0:m0 + 256]              # [256, N]
    got_rows = c1[:, m0:m0 + 256].float().cpu().numpy().T                         # C is stored [N][M]
    cols = oracle.gemm(bf[n0:n0 + 256], af)                                       # C^T band: [256, M]
    got_cols = c1[n0:n0 + 256, :].float().cpu().numpy()
    for got, ref in ((got_rows, rows), (got_cols, cols)):
        tol = 2.0 ** -10 * np.maximum(np.abs(ref), 1.0) + 2e-3   # fp16 rounding of values up to ~150, fp32 summation order
        assert (np.abs(got - ref) <= tol).all(), float(np.abs(got - ref).max())


def test_gemm_separate_source_matrix_and_integer_operands(lib, oracle, cuda):
    """D = alpha A B + beta C with C read-only and D written elsewhere, on the integer-valued operands of the
    reference's CUTLASS-library GEMM program (src/cutlass-gemm/gemm.cu:268-323): sums of products of small integers
    are exact in fp32, so every output that fp16 can hold must match the float64 result bit for bit."""
    M, N, K = 384, 256, 512
    a = torch.empty(M, K, dtype=torch.float16, device="cuda")
    b = torch.empty(N, K, dtype=torch.float16, device="cuda")
    c = torch.empty(N, M, dtype=torch.float16, device="cuda")       # column-major M x N
    d = torch.full((N, M), -7.0, dtype=torch.float16, device="cuda")
    for t, seed in ((a, 2024), (b, 2023), (c, 2022)):
        lib.fill(t, 0, t.numel(), seed, kind="integers", scale=8.0)
    assert float(a.float().abs().max()) == 8.0 and bool((a.float() == a.float().round()).all())
    c_before = c.clone()
    lib.gemm(a, b, d, dtype=0, m=M, n=N, k=K, alpha=1.0, beta=2.0, c_src=c)
    lib.check_device()
    assert torch.equal(c, c_before)                                  # the source matrix is not written
    ref = a.double().cpu() @ b.double().cpu().T + 2.0 * c.double().cpu().T
    want = ref.to(torch.float16)                                     # one rounding of the exact value
    assert torch.equal(d.cpu().T.contiguous(), want.contiguous())


def test_cutlass_gemm_cli_reports_passed(cuda):
    """The driver with the reference's flags and result lines (src/cutlass-gemm/gemm.cu:182-243, 362-419)."""
    import os
    import subprocess
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "cutlass-kernels_b200", "bin",
                       "cutlass_gemm")
    out = subprocess.run([exe, "--m=512", "--n=384", "--k=256", "--alpha=2", "--beta=0.5", "--iterations=3"],
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "Disposition: Passed" in out.stdout
    assert "Problem Size: 512x384x256" in out.stdout and "GFLOPS:" in out.stdout


@pytest.mark.parametrize("M,N,K,row_major", [(256, 512, 256, False), (1000, 776, 264, True), (2048, 1024, 2048, False)])
def test_gemm_fp32_operands_as_tf32(lib, oracle, cuda, M, N, K, row_major):
    """fp32 A, B, C with tf32 products (the reference's fp32 GEMM type, src/cute-gemm-tma-gma/gemm.cu:355-356):
    exact against the oracle when the operands are already tf32 numbers, and within tf32 operand rounding otherwise."""
    g = torch.Generator().manual_seed(3)
    a = torch.rand(M, K, generator=g) * 2 - 1
    b = torch.rand(N, K, generator=g) * 2 - 1
    c0 = torch.rand(M, N, generator=g) * 2 - 1

    def call(a_, b_):
        c = (c0 if row_major else c0.T).contiguous().cuda()
        lib.gemm(a_.cuda(), b_.cuda(), c, dtype=3, m=M, n=N, k=K, alpha=0.5, beta=2.0, c_row_major=row_major)
        lib.check_device()
        out = c.cpu()
        return (out if row_major else out.T).double()

    def tf32(x):   # keep 10 mantissa bits (truncate the low 13)
        return (x.view(torch.int32) & ~0x1fff).view(torch.float32)

    at, bt = tf32(a.clone()), tf32(b.clone())
    exact = 0.5 * (at.double() @ bt.double().T) + 2.0 * c0.double()
    # only the fp32 accumulation of K exact products remains (the tensor core does not round each add to nearest)
    assert (call(at, bt) - exact).abs().max() <= K * 2.0 ** -23 * float(exact.abs().max())
    full = 0.5 * (a.double() @ b.double().T) + 2.0 * c0.double()
    assert (call(a, b) - full).abs().max() <= 2.0 ** -10 * K ** 0.5
