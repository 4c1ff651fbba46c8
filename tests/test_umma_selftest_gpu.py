"""Each UMMA operand-descriptor form the kernels depend on, proven on one 128 x n tile against a CPU
product: K-major and MN-major shared-memory operands, A from tensor memory, 16-bit and e4m3 kinds."""
import pytest
import torch

from helpers import TORCH_DT

pytestmark = pytest.mark.gpu

CASES = [
    # n, a_fmt, b_fmt, b_mn_major, a_from_tmem
    (128, 0, 0, 0, 0), (64, 0, 0, 0, 0), (128, 1, 1, 0, 0),
    (64, 0, 0, 1, 0), (128, 0, 0, 1, 0), (128, 1, 1, 1, 0),
    (128, 0, 0, 0, 1), (128, 0, 0, 1, 1), (128, 1, 1, 1, 1), (64, 1, 1, 1, 1),
    (128, 2, 2, 0, 0), (128, 2, 2, 1, 0), (128, 2, 2, 1, 1),
]


@pytest.mark.parametrize("n,a_fmt,b_fmt,mn,ts", CASES)
def test_umma_tile(lib, cuda, n, a_fmt, b_fmt, mn, ts):
    g = torch.Generator().manual_seed(n + 7 * a_fmt + 3 * mn + ts)
    esz = 1 if a_fmt == 2 else 2
    k = 128 // esz
    a = (torch.randn(128, k, generator=g) * 0.5).to(TORCH_DT[a_fmt])
    b = (torch.randn(k, n, generator=g) * 0.5).to(TORCH_DT[b_fmt]) if mn else \
        (torch.randn(n, k, generator=g) * 0.5).to(TORCH_DT[b_fmt])
    ref = a.float() @ (b.float() if mn else b.float().t())
    d = torch.full((128, n), -7.0, device=cuda, dtype=torch.float32)
    assert lib.selftest_umma(a.to(cuda), b.to(cuda), d, n, a_fmt, b_fmt, mn, ts) == 0
    lib.check_device()
    # products of low-precision values summed in fp32: only the summation order differs
    assert (d.cpu() - ref).abs().max().item() <= 1e-4


@pytest.mark.parametrize("dtype,per_mma", [(1, 2 * 128 * 256 * 16), (2, 2 * 128 * 256 * 32)])
def test_umma_peak_probe_reports_its_work_and_finishes(lib, cuda, dtype, per_mma):
    """The tensor-core ceiling probe: the returned flop count is SMs x groups x 4 UMMAs, the launch completes
    with a clean status word, and the rate is that of a tensor core (hundreds of TFLOP/s), not of a stall."""
    import torch
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    lib.umma_peak(dtype, 500)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    flops = lib.umma_peak(dtype, 20000)
    e1.record()
    torch.cuda.synchronize()
    lib.check_device()
    assert flops == float(sms) * 20000 * 4 * per_mma
    tflops = flops / (e0.elapsed_time(e1) * 1e-3) / 1e12
    assert tflops > (600 if dtype == 1 else 1200), tflops
