"""The command-line drivers, run as the reference's programs are run: same flags, same result lines
(src/fmha-pipeline/fmha_forward.cu:687-760 for the options, :572-597 and :628-677 for the lines;
src/cute-gemm-tma-gma/gemm.cu:656-691 for the positional GEMM arguments)."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

BIN = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "cutlass-kernels_b200", "bin")


def run(exe, *args):
    out = subprocess.run([os.path.join(BIN, exe), *args], capture_output=True, text=True, timeout=300)
    return out.returncode, out.stdout + out.stderr


@pytest.mark.parametrize("prec,head", [(1, 64), (1, 128), (1, 256), (2, 64), (2, 128), (2, 256)])
def test_fmha_forward_cli_reference_check(cuda, prec, head):
    # e4m3 is held to the reference's own bound (0.001 % of entries off, :638-639) at the sequence length its
    # sweep uses; rows of 1024 keys carry the 3-bit rounding of P into too many single outputs for that bound
    seq = 1024 if prec == 1 else 4096
    rc, text = run("fmha_forward", "--batch-size=2", "--dim-size=512", f"--head-size={head}", f"--seq-length={seq}",
                   "--iterations=3", f"--prec-type={prec}", "--reference-check=true")
    assert rc == 0, text
    assert "CUTE_FMHA:" in text and "Gflop/s" in text
    assert "gemm-check-2: Passed" in text, text
    assert f"M = {seq}\nN = {seq}\nK = {head}\n" in text


def test_fmha_forward_cli_verify_all_and_streams(cuda):
    """--verify-all adds the score, row-maximum and row-sum checks of the reference's debug builds
    (fmha_forward.cu:640-677); --num-cuda-streams splits the batch as fmhaForwardDeviceLoop does (:387-419)."""
    rc, text = run("fmha_forward", "--batch-size=4", "--dim-size=256", "--head-size=128", "--seq-length=512",
                   "--iterations=2", "--prec-type=1", "--verify-all=true", "--num-cuda-streams=2")
    assert rc == 0, text
    for line in ("gemm-check-1: Passed", "max-check: Passed", "sum-check: Passed", "gemm-check-2: Passed"):
        assert line in text, text


def test_fmha_forward_cli_times_the_work_of_every_stream(cuda):
    """The CUTE_FMHA line is taken from events on stream 0 around fmhaForwardDeviceLoop; with the batch split over two
    streams those events must still bracket all the work (the reference's cudaStreamCreate streams order themselves
    against stream 0), not just the time to enqueue it."""
    import re
    ms = {}
    for streams in (1, 2):
        rc, text = run("fmha_forward", "--batch-size=4", "--dim-size=2048", "--head-size=128", "--seq-length=4096",
                       "--iterations=5", "--prec-type=1", f"--num-cuda-streams={streams}")
        assert rc == 0, text
        ms[streams] = float(re.search(r"CUTE_FMHA:.*\(\s*([0-9.]+)\)ms", text).group(1))
    assert ms[1] > 0.2                          # 2.7e11 flop cannot take less on any B200
    assert 0.5 * ms[1] <= ms[2] <= 2.0 * ms[1], ms


def test_fmha_forward_cli_hybrid_fp8_and_causal(cuda):
    rc, text = run("fmha_forward", "--batch-size=1", "--dim-size=256", "--head-size=128", "--seq-length=1024",
                   "--iterations=2", "--prec-type=2", "--hybrid-fp8=true", "--reference-check=true")
    assert rc == 0 and "gemm-check-2: Passed" in text, text
    rc, text = run("fmha_forward", "--batch-size=1", "--dim-size=256", "--head-size=128", "--seq-length=1024",
                   "--iterations=2", "--prec-type=1", "--causal=true", "--reference-check=true")
    assert rc == 0 and "gemm-check-2: Passed" in text, text


def test_fmha_forward_cli_rejects_an_unsupported_head_size(cuda):
    rc, text = run("fmha_forward", "--head-size=96", "--seq-length=256", "--dim-size=96")
    assert rc != 0 and "not supported" in text


@pytest.mark.parametrize("type_,extra", [(1, ()), (3, ()), (3, ("2", "5", "1.5", "0.5")), (4, ())])
def test_gemm_cli_types(cuda, type_, extra):
    """type 1 = fp32 operands as tf32 (the reference's default), 3 = fp16; L, iterations, alpha, beta follow."""
    rc, text = run("gemm", str(type_), "512", "384", "256", *extra)
    assert rc == 0, text
    assert "CUTE_GEMM:" in text and "sampled check: passed" in text, text


def test_gemm_cli_type_2_runs_nothing_and_others_are_refused(cuda):
    rc, text = run("gemm", "2", "512", "384", "256")
    assert rc == 0 and "CUTE_GEMM" not in text
    rc, text = run("gemm", "7")
    assert rc != 0 and "invalid type value" in text
