"""include/cfk_compat.hpp compiles and resolves the reference's call shapes: the five-parameter fmhaForwardDevice
(src/fmha-pipeline/fmha_forward.cu:86-93), its legacy three-parameter form (src/fmha/fmha_forward.cu:425-430) next to
it in one translation unit (overload resolution between the two templates), fmhaForwardDeviceLoop (:387-393) and
gemm<TA,TB,TC,Alpha,Beta> (src/cute-gemm-tma-gma/gemm.cu:336-339) for half and for float.  Host-only: nothing runs."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SOURCE = r"""
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include "cfk_compat.hpp"

// every call shape a program written against the reference uses
void legacy(const half* q, const half* k, half* v, half* s, half* d, float* mi, float* sp, cudaStream_t st) {
  fmhaForwardDevice<half, float, 128>(1024, 1024, 8, 2, q, k, v, s, d, mi, sp, 1, 0.1275f, st);
  fmhaForwardDevice<half, float, 64>(1024, 1024, 8, 2, q, k, v, s, d, mi, sp, 1, 0.1275f);
}
void pipelined(const half* q, const half* k, const half* v, half* s, half* o, float* mi, float* sp, cudaStream_t st) {
  fmhaForwardDevice<half, half, float, half, 128>(1024, 1024, 8, 2, q, k, v, s, o, mi, sp, 1, 0.1275f, st);
  fmhaForwardDeviceLoop<half, half, float, half, 256>(1024, 1024, 8, 4, q, k, v, s, o, mi, sp, 1, 2, 0.09f, st);
}
void bf16(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v, __nv_bfloat16* s, half* o,
          float* mi, float* sp) {
  fmhaForwardDevice<__nv_bfloat16, __nv_bfloat16, float, half, 128>(512, 512, 4, 1, q, k, v, s, o, mi, sp, 1, 0.1275f);
}
void gemms(const half* a, const half* b, half* c, const float* fa, const float* fb, float* fc, cudaStream_t st) {
  gemm<half, half, half, float, float>(512, 256, 128, 1.0f, a, 128, b, 128, 0.0f, c, 512);
  gemm<half, half, half, half, half>(512, 256, 128, __float2half(1.0f), a, 128, b, 128, __float2half(0.0f), c, 512,
                                     nullptr, nullptr, 2, st);
  gemm<float, float, float, float, float>(512, 256, 128, 1.0f, fa, 128, fb, 128, 0.0f, fc, 512);
}
int main() { return 0; }
"""


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="nvcc is not on PATH")
def test_compat_header_compiles_every_reference_call_shape(tmp_path):
    src = tmp_path / "compat_shapes.cu"
    src.write_text(SOURCE)
    out = subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-I", os.path.join(ROOT, "include"),
                          "-c", str(src), "-o", str(tmp_path / "compat_shapes.o")], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
