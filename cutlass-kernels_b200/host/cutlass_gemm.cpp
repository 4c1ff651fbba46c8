// cutlass_gemm — command-line driver shaped like the reference's CUTLASS-library GEMM program
// (src/cutlass-gemm/gemm.cu:182-243 options, :295-323 operands, :362-419 run loop): D = alpha * A * B + beta * C with
// A row-major M x K, B column-major K x N, C and D column-major M x N, fp16, integer-valued random operands in
// [-8, 8], one verified launch ("Disposition: Passed"), then `--iterations` timed launches and the three result
// lines.  The reference accumulates in fp16 and compares bit-exactly with a device reference GEMM that rounds the
// same way; this library accumulates in fp32, so the check here is every element against a float64 evaluation of
// the same operands, to half a unit in the last place of the fp16 result (exact for sums that fp16 can hold).
//
//   cutlass_gemm [--m=5120] [--n=4096] [--k=4096] [--alpha=1] [--beta=0] [--iterations=1000] [--help]
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "cfk_b200.h"

#define CUDA_OK(x)                                                                         \
  do {                                                                                     \
    cudaError_t e_ = (x);                                                                  \
    if (e_ != cudaSuccess) {                                                               \
      std::fprintf(stderr, "%s failed: %s\n", #x, cudaGetErrorString(e_));                 \
      return 1;                                                                            \
    }                                                                                      \
  } while (0)

static bool flag(int argc, char** argv, const char* name, std::string* value) {
  const std::string key = std::string("--") + name;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    if (a == key) { if (value) value->clear(); return true; }
    if (a.rfind(key + "=", 0) == 0) { if (value) *value = a.substr(key.size() + 1); return true; }
  }
  return false;
}

static void usage() {
  std::printf("cutlass_gemm\n\n  fp16 GEMM D = alpha * A * B + beta * C on sm_100a (tcgen05, CTA pairs).\n\nOptions:\n\n"
              "  --help                      print this text and exit\n\n"
              "  --m=<int>                   rows of A and of C, D (default 5120)\n"
              "  --n=<int>                   columns of B and of C, D (default 4096)\n"
              "  --k=<int>                   columns of A, rows of B: the reduction length (default 4096)\n"
              "  --alpha=<f32>               factor of the product A * B (default 1)\n"
              "  --beta=<f32>                factor of the source matrix C (default 0)\n\n"
              "  --iterations=<int>          timed launches after the verified one (default 1000)\n\n");
}

static int download_f32(const void* dev, int dtype, size_t n, std::vector<float>* out) {
  float* tmp = nullptr;
  CUDA_OK(cudaMalloc(&tmp, n * sizeof(float)));
  if (cfk_convert(dev, dtype, tmp, CFK_FP32, (int64_t)n, 1.f, nullptr)) return 1;
  out->resize(n);
  CUDA_OK(cudaMemcpy(out->data(), tmp, n * sizeof(float), cudaMemcpyDeviceToHost));
  cudaFree(tmp);
  return 0;
}

int main(int argc, char** argv) {
  int m = 5120, n = 4096, k = 4096, iterations = 1000;     // defaults of gemm.cu:190-195
  float alpha = 1.f, beta = 0.f;
  std::string v;
  if (flag(argc, argv, "help", nullptr)) { usage(); return 0; }
  if (flag(argc, argv, "m", &v)) m = std::atoi(v.c_str());
  if (flag(argc, argv, "n", &v)) n = std::atoi(v.c_str());
  if (flag(argc, argv, "k", &v)) k = std::atoi(v.c_str());
  if (flag(argc, argv, "alpha", &v)) alpha = (float)std::atof(v.c_str());
  if (flag(argc, argv, "beta", &v)) beta = (float)std::atof(v.c_str());
  if (flag(argc, argv, "iterations", &v)) iterations = std::atoi(v.c_str());
  if (m <= 0 || n <= 0 || k <= 0) { std::fprintf(stderr, "m, n, k must be positive\n"); return 1; }

  const size_t na = (size_t)m * k, nb = (size_t)n * k, nc = (size_t)m * n;
  __half *a, *b, *c, *d;
  CUDA_OK(cudaMalloc(&a, na * 2));
  CUDA_OK(cudaMalloc(&b, nb * 2));
  CUDA_OK(cudaMalloc(&c, nc * 2));
  CUDA_OK(cudaMalloc(&d, nc * 2));
  const uint64_t seed = 1;                                   // gemm.cu:300-302: seed + 2023 / 2022 / 2021
  if (cfk_fill(a, CFK_FP16, (int64_t)na, seed + 2023, 0, 3, 8.f, 0.f, nullptr)) return 1;
  if (cfk_fill(b, CFK_FP16, (int64_t)nb, seed + 2022, 0, 3, 8.f, 0.f, nullptr)) return 1;
  if (cfk_fill(c, CFK_FP16, (int64_t)nc, seed + 2021, 0, 3, 8.f, 0.f, nullptr)) return 1;

  cfk_gemm_args g;
  std::memset(&g, 0, sizeof(g));
  g.dtype = CFK_FP16; g.m = m; g.n = n; g.k = k; g.l = 1;
  g.a = a; g.b = b; g.c = d; g.c_src = c;
  g.alpha = alpha; g.beta = beta; g.c_row_major = 0; g.iterations = 1;
  int rc = cfk_gemm(&g, nullptr);                            // correctness / warm-up launch
  if (rc) { std::fprintf(stderr, "cfk_gemm: status %d (%s)\n", rc, cfk_last_cuda_error()); return 1; }
  CUDA_OK(cudaDeviceSynchronize());

  // verification: every element when the problem is small, else a seeded sample of 16384 entries
  std::vector<float> ha, hb, hc, hd;
  if (download_f32(a, CFK_FP16, na, &ha) || download_f32(b, CFK_FP16, nb, &hb) || download_f32(c, CFK_FP16, nc, &hc) ||
      download_f32(d, CFK_FP16, nc, &hd))
    return 1;
  const bool full = (double)m * n * k <= 2.2e9;
  const size_t checks = full ? nc : 16384;
  size_t bad = 0;
  unsigned long long s = 2024;
  for (size_t t = 0; t < checks; ++t) {
    size_t i, j;
    if (full) { i = t % m; j = t / m; }
    else {
      s = s * 6364136223846793005ull + 1442695040888963407ull; i = (size_t)((s >> 33) % (unsigned)m);
      s = s * 6364136223846793005ull + 1442695040888963407ull; j = (size_t)((s >> 33) % (unsigned)n);
    }
    double acc = 0;
    const float* ar = &ha[i * k];
    const float* br = &hb[j * k];
    for (int kk = 0; kk < k; ++kk) acc += (double)ar[kk] * br[kk];
    const double want = (double)alpha * acc + (double)beta * hc[j * m + i];
    const double got = hd[j * m + i];
    // half an fp16 unit in the last place at the magnitude of the result (fp16 spacing is 2^(e-10))
    const double mag = std::fabs(want);
    const double half_ulp = mag < 6.1e-5 ? 2.98e-8 : std::ldexp(1.0, std::ilogb(mag) - 11);
    const bool inf_ok = mag > 65504.0 && std::isinf(got);
    if (!(std::fabs(got - want) <= half_ulp * 1.0001 || inf_ok)) {
      if (bad < 5) std::printf("  D[%zu,%zu]: got %g want %g\n", i, j, got, want);
      ++bad;
    }
  }
  const bool passed = bad == 0;
  std::printf("  Disposition: %s\n", passed ? "Passed" : "Failed");

  if (iterations > 0) {
    cudaEvent_t e0, e1;
    CUDA_OK(cudaEventCreate(&e0));
    CUDA_OK(cudaEventCreate(&e1));
    g.iterations = iterations;
    CUDA_OK(cudaEventRecord(e0, 0));
    rc = cfk_gemm(&g, nullptr);
    CUDA_OK(cudaEventRecord(e1, 0));
    CUDA_OK(cudaDeviceSynchronize());
    if (rc) { std::fprintf(stderr, "cfk_gemm: status %d\n", rc); return 1; }
    float ms_total = 0.f;
    CUDA_OK(cudaEventElapsedTime(&ms_total, e0, e1));
    const double ms = (double)ms_total / iterations;
    std::printf("  Problem Size: %dx%dx%d\n", m, n, k);
    std::printf("  Avg runtime: %g ms\n", ms);
    std::printf("  GFLOPS: %g\n", 2.0 * m * n * (double)k * 1e-9 / (ms * 1e-3));
  }
  int code = 0;
  if (cfk_device_status(&code) != CFK_OK) { std::printf("  device status word %d\n", code); return 1; }
  cudaFree(a); cudaFree(b); cudaFree(c); cudaFree(d);
  return passed ? 0 : 2;
}
