// fmha_forward — command-line driver with the reference program's flags and output lines
// (src/fmha-pipeline/fmha_forward.cu:687-733 for the flags, :572-597 for the timing recipe and the
// "CUTE_FMHA" line, :611-682 for the optional check).  It goes through the reference-named launcher of
// include/cfk_compat.hpp, so it doubles as a usage example of the drop-in surface.
//
//   --batch-size=4 --dim-size=2048 --head-size=64 --seq-length=4096 --iterations=20
//   --prec-type=1|2|3 (1 = fp16, 2 = e4m3 [default, as in the reference], 3 = bf16 [addition])
//   --reference-check=true|false  --num-cuda-streams=1  --causal=true|false [addition]  --seed=3080
//
// The check is the reference's own recipe: inputs up-cast to float, unfused attention on the host,
// element-wise rule abs > 5e-3 AND rel > 10 % (include/utils/random.hpp:64-89).  To keep it quick it
// verifies the first --check-heads (default 2) heads of batch 0 and says so.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "cfk_compat.hpp"

struct e4m3_t { unsigned char bits; };   // 1-byte element: cfk::dtype_of falls back to e4m3 for it

struct Options {
  int batch = 4, dim = 2048, head = 64, seq = 4096, iterations = 20, prec = 2, streams = 1, check_heads = 2;
  bool check = false, causal = false, help = false, verify_all = false, hybrid = false;
  unsigned long long seed = 3080;
};

static bool flag(const char* arg, const char* name, std::string* val) {
  const size_t n = std::strlen(name);
  if (std::strncmp(arg, "--", 2) || std::strncmp(arg + 2, name, n)) return false;
  if (arg[2 + n] == '=') { *val = arg + 3 + n; return true; }
  if (arg[2 + n] == 0) { *val = "true"; return true; }
  return false;
}

static Options parse(int argc, char** argv) {
  Options o;
  for (int i = 1; i < argc; ++i) {
    std::string v;
    if (flag(argv[i], "help", &v)) o.help = true;
    else if (flag(argv[i], "batch-size", &v)) o.batch = std::atoi(v.c_str());
    else if (flag(argv[i], "dim-size", &v)) o.dim = std::atoi(v.c_str());
    else if (flag(argv[i], "head-size", &v)) o.head = std::atoi(v.c_str());
    else if (flag(argv[i], "seq-length", &v)) o.seq = std::atoi(v.c_str());
    else if (flag(argv[i], "iterations", &v)) o.iterations = std::atoi(v.c_str());
    else if (flag(argv[i], "prec-type", &v)) o.prec = std::atoi(v.c_str());
    else if (flag(argv[i], "num-cuda-streams", &v)) o.streams = std::atoi(v.c_str());
    else if (flag(argv[i], "check-heads", &v)) o.check_heads = std::atoi(v.c_str());
    else if (flag(argv[i], "seed", &v)) o.seed = std::strtoull(v.c_str(), nullptr, 10);
    else if (flag(argv[i], "reference-check", &v)) o.check = (v == "true" || v == "1");
    else if (flag(argv[i], "causal", &v)) o.causal = (v == "true" || v == "1");
    else if (flag(argv[i], "verify-all", &v)) o.verify_all = o.check = (v == "true" || v == "1");
    else if (flag(argv[i], "hybrid-fp8", &v)) o.hybrid = (v == "true" || v == "1");
    else std::fprintf(stderr, "ignoring unknown argument %s\n", argv[i]);
  }
  return o;
}

#define CUDA_OK(x)                                                                         \
  do {                                                                                     \
    cudaError_t e_ = (x);                                                                  \
    if (e_ != cudaSuccess) {                                                               \
      std::fprintf(stderr, "%s failed: %s\n", #x, cudaGetErrorString(e_));                 \
      return 1;                                                                            \
    }                                                                                      \
  } while (0)

// Host attention on float inputs for one (batch 0, head h): the reference's unfused recipe
// (include/utils/fmha_cutlass.hpp:275-314) with an optional lower-triangular mask.
// Optional extras for the verify-all run: raw (unscaled, unmasked) scores of the visible keys, row maxima of the
// scaled scores (natural-log domain) and inverse row sums, the three things the reference's COPYOUTMM0 / COPYOUTMI
// builds compare (src/fmha-pipeline/fmha_forward.cu:640-672).
static void host_attention_head(const std::vector<float>& q, const std::vector<float>& k, const std::vector<float>& v,
                                int S, int H, int D, int h, float scale, bool causal, std::vector<float>* out,
                                std::vector<float>* raw = nullptr, std::vector<float>* row_max = nullptr,
                                std::vector<float>* inv_sum = nullptr) {
  out->assign((size_t)S * D, 0.f);
  if (raw) raw->assign((size_t)S * S, 0.f);
  if (row_max) row_max->assign(S, 0.f);
  if (inv_sum) inv_sum->assign(S, 0.f);
#pragma omp parallel
  {
    std::vector<float> sc(S);
#pragma omp for schedule(dynamic, 16)
    for (int i = 0; i < S; ++i) {
      const int nv = causal ? i + 1 : S;
      float mx = -INFINITY;
      for (int j = 0; j < nv; ++j) {
        float acc = 0.f;
        const float* qi = &q[((size_t)i * H + h) * D];
        const float* kj = &k[((size_t)j * H + h) * D];
        for (int d = 0; d < D; ++d) acc += qi[d] * kj[d];
        sc[j] = acc * scale;
        if (raw) (*raw)[(size_t)i * S + j] = acc;
        mx = std::fmax(mx, sc[j]);
      }
      float sum = 0.f;
      for (int j = 0; j < nv; ++j) { sc[j] = std::exp(sc[j] - mx); sum += sc[j]; }
      const float inv = 1.f / sum;
      if (row_max) (*row_max)[i] = mx;
      if (inv_sum) (*inv_sum)[i] = inv;
      float* o = &(*out)[(size_t)i * D];
      for (int j = 0; j < nv; ++j) {
        const float pj = sc[j] * inv;
        const float* vj = &v[((size_t)j * H + h) * D];
        for (int d = 0; d < D; ++d) o[d] += pj * vj[d];
      }
    }
  }
}

// T: element type of Q and K; TV: of V (T, or __half in the hybrid e4m3 mode)
template <typename T, int HEADDIM, typename TV = T>
static int run(const Options& o, int dtype) {
  const int dtype_v = sizeof(TV) == sizeof(T) ? dtype : CFK_FP16;
  const int B = o.batch, S = o.seq, D = HEADDIM, H = o.dim / D;
  std::printf("M = %d\nN = %d\nK = %d\nQBLK = 128\nKBLK = 128\nL = %d : %d\n", S, S, D, B, H);
  const size_t n = (size_t)B * S * H * D;
  T *q, *k;
  TV* v;
  __half* out;
  float *mi, *sprime;
  CUDA_OK(cudaMalloc(&q, n * sizeof(T)));
  CUDA_OK(cudaMalloc(&k, n * sizeof(T)));
  CUDA_OK(cudaMalloc(&v, n * sizeof(TV)));
  CUDA_OK(cudaMalloc(&out, n * sizeof(__half)));
  CUDA_OK(cudaMalloc(&mi, (size_t)B * H * S * sizeof(float)));
  CUDA_OK(cudaMalloc(&sprime, (size_t)B * H * S * sizeof(float)));
  // Gaussian inputs, seeds base+1/+2/+3 as the reference (fmha_forward.cu:479,498-500); e4m3 inputs are
  // quantised with a per-tensor scale amax/448 (the reference casts N(0,1) straight to e4m3).
  float descale[3] = {1.f, 1.f, 1.f};
  void* ptr[3] = {q, k, v};
  const int pdt[3] = {dtype, dtype, dtype_v};
  for (int i = 0; i < 3; ++i) {
    if (pdt[i] == CFK_E4M3) {
      descale[i] = 6.0f / 448.0f;   // N(0,1) draws of this generator stay within +-6
      if (cfk_fill(ptr[i], pdt[i], (int64_t)n, o.seed + 1 + i, 0, 0, 1.0f / descale[i], 0.f, nullptr)) return 1;
    } else if (cfk_fill(ptr[i], pdt[i], (int64_t)n, o.seed + 1 + i, 0, 0, 1.f, 0.f, nullptr)) {
      return 1;
    }
  }
  if (cfk_fill(out, CFK_FP16, (int64_t)n, 0, 0, 2, 1.f, -1.f, nullptr)) return 1;   // outputs pre-filled with -1

  cfk::LaunchOptions& lo = cfk::launch_options();
  lo.causal = o.causal;
  lo.q_descale = descale[0]; lo.k_descale = descale[1]; lo.v_descale = descale[2];
  const float scale = 1.4426950408889634f / std::sqrt((float)D);   // log2(e)/sqrt(D), fmha_forward.cu:452-454

  // warm-up (10 launches), then `iterations` back-to-back launches between two events
  fmhaForwardDeviceLoop<T, TV, float, __half, HEADDIM>(S, S, H, B, q, k, v, (T*)nullptr, out, mi, sprime, 10, o.streams,
                                                     scale, 0);
  CUDA_OK(cudaDeviceSynchronize());
  cudaEvent_t e0, e1;
  CUDA_OK(cudaEventCreate(&e0));
  CUDA_OK(cudaEventCreate(&e1));
  CUDA_OK(cudaEventRecord(e0, 0));
  fmhaForwardDeviceLoop<T, TV, float, __half, HEADDIM>(S, S, H, B, q, k, v, (T*)nullptr, out, mi, sprime, o.iterations,
                                                     o.streams, scale, 0);
  CUDA_OK(cudaEventRecord(e1, 0));
  CUDA_OK(cudaDeviceSynchronize());
  float ms_total = 0.f;
  CUDA_OK(cudaEventElapsedTime(&ms_total, e0, e1));
  int dev_code = 0;
  const int rc = cfk_device_status(&dev_code);
  if (cfk::last_status() != CFK_OK || rc != CFK_OK) {
    std::printf("launch failed: status %d, device word %d\n", cfk::last_status() ? cfk::last_status() : rc, dev_code);
    return 1;
  }
  const double ms = ms_total / (o.iterations > 0 ? o.iterations : 1);
  double flops = 4.0 * B * H * (double)S * S * D;
  if (o.causal) flops *= 0.5;
  std::printf("CUTE_FMHA:     [%6.1f]Gflop/s  (%6.4f)ms\n", flops / (ms * 1e-3) / 1e9, ms);

  int ret = 0;
  if (o.check) {
    const int heads = o.check_heads < H ? o.check_heads : H;
    const size_t nb = (size_t)S * H * D;   // batch 0
    std::vector<float> hf[3];
    float* tmp;
    CUDA_OK(cudaMalloc(&tmp, nb * sizeof(float)));
    for (int i = 0; i < 3; ++i) {
      hf[i].resize(nb);
      if (cfk_convert(ptr[i], pdt[i], tmp, CFK_FP32, (int64_t)nb, descale[i], nullptr)) return 1;
      CUDA_OK(cudaMemcpy(hf[i].data(), tmp, nb * sizeof(float), cudaMemcpyDeviceToHost));
    }
    std::vector<float> ho(nb);
    if (cfk_convert(out, CFK_FP16, tmp, CFK_FP32, (int64_t)nb, 1.f, nullptr)) return 1;
    CUDA_OK(cudaMemcpy(ho.data(), tmp, nb * sizeof(float), cudaMemcpyDeviceToHost));
    cudaFree(tmp);
    // verify-all: one more launch that also writes the raw scores (the S argument of the launcher)
    const bool dump = o.verify_all && dtype != CFK_E4M3;
    std::vector<float> hs, hmi, hsp;
    if (o.verify_all) {
      T* sdump = nullptr;
      if (dump) {
        CUDA_OK(cudaMalloc(&sdump, (size_t)B * H * S * S * sizeof(T)));
        CUDA_OK(cudaMemset(sdump, 0, (size_t)B * H * S * S * sizeof(T)));
        lo.dump_scores = true;
        fmhaForwardDevice<T, TV, float, __half, HEADDIM>(S, S, H, B, q, k, v, sdump, out, mi, sprime, 1, scale, 0);
        lo.dump_scores = false;
        CUDA_OK(cudaDeviceSynchronize());
        if (cfk::last_status() != CFK_OK) return 1;
        const size_t ns = (size_t)heads * S * S;   // batch 0, first heads
        float* tmp2;
        CUDA_OK(cudaMalloc(&tmp2, ns * sizeof(float)));
        if (cfk_convert(sdump, dtype, tmp2, CFK_FP32, (int64_t)ns, 1.f, nullptr)) return 1;
        hs.resize(ns);
        CUDA_OK(cudaMemcpy(hs.data(), tmp2, ns * sizeof(float), cudaMemcpyDeviceToHost));
        cudaFree(tmp2);
        cudaFree(sdump);
      }
      hmi.resize((size_t)H * S);
      hsp.resize((size_t)H * S);
      CUDA_OK(cudaMemcpy(hmi.data(), mi, hmi.size() * sizeof(float), cudaMemcpyDeviceToHost));
      CUDA_OK(cudaMemcpy(hsp.data(), sprime, hsp.size() * sizeof(float), cudaMemcpyDeviceToHost));
    }
    auto off = [](float got, float want) {   // the reference's element rule, include/utils/random.hpp:64-89
      const float ad = std::fabs(got - want), rel = ad / std::fabs(want + 1e-5f);
      return std::isnan(want) || std::isnan(ad) || std::isinf(ad) || (ad > 5e-3f && rel > 1e-1f);
    };
    long long bad = 0, total = 0, bad_s = 0, bad_max = 0, bad_sum = 0;
    double maxabs = 0;
    for (int h = 0; h < heads; ++h) {
      std::vector<float> ref, raw, rmax, rinv;
      host_attention_head(hf[0], hf[1], hf[2], S, H, D, h, 1.f / std::sqrt((float)D), o.causal, &ref,
                          dump ? &raw : nullptr, o.verify_all ? &rmax : nullptr, o.verify_all ? &rinv : nullptr);
      if (o.verify_all) {
        for (int i = 0; i < S; ++i) {
          // mi is in the log2 domain and sprime is not inverted (fmha_forward.cu:655-672)
          if (off(hmi[(size_t)h * S + i] * 0.69314718f, rmax[i])) ++bad_max;
          if (off(1.f / hsp[(size_t)h * S + i], rinv[i])) ++bad_sum;
          if (dump) {
            const int nv = o.causal ? i + 1 : S;
            for (int j = 0; j < nv; ++j)
              if (off(hs[((size_t)h * S + i) * S + j], raw[(size_t)i * S + j])) ++bad_s;
          }
        }
      }
      for (int i = 0; i < S; ++i)
        for (int d = 0; d < D; ++d) {
          const float got = ho[((size_t)i * H + h) * D + d], want = ref[(size_t)i * D + d];
          const float ad = std::fabs(got - want), rel = ad / std::fabs(want + 1e-5f);
          if (std::isnan(want) || std::isnan(ad) || std::isinf(ad) || (ad > 5e-3f && rel > 1e-1f)) ++bad;
          if (ad > maxabs) maxabs = ad;
          ++total;
        }
    }
    const double pct = 100.0 * (double)bad / (double)total;
    if (o.verify_all) {
      if (dump) std::printf("gemm-check-1: %s\n", bad_s == 0 ? "Passed" : "Failed");
      else std::printf("gemm-check-1: not run (scores are dumped for 16-bit inputs only)\n");
      std::printf("max-check: %s\n", bad_max == 0 ? "Passed" : "Failed");
      std::printf("sum-check: %s\n", bad_sum == 0 ? "Passed" : "Failed");
      if (bad_s || bad_max || bad_sum) ret = 2;
    }
    std::printf("Error (percentage) : %f\n", pct);
    std::printf("max abs diff %g over %d head(s) of batch 0\n", maxabs, heads);
    const double allowed = dtype == CFK_E4M3 ? 0.001 : 0.0001;   // fmha_forward.cu:638-639
    std::printf("gemm-check-2: %s\n", pct <= allowed ? "Passed" : "Failed");
    if (pct > allowed) ret = 2;
  }
  cudaFree(q); cudaFree(k); cudaFree(v); cudaFree(out); cudaFree(mi); cudaFree(sprime);
  return ret;
}

int main(int argc, char** argv) {
  const Options o = parse(argc, argv);
  if (o.help) {
    std::printf("fmha_forward --batch-size=<int> --dim-size=<int> --head-size=<64|128|256> --seq-length=<int>\n"
                "             --iterations=<int> --prec-type=<1 fp16|2 e4m3|3 bf16> --num-cuda-streams=<int>\n"
                "             --reference-check=<bool> --verify-all=<bool> --causal=<bool> --check-heads=<int> --seed=<int>\n"
                "             --hybrid-fp8=<bool> (prec-type 2 only: V in fp16)\n");
    return 0;
  }
  if (o.head != 64 && o.head != 128 && o.head != 256) {
    std::printf("head size %d is not supported (64, 128 or 256)\n", o.head);   // the reference exits here too, :758-760
    return 1;
  }
  if (o.dim % o.head) { std::printf("dim-size must be a multiple of head-size\n"); return 1; }
  if (o.prec == 1)
    return o.head == 64 ? run<__half, 64>(o, CFK_FP16) : o.head == 128 ? run<__half, 128>(o, CFK_FP16) : run<__half, 256>(o, CFK_FP16);
  if (o.prec == 3)
    return o.head == 64    ? run<__nv_bfloat16, 64>(o, CFK_BF16)
           : o.head == 128 ? run<__nv_bfloat16, 128>(o, CFK_BF16)
                           : run<__nv_bfloat16, 256>(o, CFK_BF16);
  if (o.prec == 2) {
    if (o.hybrid) {   // Q, K e4m3 and V fp16: the reference's FP8 mode when it is built without GEMM2FP8
      if (o.head == 256) { std::printf("hybrid-fp8 runs at head sizes 64 and 128\n"); return 1; }
      return o.head == 64 ? run<e4m3_t, 64, __half>(o, CFK_E4M3) : run<e4m3_t, 128, __half>(o, CFK_E4M3);
    }
    return o.head == 64 ? run<e4m3_t, 64>(o, CFK_E4M3)
           : o.head == 128 ? run<e4m3_t, 128>(o, CFK_E4M3) : run<e4m3_t, 256>(o, CFK_E4M3);
  }
  std::printf("unknown prec-type %d\n", o.prec);
  return 1;
}
