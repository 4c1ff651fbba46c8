// cfk_compat.hpp — the reference's host launcher names on top of the C ABI (cfk_b200.h).
//
// A program written against the reference calls function templates that live inside its .cu files:
//   fmhaForwardDevice<PrecType, Gemm2Type, SoftType, OutputType, HEADDIM>(SEQLEN, KEYLEN, NUMHEADS, BATCH,
//       Q, K, V, S, O, miOut, sPrimeOut, iterations, scale, stream)        src/fmha-pipeline/fmha_forward.cu:86-93
//   fmhaForwardDeviceLoop<...>(..., nStreams, scale, stream)               src/fmha-pipeline/fmha_forward.cu:387-419
//   fmhaForwardDevice<PrecType, AccumType, HEADDIM>(...)                   src/fmha/fmha_forward.cu:425-430
//   gemm<TA, TB, TC, Alpha, Beta>(m, n, k, alpha, A, ldA, B, ldB, beta, C, ldC, A_out, B_out, L, stream)
//                                                                          src/cute-gemm-tma-gma/gemm.cu:336-339
// This header offers the same names, argument order and meaning, forwarding to libcfk_b200.so.  Element
// types are recognised through cfk::dtype_of<T>: specialise it for your own 16-bit / 8-bit wrappers (the
// reference uses cutlass::half_t and cutlass::float_e4m3_t); __half, __nv_bfloat16 and __nv_fp8_e4m3 are
// known when their CUDA headers were included first.
//
// Behavioural notes for a maintainer switching over:
//   * `scale` keeps the reference's meaning: softmax scale already multiplied by log2(e)
//     (fmha_forward.cu:452-454).  The shim divides it out again for the C ABI.
//   * the S debug matrix is ignored (may be nullptr); miOut / sPrimeOut are filled when non-null with the
//     reference's semantics (log2-domain row max, un-inverted row sum).
//   * functions return void like the reference; the status of the last call on this thread is available
//     from cfk::last_status() and a non-zero status is reported on stderr (the reference prints and
//     carries on as well, include/utils/cuda_launch.hpp:15-18).  Nothing calls exit().
//   * fmhaForwardDeviceLoop splits the batch over `nStreams` streams created per call and destroys them
//     after enqueueing (the reference leaks them, fmha_forward.cu:403-404).
//   * gemm: ldA / ldB / ldC and A_out / B_out are accepted and ignored exactly as in the reference
//     (gemm.cu:366-389 recomputes packed strides); alpha and beta are honoured, accumulation is fp32.
#pragma once
#include <cuda_runtime.h>

#include <cstdio>
#include <type_traits>

#include "cfk_b200.h"

namespace cfk {

template <typename T, typename Enable = void>
struct dtype_of {
  // Fallback by size: 2-byte types are taken as fp16, 1-byte types as e4m3 (the reference's two
  // precisions, fmha_forward.cu:744-791).  Specialise for bf16 wrappers.
  static constexpr int value = sizeof(T) == 2 ? CFK_FP16 : (sizeof(T) == 1 ? CFK_E4M3 : CFK_FP32);
};
#if defined(__CUDA_BF16_TYPES_EXIST__) || defined(__CUDA_BF16_H__)
template <>
struct dtype_of<__nv_bfloat16> { static constexpr int value = CFK_BF16; };
#endif

inline int& last_status_ref() {
  static thread_local int s = CFK_OK;
  return s;
}
inline int last_status() { return last_status_ref(); }
inline void note_status(const char* who, int rc) {
  last_status_ref() = rc;
  if (rc != CFK_OK) std::fprintf(stderr, "%s: cfk status %d (%s)\n", who, rc, cfk_last_cuda_error());
}

// Extra knobs the reference's signature has no room for; they apply to subsequent launcher calls made
// by this thread.
struct LaunchOptions {
  bool causal = false;
  float q_descale = 1.f, k_descale = 1.f, v_descale = 1.f;
  float* lse = nullptr;
  int out_dtype = CFK_FP16;
  int p_split_keys = -1;
  bool dump_scores = false;   // write the S argument like a COPYOUTMM0 build of the reference (16-bit inputs only)
};
inline LaunchOptions& launch_options() {
  static thread_local LaunchOptions o;
  return o;
}

}  // namespace cfk

template <typename PrecType, typename Gemm2Type, typename SoftType, typename OutputType, int HEADDIM>
void fmhaForwardDevice(int SEQLEN, int KEYLEN, int NUMHEADS, int BATCH, PrecType const* Q, PrecType const* K,
                       Gemm2Type const* V, PrecType* S, OutputType* O, SoftType* miOut, SoftType* sPrimeOut,
                       int iterations, float scale, cudaStream_t stream = 0) {
  static_assert(std::is_same<SoftType, float>::value, "softmax statistics are fp32");
  static_assert(sizeof(OutputType) == 2, "the output is a 16-bit type");
  // Gemm2Type differs from PrecType only in the reference's FP8 mode without GEMM2FP8: Q, K e4m3 and V half
  static_assert(sizeof(PrecType) == sizeof(Gemm2Type) || (sizeof(PrecType) == 1 && sizeof(Gemm2Type) == 2),
                "V has the type of Q and K, or is a 16-bit float while Q and K are e4m3");
  const cfk::LaunchOptions& opt = cfk::launch_options();
  cfk_fmha_args a{};
  a.dtype = cfk::dtype_of<PrecType>::value;
  a.out_dtype = std::is_same<OutputType, PrecType>::value && a.dtype == CFK_BF16 ? CFK_BF16 : opt.out_dtype;
  a.p_split_keys = opt.p_split_keys;
  a.batch = BATCH; a.heads = NUMHEADS; a.seqlen_q = SEQLEN; a.seqlen_kv = KEYLEN; a.head_dim = HEADDIM;
  a.q = Q; a.k = K; a.v = V; a.o = O;
  a.lse = opt.lse; a.mi = miOut; a.sprime = sPrimeOut;
  a.softmax_scale = scale / 1.4426950408889634f;   // the reference hands over scale * log2(e)
  a.causal = opt.causal ? 1 : 0;
  a.q_descale = opt.q_descale; a.k_descale = opt.k_descale; a.v_descale = opt.v_descale;
  a.iterations = iterations;
  a.s_dump = (opt.dump_scores && sizeof(PrecType) == 2) ? S : nullptr;   // else S is ignored (may be nullptr)
  a.v_fp16 = sizeof(PrecType) == 1 && sizeof(Gemm2Type) == 2;
  cfk::note_status("fmhaForwardDevice", cfk_fmha_forward(&a, stream));
}

// Legacy three-parameter form (src/fmha/fmha_forward.cu:425-430): fp16 in, fp16 out.
template <typename PrecType, typename AccumType, int HEADDIM>
void fmhaForwardDevice(int SEQLEN, int KEYLEN, int NUMHEADS, int BATCH, PrecType const* Q, PrecType const* K,
                       PrecType* V, PrecType* S, PrecType* D, AccumType* miOut, AccumType* sPrimeOut, int iterations,
                       float scale, cudaStream_t stream = 0) {
  fmhaForwardDevice<PrecType, PrecType, AccumType, PrecType, HEADDIM>(SEQLEN, KEYLEN, NUMHEADS, BATCH, Q, K, V, S, D,
                                                                      miOut, sPrimeOut, iterations, scale, stream);
}

template <typename PrecType, typename Gemm2Type, typename SoftType, typename OutputType, int HEADDIM>
void fmhaForwardDeviceLoop(int SEQLEN, int KEYLEN, int NUMHEADS, int BATCH, PrecType const* Q, PrecType const* K,
                           Gemm2Type const* V, PrecType* S, OutputType* O, SoftType* miOut, SoftType* sPrimeOut,
                           int iterations, int nStreams, float scale, cudaStream_t stream = 0) {
  if (nStreams <= 1 || BATCH % nStreams != 0) {
    fmhaForwardDevice<PrecType, Gemm2Type, SoftType, OutputType, HEADDIM>(SEQLEN, KEYLEN, NUMHEADS, BATCH, Q, K, V, S, O,
                                                                          miOut, sPrimeOut, iterations, scale, stream);
    return;
  }
  // Batch is the outermost dimension, so a batch slice is a plain pointer offset (fmha_forward.cu:406-411), the
  // debug score tensor S included (offsetS there).  The slice streams are created like the reference's
  // (cudaStreamCreate, fmha_forward.cu:403-404), so work on them is ordered against the legacy default stream; in
  // addition every slice stream waits on an event recorded on `stream` and `stream` waits on each slice's end, so
  // that events or kernels a caller puts on `stream` around this call bracket all slices whatever `stream` is.
  const int b = BATCH / nStreams;
  const size_t q_el = (size_t)b * SEQLEN * NUMHEADS * HEADDIM, kv_el = (size_t)b * KEYLEN * NUMHEADS * HEADDIM;
  const size_t st_el = (size_t)b * NUMHEADS * SEQLEN;
  const size_t s_el = (size_t)b * NUMHEADS * SEQLEN * KEYLEN;
  cudaEvent_t fork = nullptr;
  if (cudaEventCreateWithFlags(&fork, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventRecord(fork, stream) != cudaSuccess) {
    if (fork) cudaEventDestroy(fork);
    cfk::note_status("fmhaForwardDeviceLoop", CFK_ERR_LAUNCH);
    return;
  }
  for (int i = 0; i < nStreams; ++i) {
    cudaStream_t s = nullptr;
    cudaEvent_t join = nullptr;
    if (cudaStreamCreate(&s) != cudaSuccess || cudaEventCreateWithFlags(&join, cudaEventDisableTiming) != cudaSuccess ||
        cudaStreamWaitEvent(s, fork, 0) != cudaSuccess) {
      if (s) cudaStreamDestroy(s);
      if (join) cudaEventDestroy(join);
      cfk::note_status("fmhaForwardDeviceLoop", CFK_ERR_LAUNCH);
      break;
    }
    fmhaForwardDevice<PrecType, Gemm2Type, SoftType, OutputType, HEADDIM>(
        SEQLEN, KEYLEN, NUMHEADS, b, Q + i * q_el, K + i * kv_el, V + i * kv_el, S ? S + i * s_el : nullptr,
        O + i * q_el, miOut ? miOut + i * st_el : nullptr, sPrimeOut ? sPrimeOut + i * st_el : nullptr, iterations,
        scale, s);
    if (cudaEventRecord(join, s) != cudaSuccess || cudaStreamWaitEvent(stream, join, 0) != cudaSuccess)
      cfk::note_status("fmhaForwardDeviceLoop", CFK_ERR_LAUNCH);
    cudaEventDestroy(join);   // released once the event has completed
    cudaStreamDestroy(s);     // destruction is deferred until the enqueued work has finished
  }
  cudaEventDestroy(fork);
}

template <typename TA, typename TB, typename TC, typename Alpha, typename Beta>
void gemm(int m, int n, int k, Alpha alpha, TA const* A, int ldA, TB const* B, int ldB, Beta beta, TC* C, int ldC,
          TA* A_out = nullptr, TB* B_out = nullptr, int L = 1, cudaStream_t stream = 0) {
  (void)ldA; (void)ldB; (void)ldC; (void)A_out; (void)B_out;
  static_assert(sizeof(TA) == sizeof(TB) && sizeof(TA) == sizeof(TC) && (sizeof(TA) == 2 || sizeof(TA) == 4),
                "16-bit operands and output, or fp32 operands and output (products in tf32)");
  cfk_gemm_args g{};
  g.dtype = cfk::dtype_of<TA>::value;
  g.m = m; g.n = n; g.k = k; g.l = L;
  g.a = A; g.b = B; g.c = C;
  g.alpha = static_cast<float>(alpha);
  g.beta = static_cast<float>(beta);
  g.c_row_major = 0;      // the reference's C is column-major (gemm.cu:388-389)
  g.iterations = 1;
  cfk::note_status("gemm", cfk_gemm(&g, stream));
}
