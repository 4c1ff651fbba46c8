// cfk_fmha_forward_static: the FMHA forward for callers that must not allocate device memory.
//
// The ordinary entry point keeps its scratch (the status block that the kernels' bounded waits report
// into) in memory it obtains with cudaMalloc the first time a device is used, which also synchronises
// that device.  Some callers cannot afford either: serving loops that have handed all of HBM to their
// own pool (so even a 256-byte cudaMalloc can fail or fragment), latency-bound loops that cannot take a
// device-wide synchronisation, and hosts that forbid allocation after start-up.  For them the same kernels run here with the scratch
// in a fixed array that is part of the library image.  No counterpart in the reference.
#include <cmath>
#include <cstring>
#include <mutex>

#include "fmha_launch.h"
#include "host_util.h"

namespace cfk {

// The scratch itself: 256 bytes per GPU that loads the library, held until the process exits.  Word 0 is
// the status word; profiling builds keep their cycle counters in the words after it.  In host code this
// name is only a stand-in for the symbol, never a device address: the address comes from
// cudaGetSymbolAddress below.
constexpr int kStaticScratchInts = 64;
static __device__ __align__(256) int g_fmha_static_scratch[kStaticScratchInts];

// Scratch one call needs, in ints: the status block the kernels address through FmhaParams::status.
#ifdef CFK_FMHA_PROFILE
constexpr int kFmhaScratchInts = 8 + 2 * 12;   // status word, padding, twelve 64-bit cycle counters
#else
constexpr int kFmhaScratchInts = 1;
#endif

static std::mutex g_static_mu;
static int* g_static_addr[64] = {nullptr};

// Device address of the array on the current device; resolved once per device, with that device current.
static int* static_scratch_for_current_device(int* err) {
  int dev = -1;
  if (note_cuda(cudaGetDevice(&dev), "cudaGetDevice") != cudaSuccess || dev < 0 || dev >= 64) {
    *err = CFK_ERR_NO_DRIVER;
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (!g_static_addr[dev]) {
    void* ptr = nullptr;
    if (note_cuda(cudaGetSymbolAddress(&ptr, g_fmha_static_scratch), "cudaGetSymbolAddress(static scratch)") !=
            cudaSuccess || !ptr) {
      *err = CFK_ERR_NO_DRIVER;
      return nullptr;
    }
    g_static_addr[dev] = static_cast<int*>(ptr);
  }
  return g_static_addr[dev];
}

static bool packed_or_valid(const int64_t in[3], int64_t out[3], int S, int H, int D, int esz) {
  if (in[0] == 0 && in[1] == 0 && in[2] == 0) {
    out[2] = D; out[1] = (int64_t)H * D; out[0] = (int64_t)S * H * D;
  } else {
    out[0] = in[0]; out[1] = in[1]; out[2] = in[2];
  }
  for (int i = 0; i < 3; ++i)
    if (out[i] <= 0 || (out[i] * esz) % 16 != 0) return false;
  return true;
}

}  // namespace cfk

using namespace cfk;

// Same arguments, checks, kernels and results as cfk_fmha_forward; differences:
//   * nothing is allocated: no cudaMalloc / cudaFree / allocating library call, here or in what it calls;
//   * the first call on a device resolves the address of the static array (cudaGetSymbolAddress); make
//     that first call before any stream capture begins;
//   * the array is shared by every call on that device and keeps the previous call's contents, so the
//     status word is cleared on `stream` before the launches; two calls whose kernels overlap on the GPU
//     (different streams) race on it and may hide or misattribute a wait that gave up;
//   * a call whose scratch need exceeds the array (kStaticScratchInts ints; only special builds need more
//     than one word) is refused with CFK_ERR_TOO_LARGE and nothing is launched;
//   * iterations == 0 launches nothing: it waits for `stream` and returns CFK_ERR_DEVICE_WAIT if the status
//     word left by the preceding call is non-zero (cfk_device_status only sees the allocated block).
extern "C" int cfk_fmha_forward_static(const cfk_fmha_args* a, cfk_stream_t stream) {
  if (!a || !a->q || !a->k || !a->v || !a->o) return CFK_ERR_INVALID_ARG;
  if (a->batch <= 0 || a->heads <= 0 || a->seqlen_q <= 0 || a->seqlen_kv <= 0 || a->iterations < 0)
    return CFK_ERR_INVALID_ARG;
  if (a->batch > 65535 || a->heads > 65535) return CFK_ERR_INVALID_ARG;
  if (!(a->softmax_scale > 0.f) || !std::isfinite(a->softmax_scale)) return CFK_ERR_INVALID_ARG;
  if (a->dtype != CFK_FP16 && a->dtype != CFK_BF16 && a->dtype != CFK_E4M3) return CFK_ERR_INVALID_ARG;
  if (a->out_dtype != CFK_FP16 && a->out_dtype != CFK_BF16) return CFK_ERR_INVALID_ARG;
  if (a->head_dim != 64 && a->head_dim != 128) return CFK_ERR_UNSUPPORTED;
  if (a->v_fp16) return CFK_ERR_UNSUPPORTED;   // the hybrid e4m3 / fp16 mode goes through cfk_fmha_forward
  if (a->dtype == CFK_E4M3 && a->head_dim != 128) return CFK_ERR_UNSUPPORTED;
  if (a->causal && a->seqlen_kv < a->seqlen_q) return CFK_ERR_UNSUPPORTED;
  if (a->p_split_keys < -1) return CFK_ERR_INVALID_ARG;
  const bool fp8 = a->dtype == CFK_E4M3;
  const float qd = fp8 ? a->q_descale : (a->q_descale == 0.f ? 1.f : a->q_descale);
  const float kd = fp8 ? a->k_descale : (a->k_descale == 0.f ? 1.f : a->k_descale);
  const float vd = fp8 ? a->v_descale : (a->v_descale == 0.f ? 1.f : a->v_descale);
  if (!(qd > 0.f) || !(kd > 0.f) || !(vd > 0.f)) return CFK_ERR_INVALID_ARG;
  if (((uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v | (uintptr_t)a->o) & 15u) return CFK_ERR_INVALID_ARG;
  const int esz = dtype_size(a->dtype);
  int64_t qs[3], ks[3], vs[3], os[3];
  if (!packed_or_valid(a->q_stride, qs, a->seqlen_q, a->heads, a->head_dim, esz)) return CFK_ERR_INVALID_ARG;
  if (!packed_or_valid(a->k_stride, ks, a->seqlen_kv, a->heads, a->head_dim, esz)) return CFK_ERR_INVALID_ARG;
  if (!packed_or_valid(a->v_stride, vs, a->seqlen_kv, a->heads, a->head_dim, esz)) return CFK_ERR_INVALID_ARG;
  if (!packed_or_valid(a->o_stride, os, a->seqlen_q, a->heads, a->head_dim, 2)) return CFK_ERR_INVALID_ARG;

  if (kFmhaScratchInts > kStaticScratchInts) {
    (void)note_cuda(cudaErrorInvalidValue, "cfk_fmha_forward_static: this build needs more scratch than the static "
                                          "array holds (kFmhaScratchInts > kStaticScratchInts)");
    return CFK_ERR_TOO_LARGE;
  }

  int err = CFK_OK;
  int* status = static_scratch_for_current_device(&err);
  if (!status) return err;
  const cudaStream_t st = (cudaStream_t)stream;

  if (a->iterations == 0) {   // query: what did the preceding call leave in the status word?
    if (note_cuda(cudaStreamSynchronize(st), "cudaStreamSynchronize") != cudaSuccess) return CFK_ERR_LAUNCH;
    int code = 0;
    if (note_cuda(cudaMemcpy(&code, status, sizeof(int), cudaMemcpyDeviceToHost), "cudaMemcpy(static status)") !=
        cudaSuccess)
      return CFK_ERR_LAUNCH;
    return code == 0 ? CFK_OK : CFK_ERR_DEVICE_WAIT;
  }

  FmhaLaunch L;
  std::memset(&L, 0, sizeof(L));
  int rc;
  if ((rc = encode_bshd(&L.tm_q, a->dtype, a->q, a->batch, a->seqlen_q, a->heads, a->head_dim, qs[0], qs[1], qs[2], 128)))
    return rc;
  if ((rc = encode_bshd(&L.tm_k, a->dtype, a->k, a->batch, a->seqlen_kv, a->heads, a->head_dim, ks[0], ks[1], ks[2], 128)))
    return rc;
  if ((rc = encode_bshd(&L.tm_v, a->dtype, a->v, a->batch, a->seqlen_kv, a->heads, a->head_dim, vs[0], vs[1], vs[2], 128)))
    return rc;
  if ((rc = encode_bshd(&L.tm_o, a->out_dtype, a->o, a->batch, a->seqlen_q, a->heads, a->head_dim, os[0], os[1], os[2], 128)))
    return rc;

  FmhaParams& p = L.p;
  p.B = a->batch; p.H = a->heads; p.Sq = a->seqlen_q; p.Skv = a->seqlen_kv;
  p.causal = a->causal ? 1 : 0;
  p.out_bf16 = a->out_dtype == CFK_BF16;
  p.nqblk = (a->seqlen_q + 255) / 256;
  if ((long long)p.nqblk * a->heads * a->batch > 0x7fffffffLL) return CFK_ERR_UNSUPPORTED;
  p.split_keys = a->dtype == CFK_BF16 ? (a->p_split_keys < 0 ? 1024 : a->p_split_keys) : 0;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f * qd * kd;
  p.out_scale = vd;
  p.lse = a->lse; p.mi = a->mi; p.sprime = a->sprime;
  p.s_dump = a->s_dump; p.s_dump_bf16 = a->dtype == CFK_BF16;
  p.status = status;
  L.iterations = a->iterations;
  L.stream = st;
  L.exp_emu = cfk_get_tunable(CFK_TUNE_FMHA_EXP_EMU);
  if (L.exp_emu < 0) L.exp_emu = fp8 ? 2 : 1;
  const long long kv_bytes = 2LL * a->seqlen_kv * a->head_dim * esz;
  long long grp = a->causal ? ((long long)cfk_get_tunable(CFK_TUNE_FMHA_GROUP_MB) << 20) / kv_bytes : 1;
  const long long bh = (long long)a->batch * a->heads;
  p.group = (int)(grp < 1 ? 1 : (grp > bh ? bh : grp));

  // The status word must start at zero: a launch that finds it set does nothing.
  if (note_cuda(cudaMemsetAsync(status, 0, sizeof(int) * kFmhaScratchInts, st), "cudaMemsetAsync(static status)") !=
      cudaSuccess)
    return CFK_ERR_LAUNCH;
  return fmha_dispatch(a->dtype, a->dtype, a->head_dim, L);
}
