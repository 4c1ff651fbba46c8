// C-ABI entry points that are not a kernel family of their own: argument validation and dispatch for
// cfk_fmha_forward, fills / conversions, status handling.  Declarations: include/cfk_b200.h.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "fmha_launch.h"
#include "host_util.h"

namespace cfk {

// ------------------------------------------------------------------------------------------------
// error text, status block, descriptor encoding
// ------------------------------------------------------------------------------------------------
static thread_local std::string g_last_error;

cudaError_t note_cuda(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
    (void)cudaGetLastError();  // clear the sticky-less error so later calls are judged on their own
  }
  return e;
}

static std::mutex g_mu;
static int* g_status_block[64] = {nullptr};

int* device_status_block(int* err) {
  int dev = -1;
  if (note_cuda(cudaGetDevice(&dev), "cudaGetDevice") != cudaSuccess || dev < 0 || dev >= 64) {
    if (err) *err = CFK_ERR_NO_DRIVER;
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status_block[dev]) {
    int* p = nullptr;
    if (note_cuda(cudaMalloc(&p, 256), "cudaMalloc(status block)") != cudaSuccess) {
      if (err) *err = CFK_ERR_NO_DRIVER;
      return nullptr;
    }
    if (note_cuda(cudaMemset(p, 0, 256), "cudaMemset(status block)") != cudaSuccess) {
      if (err) *err = CFK_ERR_NO_DRIVER;
      return nullptr;
    }
    g_status_block[dev] = p;
  }
  return g_status_block[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (note_cuda(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres),
                  "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)") == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

int encode_tiled(CUtensorMap* map, int dtype, int rank, const void* base, const uint64_t* dims,
                 const uint64_t* strides_bytes, const uint32_t* box, int swizzle_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return CFK_ERR_NO_DRIVER;
  CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  if (dtype == CFK_BF16) dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  else if (dtype == CFK_E4M3) dt = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  else if (dtype == CFK_FP32) dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t gd[5];
  cuuint64_t gs[4];
  cuuint32_t bx[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) { gd[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) gs[i] = strides_bytes[i];
  CUresult r = fn(map, dt, (cuuint32_t)rank, const_cast<void*>(base), gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                  : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_error = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r);
    return CFK_ERR_DESCRIPTOR;
  }
  return CFK_OK;
}

int encode_bshd(CUtensorMap* map, int dtype, const void* base, int batch, int seq, int heads, int d, int64_t sb,
                int64_t ss, int64_t sh, int box_rows, int box_spans) {
  const int esz = dtype_size(dtype);
  const int span_bytes = d * esz < 128 ? d * esz : 128;   // rows shorter than 128 bytes (e4m3, d = 64) are one 64-byte span
  const uint64_t span = (uint64_t)span_bytes / esz;       // elements per span
  const uint64_t nspan = (uint64_t)d * esz / span_bytes;
  const uint64_t dims[5] = {span, (uint64_t)seq, nspan, (uint64_t)heads, (uint64_t)batch};
  const uint64_t strides[4] = {(uint64_t)ss * esz, (uint64_t)span_bytes, (uint64_t)sh * esz, (uint64_t)sb * esz};
  const uint32_t box[5] = {(uint32_t)span, (uint32_t)box_rows, (uint32_t)(box_spans > 0 ? box_spans : (int)nspan), 1, 1};
  return encode_tiled(map, dtype, 5, base, dims, strides, box, span_bytes);
}

// ------------------------------------------------------------------------------------------------
// fills and conversions
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}
__device__ __forceinline__ float unit_open(uint32_t x) { return ((float)(x >> 8) + 0.5f) * (1.0f / 16777216.0f); }

__device__ __forceinline__ void store_as(void* dst, int dtype, int64_t i, float v) {
  if (dtype == CFK_FP16) reinterpret_cast<__half*>(dst)[i] = __float2half_rn(v);
  else if (dtype == CFK_BF16) reinterpret_cast<__nv_bfloat16*>(dst)[i] = __float2bfloat16_rn(v);
  else if (dtype == CFK_E4M3)
    reinterpret_cast<uint8_t*>(dst)[i] = (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
  else reinterpret_cast<float*>(dst)[i] = v;
}
__device__ __forceinline__ float load_as(const void* src, int dtype, int64_t i) {
  if (dtype == CFK_FP16) return __half2float(reinterpret_cast<const __half*>(src)[i]);
  if (dtype == CFK_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(src)[i]);
  if (dtype == CFK_E4M3) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(reinterpret_cast<const uint8_t*>(src)[i], __NV_E4M3);
    return __half2float(__half(h));
  }
  return reinterpret_cast<const float*>(src)[i];
}

__global__ void fill_kernel(void* dst, int dtype, int64_t n, uint64_t seed, int64_t first, int kind, float scale,
                            float value) {
  const uint64_t key = mix64(seed);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float v = value;
    if (kind != 2) {
      const uint64_t r = mix64(key ^ (uint64_t)(first + i));
      const float u1 = unit_open((uint32_t)r), u2 = unit_open((uint32_t)(r >> 32));
      v = (kind == 0) ? sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2) : 2.0f * u1 - 1.0f;
      if (kind == 3) v = rintf(v * scale);   // integers in [-scale, scale]
    }
    store_as(dst, dtype, i, kind == 3 ? v : v * scale);
  }
}

__global__ void convert_kernel(const void* src, int sdt, void* dst, int ddt, int64_t n, float scale) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    store_as(dst, ddt, i, load_as(src, sdt, i) * scale);
}

// Tunables (process-wide).  Defaults are the measured best on B200.
// EXP_EMU -1 = by type: 1 of 4 pairs for 16-bit inputs, 2 of 4 for e4m3 (measured best on B200).
// SCHED -1 = by type (see fmha_prepare).
static const int kTunableDefault[CFK_TUNE_COUNT] = {-1, 64, 0, 0, -1};
static std::atomic<int> g_tunable[CFK_TUNE_COUNT] = {{-1}, {64}, {0}, {0}, {-1}};

// The knobs can also be set from the environment (CFK_TUNE_FMHA_EXP_EMU, CFK_TUNE_FMHA_GROUP_MB, CFK_TUNE_FMHA_KERNEL,
// CFK_TUNE_FMHA_GRID, CFK_TUNE_FMHA_SCHED), read once before the first FMHA call: the command-line drivers have no flags for them.
static void tunables_from_env() {
  static std::once_flag once;
  std::call_once(once, [] {
    static const char* const names[CFK_TUNE_COUNT] = {"CFK_TUNE_FMHA_EXP_EMU", "CFK_TUNE_FMHA_GROUP_MB",
                                                      "CFK_TUNE_FMHA_KERNEL", "CFK_TUNE_FMHA_GRID",
                                                      "CFK_TUNE_FMHA_SCHED"};
    for (int i = 0; i < CFK_TUNE_COUNT; ++i) {
      const char* v = std::getenv(names[i]);
      if (v && *v) (void)cfk_set_tunable(i, std::atoi(v));
    }
  });
}

static bool valid_dtype(int dt) { return dt >= CFK_FP16 && dt <= CFK_FP32; }

}  // namespace cfk

using namespace cfk;

extern "C" int cfk_version(void) { return 100; }

extern "C" int cfk_set_tunable(int which, int value) {
  if (which < 0 || which >= CFK_TUNE_COUNT) return CFK_ERR_INVALID_ARG;
  if (value < 0) value = kTunableDefault[which];
  if (which == CFK_TUNE_FMHA_EXP_EMU && value > 3) return CFK_ERR_INVALID_ARG;
  if (which == CFK_TUNE_FMHA_GROUP_MB && (value < 1 || value > 1024)) return CFK_ERR_INVALID_ARG;
  if (which == CFK_TUNE_FMHA_KERNEL && value > 2) return CFK_ERR_INVALID_ARG;
  if (which == CFK_TUNE_FMHA_SCHED && value > 1) return CFK_ERR_INVALID_ARG;
  g_tunable[which].store(value);
  return CFK_OK;
}

extern "C" int cfk_get_tunable(int which) {
  if (which < 0 || which >= CFK_TUNE_COUNT) return -1;
  return g_tunable[which].load();
}

extern "C" const char* cfk_last_cuda_error(void) { return g_last_error.c_str(); }

extern "C" int cfk_device_status(int* code_out) {
  int err = CFK_OK;
  int* blk = device_status_block(&err);
  if (!blk) return err;
  if (note_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize") != cudaSuccess) return CFK_ERR_LAUNCH;
  int code = 0;
  if (note_cuda(cudaMemcpy(&code, blk, sizeof(int), cudaMemcpyDeviceToHost), "cudaMemcpy(status)") != cudaSuccess)
    return CFK_ERR_LAUNCH;
  if (code != 0) (void)note_cuda(cudaMemset(blk, 0, sizeof(int)), "cudaMemset(status)");
  if (code_out) *code_out = code;
  return code == 0 ? CFK_OK : CFK_ERR_DEVICE_WAIT;
}

extern "C" int cfk_fill(void* dst, int dtype, int64_t n, uint64_t seed, int64_t first_index, int kind, float scale,
                        float value, cfk_stream_t stream) {
  if (!dst || n < 0 || !valid_dtype(dtype) || kind < 0 || kind > 3) return CFK_ERR_INVALID_ARG;
  if (n == 0) return CFK_OK;
  const int threads = 256;
  const int64_t want = (n + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  fill_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>(dst, dtype, n, seed, first_index, kind, scale, value);
  return note_cuda(cudaGetLastError(), "fill launch") == cudaSuccess ? CFK_OK : CFK_ERR_LAUNCH;
}

extern "C" int cfk_convert(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n, float scale,
                           cfk_stream_t stream) {
  if (!src || !dst || n < 0 || !valid_dtype(src_dtype) || !valid_dtype(dst_dtype)) return CFK_ERR_INVALID_ARG;
  if (n == 0) return CFK_OK;
  const int threads = 256;
  const int64_t want = (n + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  convert_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>(src, src_dtype, dst, dst_dtype, n, scale);
  return note_cuda(cudaGetLastError(), "convert launch") == cudaSuccess ? CFK_OK : CFK_ERR_LAUNCH;
}

// ------------------------------------------------------------------------------------------------
// FMHA forward: validation + dispatch
// ------------------------------------------------------------------------------------------------
static bool resolve_strides(const int64_t in[3], int64_t out[3], int S, int H, int D, int esz) {
  if (in[0] == 0 && in[1] == 0 && in[2] == 0) {
    out[2] = D;
    out[1] = (int64_t)H * D;
    out[0] = (int64_t)S * H * D;
  } else {
    out[0] = in[0]; out[1] = in[1]; out[2] = in[2];
  }
  for (int i = 0; i < 3; ++i)
    if (out[i] <= 0 || (out[i] * esz) % 16 != 0) return false;
  return true;
}

// Argument checks, TMA descriptors, kernel parameters and kernel choice of one FMHA call: everything of the launch
// except the status pointer and the stream, which the two entry points supply (allocated block / static array).
// *p_dtype receives the type P is rounded to (and V is stored in).
int cfk::fmha_prepare(const cfk_fmha_args* a, FmhaLaunch* out, int* p_dtype) {
  if (!a || !a->q || !a->k || !a->v || !a->o) return CFK_ERR_INVALID_ARG;
  if (a->batch <= 0 || a->heads <= 0 || a->seqlen_q <= 0 || a->seqlen_kv <= 0 || a->iterations < 0)
    return CFK_ERR_INVALID_ARG;
  if (a->batch > 65535 || a->heads > 65535) return CFK_ERR_INVALID_ARG;
  if (!(a->softmax_scale > 0.f) || !std::isfinite(a->softmax_scale)) return CFK_ERR_INVALID_ARG;
  if (a->dtype != CFK_FP16 && a->dtype != CFK_BF16 && a->dtype != CFK_E4M3) return CFK_ERR_INVALID_ARG;
  if (a->out_dtype != CFK_FP16 && a->out_dtype != CFK_BF16) return CFK_ERR_INVALID_ARG;
  if (a->head_dim != 64 && a->head_dim != 128 && a->head_dim != 256) return CFK_ERR_UNSUPPORTED;
  if (a->causal && a->seqlen_kv < a->seqlen_q) return CFK_ERR_UNSUPPORTED;
  if (a->p_split_keys < -1) return CFK_ERR_INVALID_ARG;
  if (a->v_fp16 && (a->dtype != CFK_E4M3 || a->head_dim == 256)) return CFK_ERR_UNSUPPORTED;
  const int vdt = a->v_fp16 ? CFK_FP16 : a->dtype;   // element type of V, and the type P is rounded to
  const int pdt = vdt;
  const float qd = a->dtype == CFK_E4M3 ? a->q_descale : (a->q_descale == 0.f ? 1.f : a->q_descale);
  const float kd = a->dtype == CFK_E4M3 ? a->k_descale : (a->k_descale == 0.f ? 1.f : a->k_descale);
  const float vd = a->dtype == CFK_E4M3 ? a->v_descale : (a->v_descale == 0.f ? 1.f : a->v_descale);
  if (!(qd > 0.f) || !(kd > 0.f) || !(vd > 0.f)) return CFK_ERR_INVALID_ARG;
  const uintptr_t align_or = (uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v | (uintptr_t)a->o;
  if (align_or & 15u) return CFK_ERR_INVALID_ARG;

  const int esz = dtype_size(a->dtype);
  int64_t qs[3], ks[3], vs[3], os[3];
  if (!resolve_strides(a->q_stride, qs, a->seqlen_q, a->heads, a->head_dim, esz)) return CFK_ERR_INVALID_ARG;
  if (!resolve_strides(a->k_stride, ks, a->seqlen_kv, a->heads, a->head_dim, esz)) return CFK_ERR_INVALID_ARG;
  if (!resolve_strides(a->v_stride, vs, a->seqlen_kv, a->heads, a->head_dim, dtype_size(vdt))) return CFK_ERR_INVALID_ARG;
  if (!resolve_strides(a->o_stride, os, a->seqlen_q, a->heads, a->head_dim, 2)) return CFK_ERR_INVALID_ARG;

  tunables_from_env();
  FmhaLaunch& L = *out;
  std::memset(&L, 0, sizeof(L));
  int rc;
  if ((rc = encode_bshd(&L.tm_q, a->dtype, a->q, a->batch, a->seqlen_q, a->heads, a->head_dim, qs[0], qs[1], qs[2], 128)))
    return rc;
  // head dimension 256: K and V tiles travel as two halves of 128 columns (two 128-byte spans) each
  const int kv_spans = a->head_dim == 256 ? esz : 0;   // 128 columns = esz spans of 128 bytes
  if ((rc = encode_bshd(&L.tm_k, a->dtype, a->k, a->batch, a->seqlen_kv, a->heads, a->head_dim, ks[0], ks[1], ks[2], 128, kv_spans)))
    return rc;
  if ((rc = encode_bshd(&L.tm_v, vdt, a->v, a->batch, a->seqlen_kv, a->heads, a->head_dim, vs[0], vs[1], vs[2], 128, kv_spans)))
    return rc;
  if ((rc = encode_bshd(&L.tm_o, a->out_dtype, a->o, a->batch, a->seqlen_q, a->heads, a->head_dim, os[0], os[1], os[2], 128)))
    return rc;

  L.variant = g_tunable[CFK_TUNE_FMHA_KERNEL].load();
  if (L.variant == 1 && (a->dtype == CFK_E4M3 || a->head_dim != 128)) L.variant = 0;
  if (a->head_dim == 256) L.variant = 0;
  L.grid_ctas = g_tunable[CFK_TUNE_FMHA_GRID].load();
  if (L.variant == 1) {   // CTA-pair kernel: each CTA loads 64 keys of a K tile and one 64-column span of a V tile
    if ((rc = encode_bshd(&L.tm_k_half, a->dtype, a->k, a->batch, a->seqlen_kv, a->heads, a->head_dim, ks[0], ks[1], ks[2], 64)))
      return rc;
    if ((rc = encode_bshd(&L.tm_v_half, a->dtype, a->v, a->batch, a->seqlen_kv, a->heads, a->head_dim, vs[0], vs[1], vs[2], 128, 1)))
      return rc;
  }

  FmhaParams& p = L.p;
  p.B = a->batch; p.H = a->heads; p.Sq = a->seqlen_q; p.Skv = a->seqlen_kv;
  p.causal = a->causal ? 1 : 0;
  p.out_bf16 = a->out_dtype == CFK_BF16;
  // one 128-row tile per CTA at head dimension 256 and in the persistent kernel, two side by side otherwise
  p.nqblk = (a->head_dim == 256 || L.variant == 2) ? (a->seqlen_q + 127) / 128 : (a->seqlen_q + 255) / 256;
  {
    // Default by input type, the measured best: with e4m3 Q and K the first GEMM is short enough for the two query
    // tiles to take turns on one score buffer (+8-12 % on every e4m3 shape together with the share of exponentials on
    // the FMA pipe that goes with it, below); with 16-bit inputs the hand-over of
    // the buffer would set the pace (c3 1246 -> 1221 TFLOP/s).
    const int sched = g_tunable[CFK_TUNE_FMHA_SCHED].load();
    p.sched = sched < 0 ? (a->dtype == CFK_E4M3 ? 1 : 0) : sched;
  }
  p.split_keys = a->dtype == CFK_BF16 ? (a->p_split_keys < 0 ? 1024 : a->p_split_keys) : 0;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f * qd * kd;
  p.out_scale = vd;
  p.lse = a->lse; p.mi = a->mi; p.sprime = a->sprime;
  p.s_dump = a->s_dump; p.s_dump_bf16 = a->dtype == CFK_BF16;
  L.iterations = a->iterations;
  L.exp_emu = g_tunable[CFK_TUNE_FMHA_EXP_EMU].load();
  // e4m3 at d = 128 on the shared score buffer: 1 of 4 (c5 1631 against 1486 TFLOP/s with 2 of 4 and 1386 with none)
  // 16-bit at d = 256 (one softmax warpgroup, tensor-bound): none (fp16 1302 / 1266 / 1224 / 1195 for 0..3 of 4)
  if (L.exp_emu < 0) {
    if (a->dtype != CFK_E4M3) L.exp_emu = a->head_dim == 256 ? 0 : 1;
    else L.exp_emu = (a->head_dim == 128 && L.variant == 0 && p.sched == 1) ? 1 : 2;
  }
  {
    // Causal: CTAs differ in length, so heads are interleaved (heaviest blocks of a group of heads first);
    // the group is sized so that its K and V stay in L2.  Non-causal: one head at a time.
    const long long kv_bytes = 2LL * a->seqlen_kv * a->head_dim * esz;
    long long grp = a->causal ? ((long long)g_tunable[CFK_TUNE_FMHA_GROUP_MB].load() << 20) / kv_bytes : 1;
    const long long bh = (long long)a->batch * a->heads;
    p.group = (int)(grp < 1 ? 1 : (grp > bh ? bh : grp));
  }
  if ((long long)p.nqblk * a->heads * a->batch > 0x7fffffffLL) return CFK_ERR_UNSUPPORTED;
  *p_dtype = pdt;
  return CFK_OK;
}

extern "C" int cfk_fmha_forward(const cfk_fmha_args* a, cfk_stream_t stream) {
  FmhaLaunch L;
  int pdt = 0;
  const int rc = fmha_prepare(a, &L, &pdt);
  if (rc != CFK_OK) return rc;
  int err = CFK_OK;
  int* status = device_status_block(&err);
  if (!status) return err;
  L.p.status = status;
  L.stream = (cudaStream_t)stream;
  return fmha_dispatch(a->dtype, pdt, a->head_dim, L);
}

#ifdef CFK_FMHA_PROFILE
// Profiling builds only: copies the 64-word status block (per-role cycle counters live in words 8..)
// to the host and clears it.
extern "C" int cfk_debug_read_status_block(int* out64) {
  int err = CFK_OK;
  int* blk = device_status_block(&err);
  if (!blk) return err;
  if (note_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize") != cudaSuccess) return CFK_ERR_LAUNCH;
  if (note_cuda(cudaMemcpy(out64, blk, 256, cudaMemcpyDeviceToHost), "cudaMemcpy(status block)") != cudaSuccess)
    return CFK_ERR_LAUNCH;
  (void)note_cuda(cudaMemset(blk, 0, 256), "cudaMemset(status block)");
  return CFK_OK;
}
#endif
