// Single-CTA UMMA self-test: one 128 x n x (128 bytes of K) product through each operand path the
// FMHA and GEMM kernels rely on, so that a wrong descriptor shows up as a wrong number in a tiny
// test and not inside a fused kernel.  No counterpart in the reference.
#include <cstring>

#include "common.cuh"
#include "host_util.h"

namespace cfk {

constexpr int kErrSelfFull = 301, kErrSelfDone = 302;

struct SelfParams {
  int n;            // columns of D: 64 or 128
  int esz;          // operand element size (1 or 2)
  int b_mn_major;   // B stored [k][n] (1) or [n][k] (0)
  int a_from_tmem;
  uint32_t idesc;
  int kind8;
  uint32_t lbo, sbo, step;   // B descriptor fields (bytes) and start-address advance per K step
  const uint32_t* a_words;   // A as 32-bit words, row-major [128][32], for the tensor-memory path
  float* d;                  // [128][n]
  int* status;
};

__global__ void __launch_bounds__(128, 1)
selftest_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const SelfParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sA = smem_base;             // 128 rows x 128 B
  const uint32_t sB = smem_base + 16384;     // up to 2 x (128 rows x 128 B)
  const uint32_t sBar = sB + 32768;
  const uint32_t bar_full = sBar, bar_done = sBar + 8;
  volatile uint32_t* s_tmem_base = reinterpret_cast<volatile uint32_t*>(smem_gen + (sBar - smem_base) + 16);
  volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(smem_gen + (sBar - smem_base) + 20);
  const AbortCtx actx{s_abort, p.status};
  const int tid = threadIdx.x, warp = tid >> 5;

  if (cta_should_skip(p.status)) return;
  if (tid == 0) {
    mbar_init(bar_full, 1);
    mbar_init(bar_done, 1);
    *s_abort = 0u;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(s_tmem_base)), 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *s_tmem_base;
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  const uint32_t tD = tmem_base, tA = tmem_base + 128;

  const int k_rows = 128 / p.esz;                       // K extent in elements
  const uint32_t a_bytes = 16384;
  const uint32_t b_bytes = p.b_mn_major ? (uint32_t)(k_rows * p.n * p.esz) : (uint32_t)(p.n * 128);
  if (tid == 0) {
    mbar_arrive_expect_tx(bar_full, (p.a_from_tmem ? 0u : a_bytes) + b_bytes);
    if (!p.a_from_tmem) tma_load_3d(sA, &tm_a, bar_full, 0, 0, 0);
    tma_load_3d(sB, &tm_b, bar_full, 0, 0, 0);
  }
  if (p.a_from_tmem) {
    uint32_t w[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) w[i] = p.a_words[tid * 32 + i];
    tmem_st_x32(tA + lane_base, w);
    tmem_wait_st();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0) {
    if (mbar_wait(bar_full, 0, actx, kErrSelfFull)) {
      tc_fence_after_sync();
      const uint64_t a0 = make_smem_desc(sA, 16, 1024, kSwizzle128B);
      const uint64_t b0 = make_smem_desc(sB, p.lbo, p.sbo, kSwizzle128B);
      for (int kk = 0; kk < 4; ++kk) {
        const uint64_t bd = desc_advance(b0, kk * p.step);
        if (p.a_from_tmem) {
          if (p.kind8) umma_ts<true>(tD, tA + kk * 8, bd, p.idesc, kk > 0);
          else umma_ts<false>(tD, tA + kk * 8, bd, p.idesc, kk > 0);
        } else {
          const uint64_t ad = desc_advance(a0, kk * 32);
          if (p.kind8) umma_ss<true>(tD, ad, bd, p.idesc, kk > 0);
          else umma_ss<false>(tD, ad, bd, p.idesc, kk > 0);
        }
      }
      umma_commit(bar_done);
    }
  }
  if (mbar_wait_warp(bar_done, 0, actx, kErrSelfDone)) {
    tc_fence_after_sync();
    for (int c = 0; c < p.n / 32; ++c) {
      uint32_t acc[32];
      tmem_ld_x32(tD + lane_base + c * 32, acc);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) p.d[(size_t)tid * p.n + c * 32 + i] = __uint_as_float(acc[i]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 256);
  }
}


// Dense-UMMA rate probe: every CTA (one per SM) issues `groups` x 4 UMMAs of 128 x 256 x (32 bytes of K) on
// pseudo-random operands that never leave shared memory, alternating two accumulators.  Nothing but the tensor core
// and its shared-memory operand reads is exercised, so flops / time is the ceiling a kernel of this family can see
// at the clock the run settles on (the fp8 figure has no vendor-library counterpart to take from a GEMM).
constexpr int kErrPeakDone = 303;

template <bool KIND8>
__global__ void __launch_bounds__(128, 1) umma_peak_kernel(int groups, uint32_t idesc, uint32_t seed, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sA = smem_base;             // 128 rows x 128 B
  const uint32_t sB = smem_base + 16384;     // 256 rows x 128 B
  const uint32_t sBar = sB + 32768;
  volatile uint32_t* s_tmem_base = reinterpret_cast<volatile uint32_t*>(smem_gen + (sBar - smem_base) + 16);
  volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(smem_gen + (sBar - smem_base) + 20);
  const AbortCtx actx{s_abort, status};
  const int tid = threadIdx.x, warp = tid >> 5;
  if (cta_should_skip(status)) return;
  // finite pseudo-random operands: e4m3 bytes with exponent 0..7 / bf16 halves in [1, 2) with random sign
  uint32_t* words = reinterpret_cast<uint32_t*>(smem_gen);
  for (int i = tid; i < (16384 + 32768) / 4; i += 128) {
    uint32_t h = (uint32_t)i * 2654435761u ^ seed ^ (blockIdx.x * 40503u);
    h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
    words[i] = KIND8 ? (h & 0xbfbfbfbfu) : ((h & 0x807f807fu) | 0x3f803f80u);
  }
  if (tid == 0) {
    mbar_init(sBar, 1);
    *s_abort = 0u;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(s_tmem_base)), 512);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *s_tmem_base;
  if (warp == 1) {   // warp-uniform issue loop, one elected lane executes the instructions
    const uint32_t leader = elect_one();
    const uint64_t a0 = make_smem_desc(sA, 16, 1024, kSwizzle128B);
    const uint64_t b0 = make_smem_desc(sB, 16, 1024, kSwizzle128B);
    for (int g = 0; g < groups; ++g) {
      const uint32_t d = tmem_base + (g & 1) * 256;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_ss_e<KIND8, false>(d, desc_advance_lo(a0, kk * 32), desc_advance_lo(b0, kk * 32), idesc, (g > 1 || kk > 0) ? 1u : 0u,
                                leader);
    }
    umma_commit_e<false>(sBar, leader);
    (void)mbar_wait_warp(sBar, 0, actx, kErrPeakDone);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace cfk

using namespace cfk;

extern "C" int cfk_selftest_umma(const void* a, const void* b, float* d, int n, int a_fmt, int b_fmt, int b_mn_major,
                                 int a_from_tmem, cfk_stream_t stream) {
  if (!a || !b || !d) return CFK_ERR_INVALID_ARG;
  if (n != 64 && n != 128) return CFK_ERR_UNSUPPORTED;
  if (a_fmt < CFK_FP16 || a_fmt > CFK_E4M3 || b_fmt < CFK_FP16 || b_fmt > CFK_E4M3) return CFK_ERR_INVALID_ARG;
  // One MMA instruction takes both operands in one format: fp16 A with bf16 B (or any other mix) is refused here,
  // before anything is launched, because the tensor core raises an illegal-instruction fault on it.
  if (a_fmt != b_fmt) return CFK_ERR_UNSUPPORTED;
  const int esz = dtype_size(a_fmt);
  if (b_mn_major && n * esz < 128) return CFK_ERR_UNSUPPORTED;
  int err = CFK_OK;
  int* status = device_status_block(&err);
  if (!status) return err;

  const int k = 128 / esz;
  CUtensorMap tm_a, tm_b;
  {
    const uint64_t dims[3] = {(uint64_t)k, 128, 1};
    const uint64_t str[2] = {128, 128 * 128};
    const uint32_t box[3] = {(uint32_t)k, 128, 1};
    int rc = encode_tiled(&tm_a, a_fmt, 3, a, dims, str, box, 128);
    if (rc) return rc;
  }
  if (!b_mn_major) {
    const uint64_t dims[3] = {(uint64_t)k, (uint64_t)n, 1};
    const uint64_t str[2] = {128, (uint64_t)128 * n};
    const uint32_t box[3] = {(uint32_t)k, (uint32_t)n, 1};
    int rc = encode_tiled(&tm_b, b_fmt, 3, b, dims, str, box, 128);
    if (rc) return rc;
  } else {
    const uint64_t span = 128 / esz;                 // elements per 128-byte span of n
    const uint64_t nspan = (uint64_t)n / span;
    const uint64_t dims[3] = {span, (uint64_t)k, nspan};
    const uint64_t str[2] = {(uint64_t)n * esz, 128};
    const uint32_t box[3] = {(uint32_t)span, (uint32_t)k, (uint32_t)nspan};
    int rc = encode_tiled(&tm_b, b_fmt, 3, b, dims, str, box, 128);
    if (rc) return rc;
  }
  SelfParams p;
  std::memset(&p, 0, sizeof(p));
  p.n = n; p.esz = esz; p.b_mn_major = b_mn_major; p.a_from_tmem = a_from_tmem;
  p.kind8 = esz == 1;
  const uint32_t af = a_fmt == CFK_BF16 ? kFmtBF16 : 0u, bf = b_fmt == CFK_BF16 ? kFmtBF16 : 0u;
  p.idesc = make_idesc(1, af, bf, 0, b_mn_major ? 1 : 0, 128, (uint32_t)n);
  // defaults: K-major B -> 8-row groups 1024 B apart, 32 B per K step; MN-major B -> column groups
  // one [k rows][128 B] block apart, 8-row groups 1024 B apart, (32/esz) rows per K step.
  p.lbo = b_mn_major ? (uint32_t)(k * 128) : 16u;
  p.sbo = 1024u;
  p.step = b_mn_major ? (uint32_t)((32 / esz) * 128) : 32u;
  p.a_words = reinterpret_cast<const uint32_t*>(a);
  p.d = d;
  p.status = status;
  const int smem = 1024 + 16384 + 32768 + 64;
  static thread_local int attr_dev = -1;
  int dev = 0;
  if (note_cuda(cudaGetDevice(&dev), "cudaGetDevice") != cudaSuccess) return CFK_ERR_NO_DRIVER;
  if (attr_dev != dev) {
    if (note_cuda(cudaFuncSetAttribute(selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                  "cudaFuncSetAttribute(selftest smem)") != cudaSuccess)
      return CFK_ERR_LAUNCH;
    attr_dev = dev;
  }
  selftest_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(tm_a, tm_b, p);
  return note_cuda(cudaGetLastError(), "selftest launch") == cudaSuccess ? CFK_OK : CFK_ERR_LAUNCH;
}

extern "C" int cfk_umma_peak(int dtype, int groups, double* flops_out, cfk_stream_t stream) {
  if (groups < 1 || groups > (1 << 24) || !flops_out) return CFK_ERR_INVALID_ARG;
  if (dtype != CFK_FP16 && dtype != CFK_BF16 && dtype != CFK_E4M3) return CFK_ERR_UNSUPPORTED;
  int err = CFK_OK;
  int* status = device_status_block(&err);
  if (!status) return err;
  int dev = 0, sms = 0;
  if (note_cuda(cudaGetDevice(&dev), "cudaGetDevice") != cudaSuccess) return CFK_ERR_NO_DRIVER;
  if (note_cuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "sm count") != cudaSuccess)
    return CFK_ERR_LAUNCH;
  const bool k8 = dtype == CFK_E4M3;
  const uint32_t fmt = dtype == CFK_BF16 ? kFmtBF16 : 0u;
  const uint32_t idesc = make_idesc(1, fmt, fmt, 0, 0, 128, 256);
  const int smem = 1024 + 16384 + 32768 + 64;
  auto kern = k8 ? umma_peak_kernel<true> : umma_peak_kernel<false>;
  if (note_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "cudaFuncSetAttribute(peak)") !=
      cudaSuccess)
    return CFK_ERR_LAUNCH;
  kern<<<sms, 128, smem, (cudaStream_t)stream>>>(groups, idesc, 12345u, status);
  // per UMMA: 2 * 128 * 256 * (32 bytes of K / element size) flops
  *flops_out = (double)sms * groups * 4.0 * 2.0 * 128 * 256 * (32 / dtype_size(dtype));
  return note_cuda(cudaGetLastError(), "umma peak launch") == cudaSuccess ? CFK_OK : CFK_ERR_LAUNCH;
}

// ---- the bounded wait, exercised on purpose ---------------------------------------------------------------
// One warp waits on an mbarrier that nothing ever arrives on, through the same mbar_wait the kernels use but
// with a limit of `limit_ns`.  The wait gives up, writes kErrSelftestWait into the status word and the kernel
// returns normally: no trap, no fault, the context stays usable.
namespace cfk {
constexpr int kErrSelftestWait = 901;

__global__ void __launch_bounds__(32, 1) wait_gives_up_kernel(int* status, unsigned long long limit_ns) {
  __shared__ uint64_t s_bar;
  __shared__ uint32_t s_abort;
  const uint32_t bar = smem_u32(&s_bar);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    s_abort = 0u;
    fence_barrier_init();
  }
  __syncwarp();
  const AbortCtx actx{&s_abort, status};
  (void)mbar_wait(bar, 0, actx, kErrSelftestWait, limit_ns);
}
}  // namespace cfk

static int launch_wait_gives_up(int* status, int limit_ms, cfk_stream_t stream) {
  wait_gives_up_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, (unsigned long long)limit_ms * 1000000ull);
  return note_cuda(cudaGetLastError(), "wait selftest launch") == cudaSuccess ? CFK_OK : CFK_ERR_LAUNCH;
}

extern "C" int cfk_selftest_wait_gives_up(int limit_ms, cfk_stream_t stream) {
  if (limit_ms < 1 || limit_ms > 1000) return CFK_ERR_INVALID_ARG;
  int err = CFK_OK;
  int* status = device_status_block(&err);
  if (!status) return err;
  return launch_wait_gives_up(status, limit_ms, stream);
}

// The same wait, reporting into the status word of the fixed array that cfk_fmha_forward_static uses: the way to
// see that entry point's own failure path (its status query, and the clearing of the word by the next call)
// without a real failure.  Allocates nothing.
extern "C" int cfk_selftest_wait_gives_up_static(int limit_ms, cfk_stream_t stream) {
  if (limit_ms < 1 || limit_ms > 1000) return CFK_ERR_INVALID_ARG;
  int err = CFK_OK;
  int* status = cfk::static_scratch_for_current_device(&err);
  if (!status) return err;
  return launch_wait_gives_up(status, limit_ms, stream);
}
