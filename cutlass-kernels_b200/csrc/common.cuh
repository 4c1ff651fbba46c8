// Device-side building blocks for the sm_100a kernels: mbarrier, TMA (bulk tensor copies),
// tcgen05 (tensor memory + UMMA) wrappers and descriptor encoders.  Everything is inline PTX;
// no CUTLASS/CuTe.  These replace the roles of cfk::barrierInit / cfk::copy / cfk::gemm in the
// reference (lib/gemm/copy_tensor.hpp:15-100, lib/gemm/gemm_tensor.hpp:12-45), which wrap the
// Hopper TMA + WGMMA atoms.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cfk {

// ---- device status word ---------------------------------------------------------------------
// Every wait in the kernels is bounded.  A wait that gives up writes (code | where) into the
// status word once (first failure wins), raises a CTA-wide abort flag in shared memory, and the
// role returns to the common tear-down, so a broken pipeline ends as an error code, not a hang.
constexpr int kDevOk = 0;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s per individual wait

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier ---------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One arrival for a whole warp: every lane has finished its part (the caller has executed the warp-collective
// wait or a __syncwarp), lane 0 arrives.  32 arrivals of a warp on one barrier are serialised; this is one.
__device__ __forceinline__ void mbar_arrive_warp(uint32_t bar) {
  __syncwarp();
  asm volatile("{\n\t.reg .pred q;\n\tsetp.eq.u32 q, %1, 0;\n\t@q mbarrier.arrive.shared::cta.b64 _, [%0];\n\t}"
               ::"r"(bar), "r"(threadIdx.x & 31u) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Non-blocking form: true if the phase of the given parity has completed.
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

struct AbortCtx {
  volatile uint32_t* cta_abort;  // shared memory flag
  int* status;                   // global status word
};

// Returns false if the wait was abandoned (time limit, or another role of this CTA aborted).
// `backoff_ns` > 0: sleep that long between looks.  For roles that wait long and are in no hurry (an epilogue waiting
// for its item to end, a producer waiting for a free slot): a warp that polls takes issue slots from the warps of its
// scheduler that are computing.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const AbortCtx& ctx, int where,
                                          unsigned long long limit_ns = kWaitLimitNs, unsigned backoff_ns = 0) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (backoff_ns) __nanosleep(backoff_ns);
    if ((++spins & 0xffu) == 0) {
      if (*ctx.cta_abort) return false;
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) {
        *ctx.cta_abort = 1u;
        atomicCAS(ctx.status, kDevOk, where);
        return false;
      }
    }
  }
}
// Same, with a warp-uniform answer (needed before warp-collective tcgen05.ld/st).
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, const AbortCtx& ctx, int where,
                                               unsigned backoff_ns = 0) {
  const bool ok = mbar_wait(bar, parity, ctx, where, kWaitLimitNs, backoff_ns);
  return __all_sync(0xffffffffu, ok);
}

// Tear-down of a CTA whose roles gave up: what it has in flight (TMA copies into its shared memory, UMMAs into its
// tensor memory) signals barriers that nobody waits on any more, so every thread lets a fixed time pass, far longer
// than such an operation takes and bounded, before shared and tensor memory are given back.
__device__ __forceinline__ void settle_if_aborted(volatile uint32_t* cta_abort) {
  if (*cta_abort) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
}

// CTA-uniform test of the status word (one thread reads, everybody gets the same answer).
__device__ __forceinline__ bool cta_should_skip(const int* status) {
  __shared__ int s_skip;
  if (threadIdx.x == 0) s_skip = *reinterpret_cast<const volatile int*>(status);
  __syncthreads();
  return s_skip != 0;
}

// ---- fences -----------------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---- TMA ----------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1,
                                            int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1,
                                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_store_5d(const CUtensorMap* m, uint32_t src, int c0, int c1, int c2, int c3,
                                             int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, uint32_t src, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read0() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// all but the most recent store group have finished reading their shared-memory source
__device__ __forceinline__ void tma_store_wait_read1() {
  asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
}

// ---- tensor memory ------------------------------------------------------------------------------
// One warp allocates `ncols` (power of two, 32..512) columns; the base address lands in shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

#include "tmem_ldst.inc"
// One 32-bit column of this thread's TMEM lane (warp-collective): per-row scalars that travel between roles.
__device__ __forceinline__ void tmem_st_x1(uint32_t taddr, uint32_t v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t tmem_ld_x1(uint32_t taddr) {
  uint32_t v;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(v) : "r"(taddr));
  return v;
}

// ---- UMMA descriptors -----------------------------------------------------------------------------
// Shared-memory matrix descriptor (64 bit): start address, leading/stride byte offsets (all >> 4),
// descriptor version 1 (bits 46-47), swizzle mode in bits 61-63.
constexpr uint32_t kSwizzleNone = 0, kSwizzle128B = 2, kSwizzle64B = 4, kSwizzle32B = 6;

__host__ __device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                            uint32_t swizzle) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= 1ull << 46;
  d |= static_cast<uint64_t>(swizzle & 7u) << 61;
  return d;
}
// Advance the start address of a descriptor by `bytes` (a multiple of 16).
__device__ __forceinline__ uint64_t desc_advance(uint64_t d, uint32_t bytes) { return d + (bytes >> 4); }

// Instruction descriptor (32 bit) for kind::f16 / kind::tf32 / kind::f8f6f4.
//   c_format: 0 f16, 1 f32.  a/b format: kind::f16 -> 0 f16, 1 bf16; kind::f8f6f4 -> 0 e4m3, 1 e5m2.
//   major: 0 = K-major, 1 = MN-major.
constexpr uint32_t kFmtF16 = 0, kFmtBF16 = 1, kFmtE4M3 = 0;
__host__ __device__ constexpr uint32_t make_idesc(uint32_t c_format, uint32_t a_format, uint32_t b_format,
                                                  uint32_t a_major, uint32_t b_major, uint32_t M, uint32_t N) {
  return (c_format << 4) | (a_format << 7) | (b_format << 10) | (a_major << 15) | (b_major << 16) |
         ((N >> 3) << 17) | ((M >> 4) << 24);
}

// Same, touching only the low word (start address and leading offset share it, and the address field cannot
// carry out of it): one 32-bit add instead of a 64-bit one on the single thread that issues every UMMA.
__device__ __forceinline__ uint64_t desc_advance_lo(uint64_t d, uint32_t bytes) {
  return (d & 0xffffffff00000000ull) | static_cast<uint32_t>(static_cast<uint32_t>(d) + (bytes >> 4));
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.  KIND8 selects kind::f8f6f4, else kind::f16.
template <bool KIND8>
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  if constexpr (KIND8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// D[tmem] (+)= A[tmem] * B[smem].
template <bool KIND8>
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  if constexpr (KIND8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// ---- warp-uniform issue ---------------------------------------------------------------------------
// The UMMA-issuing warp runs its loop with all 32 lanes (uniform control flow, so descriptors and loop state can
// live in uniform registers) and predicates only the tcgen05 instruction itself on one elected lane.  Measured
// on B200 with eight other warps saturating the FMA pipe: 65 clk per UMMA this way against 225 clk when the
// whole loop sits inside an `if (lane == 0)` branch, because the branchy form needs several times the issue slots.
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t is_leader;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(is_leader));
  return is_leader;
}
template <bool KIND8, bool PAIR>
__device__ __forceinline__ void umma_ss_e(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate, uint32_t leader) {
  if constexpr (KIND8 && !PAIR)
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                 "@q tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader) : "memory");
  else if constexpr (!KIND8 && !PAIR)
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                 "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader) : "memory");
  else if constexpr (KIND8 && PAIR)
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                 "@q tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader) : "memory");
  else
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                 "@q tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader) : "memory");
}
template <bool KIND8, bool PAIR>
__device__ __forceinline__ void umma_ts_e(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate, uint32_t leader) {
  if constexpr (KIND8 && !PAIR)
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                 "@q tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader) : "memory");
  else if constexpr (!KIND8 && !PAIR)
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                 "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader) : "memory");
  else if constexpr (KIND8 && PAIR)
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                 "@q tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader) : "memory");
  else
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
                 "@q tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader) : "memory");
}
template <bool PAIR>
__device__ __forceinline__ void umma_commit_e(uint32_t bar, uint32_t leader) {
  if constexpr (PAIR)
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
                 "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
                 ::"r"(bar), "r"(leader) : "memory");
  else
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
                 "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
                 ::"r"(bar), "r"(leader) : "memory");
}

// The mbarrier receives one arrival once every tcgen05 operation issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// ---- thread-block clusters and CTA pairs (cta_group::2) ----------------------------------------------
// Remote barrier operations use the default semantics on purpose: the .release.cluster / .acquire.cluster
// forms were measured at about a thousand cycles per operation on B200, which serialises a pipeline.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The skip decision of a CTA pair (see cta_should_skip), taken ONCE for the pair: if each CTA read the status word
// for itself, another CTA's wait could give up between the two reads, one CTA of the pair would return and its peer
// would go on to allocate tensor memory for the pair (which has no time limit) and to signal barriers in the shared
// memory of a CTA that is gone.  Rank 0 reads the word and stores the decision into both CTAs' shared memory; after
// the cluster barrier both branch on their own copy.  Every thread of both CTAs must call this.
__device__ __forceinline__ bool pair_should_skip(const int* status) {
  __shared__ uint32_t s_pair_skip;
  if (threadIdx.x == 0 && cluster_ctarank() == 0) {
    const uint32_t v = (uint32_t)(*reinterpret_cast<const volatile int*>(status) != 0);
    const uint32_t here = smem_u32(&s_pair_skip);
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(map_to_cta(here, 0)), "r"(v) : "memory");
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(map_to_cta(here, 1)), "r"(v) : "memory");
  }
  cluster_sync_all();   // release / acquire at cluster scope: the peer's copy is written before anyone reads
  return *reinterpret_cast<volatile uint32_t*>(&s_pair_skip) != 0u;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster_warp(uint32_t cluster_bar) {   // see mbar_arrive_warp
  __syncwarp();
  asm volatile("{\n\t.reg .pred q;\n\tsetp.eq.u32 q, %1, 0;\n\t@q mbarrier.arrive.shared::cluster.b64 _, [%0];\n\t}"
               ::"r"(cluster_bar), "r"(threadIdx.x & 31u) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar), "r"(bytes) : "memory");
}
// TMA load whose completion is signalled on a barrier of either CTA of the pair (no multicast: every CTA
// fetches its own data into its own shared memory).
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* m, uint32_t cluster_bar, int c0, int c1,
                                                 int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(cluster_bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_5d_pair(uint32_t dst, const CUtensorMap* m, uint32_t cluster_bar, int c0, int c1,
                                                 int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(cluster_bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
// Tensor memory of a CTA pair: one warp of each CTA allocates; both get the same column base.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// UMMA over a CTA pair (umma_ss_e / umma_ts_e with PAIR = true): M = 256, rows 0-127 in the leader's tensor memory,
// 128-255 in its peer's; each CTA supplies its own A rows and its own half of B's N extent from the same
// shared-memory offsets.
// fp32 operands run as tf32: 8 elements (32 bytes) of reduction per instruction (the reference runs its fp32 GEMM
// type the same way, src/cute-gemm-tma-gma/gemm.cu:355-356).
__device__ __forceinline__ void umma_ss_pair_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                  uint32_t accumulate, uint32_t leader) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(leader)
      : "memory");
}
// Move registers between warpgroups (executed by every warp of a warpgroup).
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// ---- small numeric helpers --------------------------------------------------------------------------
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// two floats -> packed half2 / bfloat162 (lo in the low 16 bits), round to nearest even
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// four floats -> packed e4m3x4 (x0 in the lowest byte), saturating
__device__ __forceinline__ uint32_t pack_e4m3x4(float x0, float x1, float x2, float x3) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(x1), "f"(x0));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(x3), "f"(x2));
  // the two halves are joined as a register pair, not with shift and or: one instruction less where it is not free
  // (c5 1710-1724 -> 1771-1772 TFLOP/s)
  uint32_t r;
  asm("mov.b32 %0, {%1, %2};" : "=r"(r) : "h"(lo), "h"(hi));
  return r;
}

}  // namespace cfk
