// Dense GEMM for sm_100a:  D[r][c] = alpha * sum_k X[r][k] * Y[c][k] + beta * D[r][c], X and Y
// K-contiguous, D row-major with leading dimension ldd, fp32 accumulation in tensor memory.
// It stands where the reference has gemm<> / gemm_device (src/cute-gemm-tma-gma/gemm.cu:336-463,
// 57-334): that kernel is a single-stage TMA -> WGMMA loop that stores register accumulators straight
// to global memory, ignores alpha / beta and accumulates in the output type.  Here a pair of CTAs on two
// SMs (a cluster of 2, tcgen05 cta_group::2) computes a 256 x 256 tile:
//
//   warp 0     TMA producer: this CTA's 128 rows of X and its 128 rows of Y per 64-wide k-block, into a
//              6-stage ring; both CTAs signal the same barrier in the leader (no multicast: each CTA
//              fetches only what its own SM consumes)
//   warp 1     UMMA issuer (leader CTA only): 256 x 256 x 16 tcgen05.mma over the pair, two accumulator
//              buffers of 256 TMEM columns per CTA
//   warps 2-5  epilogue: TMEM -> registers -> alpha/beta -> output type -> a swizzled staging tile in shared
//              memory (128 rows x 128 bytes, two of them) -> TMA store, overlapped with the next tile's main
//              loop.  (The reference writes its register accumulators to global memory thread by thread,
//              gemm.cu:329-331.)
//
// The pair halves the B-operand bytes each SM reads from shared memory per FLOP, which is what bounds a
// single-CTA 128 x 256 tile.  Pairs are persistent (one per two SMs) and walk the tile list in bands of
// 8 row-tiles so that concurrently running tiles share X and Y panels in L2.  The reference's column-major
// C (gemm.cu:388-389) is the row-major D of the swapped problem (X = B, Y = A), so one kernel serves both
// output orders.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstring>

#include "common.cuh"
#include "host_util.h"

namespace cfk {

constexpr int kErrGemmFull = 201, kErrGemmEmpty = 202, kErrGemmAccFull = 203, kErrGemmAccEmpty = 204,
              kErrGemmStaged = 205, kErrGemmStageFree = 206;

struct GemmParams {
  int R, Cn, K, L;       // rows of X / D, rows of Y (= columns of D), reduction length, batch count
  int64_t ldd;           // leading dimension of D (elements)
  int64_t d_batch;       // elements between consecutive D matrices
  void* d;
  const void* src;       // matrix of the beta term (same layout as D); D itself when the update is in place
  float alpha, beta;
  int bf16;
  int tf32;              // operands and D are fp32; the tensor core runs them as tf32 (kind::tf32, 8 elements per k-step)
  int tiles_r, tiles_c;  // 256 x 256 tiles
  int* status;
};

struct GemmCfg {
  static constexpr int BM = 128, BNH = 128, BK = 64;         // per CTA: rows of X, rows of Y, k extent
  static constexpr int TILE = 256;                            // tile edge of the CTA pair
  static constexpr int XB = BM * BK * 2, YB = BNH * BK * 2;   // bytes per stage
  static constexpr int NSTAGE = 6;
  static constexpr int STAGEB = 128 * 128;                    // output staging tile: 128 rows x 128 bytes
  static constexpr int SMEM_BYTES = 1024 + NSTAGE * (XB + YB) + 2 * STAGEB + 256;
  static constexpr int NTHREADS = 192;
  static constexpr int BAND = 8;
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_r, int tiles_c, int& tr, int& tc, int& batch) {
  const int per_batch = tiles_r * tiles_c;
  batch = tile / per_batch;
  int t = tile - batch * per_batch;
  const int band_tiles = GemmCfg::BAND * tiles_c;
  const int band = t / band_tiles;
  const int first_r = band * GemmCfg::BAND;
  const int rows_in_band = (tiles_r - first_r) < GemmCfg::BAND ? (tiles_r - first_r) : GemmCfg::BAND;
  t -= band * band_tiles;
  tr = first_r + t % rows_in_band;
  tc = t / rows_in_band;
  if (band & 1) tc = tiles_c - 1 - tc;   // back and forth: a band starts on the Y panels the band before it ended on
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_y,
            const __grid_constant__ CUtensorMap tm_d, const GemmParams p) {
  using C = GemmCfg;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sX = smem_base;
  const uint32_t sY = smem_base + C::NSTAGE * C::XB;
  const uint32_t sStage = sY + C::NSTAGE * C::YB;             // [2] output staging tiles
  const uint32_t sBar = sStage + 2 * C::STAGEB;
  const uint32_t bar_full = sBar;                            // [NSTAGE] leader: both CTAs' loads of a stage landed
  const uint32_t bar_empty = sBar + 8 * C::NSTAGE;           // [NSTAGE] each CTA: its stage was consumed
  const uint32_t bar_acc_full = bar_empty + 8 * C::NSTAGE;   // [2] each CTA: accumulator complete
  const uint32_t bar_acc_empty = bar_acc_full + 16;          // [2] leader: both epilogues have read it
  const uint32_t bar_staged = bar_acc_empty + 16;            // [2] a staging tile is complete (4 epilogue warps)
  const uint32_t bar_stage_free = bar_staged + 16;           // [2] the TMA store has read a staging tile
  uint8_t* gBar = smem_gen + (sBar - smem_base);
  const uint32_t off_misc = 8 * (2 * C::NSTAGE + 8);
  volatile uint32_t* s_tmem_base = reinterpret_cast<volatile uint32_t*>(gBar + off_misc);
  volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(gBar + off_misc + 4);
  const AbortCtx actx{s_abort, p.status};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int total_tiles = p.tiles_r * p.tiles_c * p.L;
  const int bk = p.tf32 ? C::BK / 2 : C::BK;   // elements per 128-byte stage row
  const int nkb = (p.K + bk - 1) / bk;

  // One decision for the pair: both CTAs skip or both run (pair_should_skip).
  if (pair_should_skip(p.status)) return;
  if (tid == 0) {
    for (int i = 0; i < C::NSTAGE; ++i) { mbar_init(bar_full + 8 * i, 2); mbar_init(bar_empty + 8 * i, 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(bar_acc_full + 8 * i, 1); mbar_init(bar_acc_empty + 8 * i, 256); }
    for (int i = 0; i < 2; ++i) { mbar_init(bar_staged + 8 * i, 4); mbar_init(bar_stage_free + 8 * i, 1); }
    *s_abort = 0u;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(s_tmem_base)), 512);
    tmem_relinquish_pair();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tm_x); tma_prefetch_desc(&tm_y); tma_prefetch_desc(&tm_d); }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();           // the peer's barriers exist before anything is signalled on them
  tc_fence_after_sync();
  const uint32_t tmem_base = *s_tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      int idx = 0, local = 0;
      bool ok = true;
      for (int tile = pair_id; tile < total_tiles && ok; tile += n_pairs, ++local) {
        int tr, tc, b;
        tile_coords(tile, p.tiles_r, p.tiles_c, tr, tc, b);
        // Every other tile of a pair walks the reduction backwards: its first k-blocks are the ones the tile before
        // it (same row panels, as a rule) touched last, which are the ones still in L2.  The sum does not care.
        for (int i = 0; i < nkb; ++i, ++idx) {
          const int kb = (local & 1) ? nkb - 1 - i : i;
          const int s = idx % C::NSTAGE;
          const uint32_t ph = (idx / C::NSTAGE) & 1;
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1u, actx, kErrGemmEmpty)) { ok = false; break; }
          const uint32_t leader_full = map_to_cta(bar_full + 8 * s, 0);
          mbar_arrive_expect_tx_cluster(leader_full, C::XB + C::YB);
          tma_load_3d_pair(sX + s * C::XB, &tm_x, leader_full, kb * bk, tr * C::TILE + (int)rank * C::BM, b);
          tma_load_3d_pair(sY + s * C::YB, &tm_y, leader_full, kb * bk, tc * C::TILE + (int)rank * C::BNH, b);
        }
      }
    }
  } else if (warp == 1) {
    // UMMA issue: all 32 lanes of the leader's warp run the loop, one elected lane executes the instructions
    if (rank == 0) {
      const uint32_t leader = elect_one();
      const uint32_t peer_delta = map_to_cta(sBar, 1) - sBar;
      constexpr uint32_t idesc_f16 = make_idesc(1, kFmtF16, kFmtF16, 0, 0, C::TILE, C::TILE);
      constexpr uint32_t idesc_bf16 = make_idesc(1, kFmtBF16, kFmtBF16, 0, 0, C::TILE, C::TILE);
      constexpr uint32_t idesc_tf32 = make_idesc(1, 2u, 2u, 0, 0, C::TILE, C::TILE);   // kind::tf32: format code 2
      const uint32_t idesc = p.tf32 ? idesc_tf32 : (p.bf16 ? idesc_bf16 : idesc_f16);
      int idx = 0, local = 0;
      bool ok = true;
      for (int tile = pair_id; tile < total_tiles && ok; tile += n_pairs, ++local) {
        const int buf = local & 1;
        const uint32_t acc_ph = (local >> 1) & 1;
        if (!mbar_wait_warp(bar_acc_empty + 8 * buf, acc_ph ^ 1u, actx, kErrGemmAccEmpty)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d = tmem_base + buf * 256;
        for (int kb = 0; kb < nkb; ++kb, ++idx) {
          const int s = idx % C::NSTAGE;
          if (!mbar_wait_warp(bar_full + 8 * s, (idx / C::NSTAGE) & 1, actx, kErrGemmFull)) { ok = false; break; }
          tc_fence_after_sync();
          const uint64_t a0 = make_smem_desc(sX + s * C::XB, 16, 1024, kSwizzle128B);
          const uint64_t b0 = make_smem_desc(sY + s * C::YB, 16, 1024, kSwizzle128B);
          if (p.tf32) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)   // 32 bytes of reduction per UMMA: 8 tf32 elements
              umma_ss_pair_tf32(d, desc_advance(a0, kk * 32), desc_advance(b0, kk * 32), idesc, (kb | kk) != 0 ? 1u : 0u, leader);
          } else {
#pragma unroll
            for (int kk = 0; kk < C::BK / 16; ++kk)
              umma_ss_e<false, true>(d, desc_advance(a0, kk * 32), desc_advance(b0, kk * 32), idesc,
                                     (kb | kk) != 0 ? 1u : 0u, leader);
          }
          umma_commit_e<true>(bar_empty + 8 * s, leader);                // this CTA's stage
          umma_commit_e<true>(bar_empty + 8 * s + peer_delta, leader);   // the peer's stage
        }
        if (ok) {
          umma_commit_e<true>(bar_acc_full + 8 * buf, leader);
          umma_commit_e<true>(bar_acc_full + 8 * buf + peer_delta, leader);
        }
      }
    }
  } else {
    // epilogue warps 2..5; warp w may touch TMEM lanes 32*(w%4) .. +31.  A tile leaves in chunks of 128 bytes per
    // row (64 columns, 32 for fp32 output): every thread turns its row's part of the accumulator into the output
    // type and writes it into a staging tile in the 128-byte swizzled layout; when the four warps have done so, one
    // thread hands the tile to a TMA store, which clips it at the edges of D.  Two staging tiles alternate.
    const int q = warp & 3;
    const int r = q * 32 + lane;                       // row within this CTA's 128 rows
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    const int row_in_tile = (int)rank * C::BM + r;
    const uint32_t leader_acc_empty = map_to_cta(bar_acc_empty, 0);
    const int esz = p.tf32 ? 4 : 2;
    const int ccols = 128 / esz;                       // columns per chunk
    const int nchunk = C::TILE / ccols;
    const bool storer = (warp == 2 && lane == 0);
    int local = 0;
    uint32_t n = 0;                                    // chunks staged so far: chunk n uses staging tile n & 1
    bool ok = true;
    for (int tile = pair_id; tile < total_tiles && ok; tile += n_pairs, ++local) {
      int tr, tc, b;
      tile_coords(tile, p.tiles_r, p.tiles_c, tr, tc, b);
      const int buf = local & 1;
      ok = mbar_wait_warp(bar_acc_full + 8 * buf, (local >> 1) & 1, actx, kErrGemmAccFull);
      if (!ok) break;
      tc_fence_after_sync();
      const int row = tr * C::TILE + row_in_tile;
      const int col0 = tc * C::TILE;
      const size_t src_row = (size_t)b * p.d_batch + (size_t)row * p.ldd;
#pragma unroll 1
      for (int ch = 0; ch < nchunk; ++ch, ++n) {
        const uint32_t sb = n & 1u;
        const uint32_t stage = sStage + sb * C::STAGEB;
        if (n >= 2u) {   // the store that last used this staging tile has read it
          ok = mbar_wait_warp(bar_stage_free + 8 * sb, ((n >> 1) & 1u) ^ 1u, actx, kErrGemmStageFree);
          if (!ok) break;
        }
        const uint32_t row_addr = stage + r * 128;
#pragma unroll 1
        for (int h = 0; h < ccols / 32; ++h) {         // 32 accumulator columns at a time
          uint32_t acc[32];
          const int cbase = ch * ccols + h * 32;       // first of these columns within the tile
          tmem_ld_x32(tmem_base + lane_base + buf * 256 + cbase, acc);
          tmem_wait_ld();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = p.alpha * __uint_as_float(acc[i]);
          if (p.beta != 0.f && row < p.R) {            // the source matrix: this thread's row, straight from global memory
            if (p.tf32) {
              const float* srow = reinterpret_cast<const float*>(p.src) + src_row + col0 + cbase;
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                if (col0 + cbase + g * 4 < p.Cn) {
                  const float4 old = *reinterpret_cast<const float4*>(srow + g * 4);
                  v[g * 4] += p.beta * old.x; v[g * 4 + 1] += p.beta * old.y;
                  v[g * 4 + 2] += p.beta * old.z; v[g * 4 + 3] += p.beta * old.w;
                }
              }
            } else {
              const uint16_t* srow = reinterpret_cast<const uint16_t*>(p.src) + src_row + col0 + cbase;
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                if (col0 + cbase + g * 8 < p.Cn) {
                  const uint4 old = *reinterpret_cast<const uint4*>(srow + g * 8);
                  const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    float lo, hi;
                    if (p.bf16) {
                      lo = __uint_as_float(ow[i] << 16);
                      hi = __uint_as_float(ow[i] & 0xffff0000u);
                    } else {
                      const __half2 hh = *reinterpret_cast<const __half2*>(&ow[i]);
                      lo = __low2float(hh);
                      hi = __high2float(hh);
                    }
                    v[g * 8 + 2 * i] += p.beta * lo;
                    v[g * 8 + 2 * i + 1] += p.beta * hi;
                  }
                }
              }
            }
          }
          // 16-byte pieces of the row, piece index XOR (row & 7): the 128-byte swizzle the TMA store undoes
          if (p.tf32) {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const uint32_t piece = (uint32_t)g ^ (uint32_t)(r & 7);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + piece * 16),
                           "r"(__float_as_uint(v[g * 4])), "r"(__float_as_uint(v[g * 4 + 1])),
                           "r"(__float_as_uint(v[g * 4 + 2])), "r"(__float_as_uint(v[g * 4 + 3])) : "memory");
            }
          } else {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint32_t w0, w1, w2, w3;
              if (p.bf16) {
                w0 = pack_bf16x2(v[g * 8], v[g * 8 + 1]); w1 = pack_bf16x2(v[g * 8 + 2], v[g * 8 + 3]);
                w2 = pack_bf16x2(v[g * 8 + 4], v[g * 8 + 5]); w3 = pack_bf16x2(v[g * 8 + 6], v[g * 8 + 7]);
              } else {
                w0 = pack_f16x2(v[g * 8], v[g * 8 + 1]); w1 = pack_f16x2(v[g * 8 + 2], v[g * 8 + 3]);
                w2 = pack_f16x2(v[g * 8 + 4], v[g * 8 + 5]); w3 = pack_f16x2(v[g * 8 + 6], v[g * 8 + 7]);
              }
              const uint32_t piece = (uint32_t)(h * 4 + g) ^ (uint32_t)(r & 7);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + piece * 16), "r"(w0), "r"(w1),
                           "r"(w2), "r"(w3) : "memory");
            }
          }
        }
        if (ch == nchunk - 1) {   // the accumulator has been read: the next tile but one may overwrite it
          tc_fence_before_sync();
          mbar_arrive_cluster(leader_acc_empty + 8 * buf);
        }
        fence_proxy_async_smem();
        mbar_arrive_warp(bar_staged + 8 * sb);
        if (storer) {
          if (!mbar_wait(bar_staged + 8 * sb, (n >> 1) & 1u, actx, kErrGemmStaged)) { ok = false; }
          else {
            tma_store_3d(&tm_d, stage, col0 + ch * ccols, tr * C::TILE + (int)rank * C::BM, b);
            tma_store_commit();
            tma_store_wait_read1();            // every store but this one has read its staging tile
            if (n >= 1u) mbar_arrive(bar_stage_free + 8 * (sb ^ 1u));
          }
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
    }
    if (storer) tma_store_wait_read0();
  }

  settle_if_aborted(s_abort);
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();           // no CTA leaves while its peer may still read its shared memory or signal it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

}  // namespace cfk

using namespace cfk;

extern "C" int cfk_gemm(const cfk_gemm_args* a, cfk_stream_t stream) {
  if (!a || !a->a || !a->b || !a->c) return CFK_ERR_INVALID_ARG;
  if (a->m <= 0 || a->n <= 0 || a->k <= 0 || a->l <= 0 || a->iterations < 0) return CFK_ERR_INVALID_ARG;
  if (a->dtype != CFK_FP16 && a->dtype != CFK_BF16 && a->dtype != CFK_FP32) return CFK_ERR_UNSUPPORTED;
  if ((a->m % 8) || (a->n % 8) || (a->k % 8)) return CFK_ERR_UNSUPPORTED;
  if (((uintptr_t)a->a | (uintptr_t)a->b | (uintptr_t)a->c | (uintptr_t)a->c_src) & 15u) return CFK_ERR_INVALID_ARG;

  int err = CFK_OK;
  int* status = device_status_block(&err);
  if (!status) return err;

  // Row-major C: X = A (rows m), Y = B (rows n).  Column-major C is the row-major n x m matrix of
  // the swapped product.
  const void* x = a->c_row_major ? a->a : a->b;
  const void* y = a->c_row_major ? a->b : a->a;
  const int R = a->c_row_major ? a->m : a->n;
  const int Cn = a->c_row_major ? a->n : a->m;

  CUtensorMap tm_x, tm_y;
  const uint64_t esz = (uint64_t)dtype_size(a->dtype);
  const uint32_t bk = (uint32_t)(128 / esz);                   // one 128-byte span of the reduction per stage
  const uint64_t xd[3] = {(uint64_t)a->k, (uint64_t)R, (uint64_t)a->l};
  const uint64_t xs[2] = {(uint64_t)a->k * esz, (uint64_t)a->k * esz * (uint64_t)R};
  const uint32_t xb[3] = {bk, GemmCfg::BM, 1};                 // per CTA: 128 rows of X
  const uint64_t yd[3] = {(uint64_t)a->k, (uint64_t)Cn, (uint64_t)a->l};
  const uint64_t ys[2] = {(uint64_t)a->k * esz, (uint64_t)a->k * esz * (uint64_t)Cn};
  const uint32_t yb[3] = {bk, GemmCfg::BNH, 1};                // per CTA: 128 rows of Y
  int rc;
  if ((rc = encode_tiled(&tm_x, a->dtype, 3, x, xd, xs, xb, 128))) return rc;
  if ((rc = encode_tiled(&tm_y, a->dtype, 3, y, yd, ys, yb, 128))) return rc;

  // D (row-major R x Cn per batch) for the TMA store of the epilogue: boxes of 128 rows x 128 bytes
  CUtensorMap tm_d;
  const uint64_t dd[3] = {(uint64_t)Cn, (uint64_t)R, (uint64_t)a->l};
  const uint64_t ds[2] = {(uint64_t)Cn * esz, (uint64_t)Cn * esz * (uint64_t)R};
  const uint32_t db[3] = {bk, GemmCfg::BM, 1};
  if ((rc = encode_tiled(&tm_d, a->dtype, 3, a->c, dd, ds, db, 128))) return rc;

  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.R = R; p.Cn = Cn; p.K = a->k; p.L = a->l;
  p.ldd = Cn;
  p.d_batch = (int64_t)R * Cn;
  p.d = a->c;
  p.src = a->c_src ? a->c_src : a->c;
  p.alpha = a->alpha; p.beta = a->beta;
  p.bf16 = a->dtype == CFK_BF16;
  p.tf32 = a->dtype == CFK_FP32;
  p.tiles_r = (R + GemmCfg::TILE - 1) / GemmCfg::TILE;
  p.tiles_c = (Cn + GemmCfg::TILE - 1) / GemmCfg::TILE;
  p.status = status;

  static thread_local int attr_dev = -1;
  static thread_local int sm_count = 0;
  int dev = 0;
  if (note_cuda(cudaGetDevice(&dev), "cudaGetDevice") != cudaSuccess) return CFK_ERR_NO_DRIVER;
  if (attr_dev != dev) {
    if (note_cuda(cudaFuncSetAttribute(gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg::SMEM_BYTES),
                  "cudaFuncSetAttribute(gemm smem)") != cudaSuccess)
      return CFK_ERR_LAUNCH;
    if (note_cuda(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev), "sm count") != cudaSuccess)
      return CFK_ERR_LAUNCH;
    attr_dev = dev;
  }
  const long long total = (long long)p.tiles_r * p.tiles_c * p.L;
  if (total > 0x7fffffffLL) return CFK_ERR_UNSUPPORTED;
  const long long pairs = total < sm_count / 2 ? total : sm_count / 2;   // one CTA pair per two SMs
  const int grid = (int)(2 * pairs);
  for (int it = 0; it < a->iterations; ++it)
    gemm_kernel<<<grid, GemmCfg::NTHREADS, GemmCfg::SMEM_BYTES, (cudaStream_t)stream>>>(tm_x, tm_y, tm_d, p);
  return note_cuda(cudaGetLastError(), "gemm launch") == cudaSuccess ? CFK_OK : CFK_ERR_LAUNCH;
}
