// Flash-attention forward for sm_100a: O = softmax(Q K^T * scale) V, one CTA per (256 query rows,
// head, batch).  It stands where the reference has fmhaForwardPipelinedWspl / ...NoWspl /
// fmhaForwardNoPipeline (src/fmha-pipeline/fmha_pipe_ws.h:69-365, fmha_pipe_nows.h:72-331,
// fmha_nopipe.h:43-342) with their producer / consumer / softmax / epilogue pieces
// (fmha_producer.h:4-79, fmha_consumer.h:8-73, online_softmax.h:87-207, fmha_epilogue.h:120-177),
// but is organised around Blackwell's tensor memory instead of WGMMA register fragments:
//
//   warps 0-3   softmax for query tile 0 (thread r owns row r == TMEM lane r)
//   warps 4-7   softmax for query tile 1
//   warp 8      UMMA issuer (one thread): S_t = Q_t K_j^T and O_t += P_t V_j, accumulators in TMEM
//   warp 9      TMA producer: Q tiles once, then K_j, V_j tiles into a ring of shared-memory slots
//   warps 10-11 idle; they complete the third warpgroup so that registers can be moved from it to the
//               softmax warpgroups (setmaxnreg works on whole warpgroups)
//
// Two 128-row query tiles are in flight per CTA so that the tensor core works on one tile's GEMMs
// while the other tile's softmax runs.  P (unnormalised, rounded to the GEMM-II operand type exactly
// as fmha_consumer.h:54 does) is written back over S in TMEM and consumed from there; V is used in
// its natural [key][d] layout through an MN-major operand descriptor, so neither the host-side V
// transpose (src/fmha-pipeline/fmha_forward.cu:514-532) nor the register shuffle of reg2reg.h:45-108
// exists here.  The running maximum is only moved (and O only rescaled) when the new maximum exceeds
// the one in use by more than kTau in the log2 domain; the reference rescales on every tile
// (online_softmax.h:144-165).  Both carry the same factor into O and the row sum, so O / l is
// unchanged.
#pragma once
#include <type_traits>

#include "common.cuh"
#include "fmha_params.h"

namespace cfk {

template <int DT, int PT, int HD>
struct FmhaCfg {
  static constexpr int ESZ = (DT == kDtE4M3) ? 1 : 2;
  static constexpr int PESZ = (PT == kDtE4M3) ? 1 : 2;
  static_assert(ESZ == PESZ, "P and V must share an MMA kind");
  static constexpr bool KIND8 = (ESZ == 1);
  static constexpr int BM = 128, BN = 128;
  static constexpr int ROWB = HD * ESZ;            // bytes per row of a Q/K/V tile
  static_assert(ROWB % 128 == 0, "rows must be whole 128-byte swizzle spans");
  static constexpr int NSUB = ROWB / 128;          // 128-byte wide sub-tiles per tile
  static constexpr int SUBB = 128 * 128;           // bytes per sub-tile (128 rows x 128 B)
  static constexpr int TILEB = NSUB * SUBB;        // bytes per Q/K/V tile
  static constexpr int ONSUB = HD * 2 / 128;       // output is always 16 bit
  static constexpr int OTILEB = ONSUB * SUBB;
  static constexpr bool O_SEPARATE = (OTILEB > TILEB);  // else O is staged over the Q tile
  static constexpr int SMEM_LIMIT = 232448;
  static constexpr int FIXEDB = 2 * TILEB + (O_SEPARATE ? 2 * OTILEB : 0);
  static constexpr int BARB = 512;
  static constexpr int NSLOT_FIT = (SMEM_LIMIT - 1024 - BARB - FIXEDB) / TILEB;
  static constexpr int NSLOT = NSLOT_FIT > 8 ? 8 : NSLOT_FIT;
  static_assert(NSLOT >= 3, "ring too small");
  static constexpr int SMEM_BYTES = 1024 + FIXEDB + NSLOT * TILEB + BARB;
  static constexpr int QK_KSTEPS = ROWB / 32;      // each UMMA consumes 32 bytes of K extent
  static constexpr int PV_KSTEPS = BN * ESZ / 32;
  static constexpr int V_STEPB = (32 / ESZ) * 128; // bytes between successive 32-byte-K groups of V rows
  static constexpr int PCOLS = BN * PESZ / 4;      // TMEM columns taken by P
  static constexpr int TMEM_COLS = 512;
  static constexpr int O_COL0 = 256;
  static constexpr uint32_t FMT_IN = (DT == kDtBF16) ? kFmtBF16 : 0u;   // f16 / e4m3 are both code 0
  static constexpr uint32_t FMT_P = (PT == kDtBF16) ? kFmtBF16 : 0u;
  static constexpr uint32_t IDESC_QK = make_idesc(1, FMT_IN, FMT_IN, 0, 0, BM, BN);
  static constexpr uint32_t IDESC_PV = make_idesc(1, FMT_P, FMT_IN, 0, 1, BM, HD);
  static constexpr int NTHREADS = 384;
  // Register budget after setmaxnreg.  The pool is what the CTA was launched with: 384 threads at the
  // 168 registers a 384-thread launch bound allows.  setmaxnreg.inc blocks until the registers it asks
  // for are free, with no time limit, so the sum below must never exceed that pool.
  static constexpr int LAUNCH_REGS = 168, SOFTMAX_REGS = 216, AUX_REGS = 72;
  static_assert(2 * 128 * SOFTMAX_REGS + 128 * AUX_REGS <= NTHREADS * LAUNCH_REGS, "setmaxnreg would block forever");
  // log2-domain slack before the running maximum is moved, and a constant exponent offset that puts
  // P into the well-represented range of its type (it cancels in O / l).
  static constexpr float TAU = (PT == kDtE4M3) ? 2.0f : 8.0f;
  static constexpr float PSHIFT = (PT == kDtE4M3) ? 6.0f : 0.0f;
};

// exp2 of a pair of log2-domain scores on the special-function unit ...
__device__ __forceinline__ float2 exp2_pair_sfu(float2 x) { return make_float2(ex2_approx(x.x), ex2_approx(x.y)); }
// ... or on the FMA pipe: x = n + f with n = round(x), f in [-0.5, 0.5]; 2^f by a cubic whose relative
// error (7.5e-5) is below the rounding step of every P format; 2^n by adding n to the exponent bits.
// The special-function unit delivers 16 results per clock per SM, exactly what the tensor core consumes
// at D=128, so a share of the exponentials is moved here (packed two-wide FMA instructions).
__device__ __forceinline__ float2 exp2_pair_fma(float2 x) {
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 t = __fadd2_rn(x, make_float2(12582912.f, 12582912.f));      // 1.5 * 2^23: n sits in the low bits
  const float2 nf = __fadd2_rn(t, make_float2(-12582912.f, -12582912.f));
  const float2 f = __ffma2_rn(nf, make_float2(-1.f, -1.f), x);
  float2 q = __ffma2_rn(make_float2(0.0551716648f, 0.0551716648f), f, make_float2(0.2426111251f, 0.2426111251f));
  q = __ffma2_rn(q, f, make_float2(0.6932609677f, 0.6932609677f));
  q = __ffma2_rn(q, f, make_float2(0.9999280572f, 0.9999280572f));
  q.x = __int_as_float(__float_as_int(q.x) + (__float_as_int(t.x) << 23));
  q.y = __int_as_float(__float_as_int(q.y) + (__float_as_int(t.y) << 23));
  return q;
}

// Optional per-role cycle counters (build with -DCFK_FMHA_PROFILE): lane 0 of the first warp of softmax
// warpgroup 0 and the UMMA thread add the cycles they spend in each phase to words 8.. of the status
// block.  Off in the shipped library.
#ifdef CFK_FMHA_PROFILE
#define CFK_PROF_DECL(n) long long prof_t[n] = {0}; long long prof_last = clock64();
#define CFK_PROF_MARK(i) { const long long now_ = clock64(); prof_t[i] += now_ - prof_last; prof_last = now_; }
#define CFK_PROF_FLUSH(base, n, cond) if (cond) { for (int i_ = 0; i_ < n; ++i_) atomicAdd(reinterpret_cast<unsigned long long*>(p.status + 8) + base + i_, (unsigned long long)prof_t[i_]); }
#else
#define CFK_PROF_DECL(n)
#define CFK_PROF_MARK(i)
#define CFK_PROF_FLUSH(base, n, cond)
#endif

// EMU: of every four pairs of probabilities, how many are computed on the FMA pipe (0..3).
template <int DT, int PT, int HD, int EMU>
__global__ void __launch_bounds__(384, 1)
fmha_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                const FmhaParams p) {
  using C = FmhaCfg<DT, PT, HD>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t sQ = smem_base;                                    // 2 tiles
  const uint32_t sOst = smem_base + 2 * C::TILEB;                   // separate O staging (if any)
  const uint32_t sRing = sOst + (C::O_SEPARATE ? 2 * C::OTILEB : 0);
  const uint32_t sBar = sRing + C::NSLOT * C::TILEB;
  uint8_t* gBar = smem_gen + (sBar - smem_base);
  // barrier map (8 bytes each)
  const uint32_t bar_q_full = sBar;
  const uint32_t bar_kv_full = sBar + 8;                   // [NSLOT]
  const uint32_t bar_kv_empty = bar_kv_full + 8 * C::NSLOT;  // [NSLOT]
  const uint32_t bar_s_full = bar_kv_empty + 8 * C::NSLOT;   // [2]
  const uint32_t bar_p_full = bar_s_full + 16;               // [2]
  const uint32_t bar_o_full = bar_p_full + 16;               // [2]
  const uint32_t bar_o_staged = bar_o_full + 16;             // [2]
  const uint32_t off_misc = (bar_o_staged + 16) - sBar;
  volatile uint32_t* s_tmem_base = reinterpret_cast<volatile uint32_t*>(gBar + off_misc);
  volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(gBar + off_misc + 4);
  const AbortCtx actx{s_abort, p.status};

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // Work item.  The grid is one-dimensional.  (batch, head) pairs are taken in groups whose K and V
  // fit in L2 together; inside a group the 256-row query blocks go from the last (heaviest when causal)
  // to the first, all pairs of the group side by side, so that CTAs finish together and the tail is light.
  int qblk, head, batch;
  {
    const int bh_total = p.B * p.H;
    const int per_group = p.group * p.nqblk;
    const int g = (int)blockIdx.x / per_group;
    const int r = (int)blockIdx.x - g * per_group;
    const int left = bh_total - g * p.group;
    const int gsz = left < p.group ? left : p.group;
    qblk = p.nqblk - 1 - r / gsz;
    const int bh = g * p.group + r % gsz;
    batch = bh / p.H;
    head = bh - batch * p.H;
  }
  const int nkv_total = (p.Skv + C::BN - 1) / C::BN;
  const int diag_off = p.Skv - p.Sq;
  auto tiles_for = [&](int t) -> int {
    const int row0 = qblk * 256 + t * 128;
    if (row0 >= p.Sq) return 0;
    int n = nkv_total;
    if (p.causal) {
      const int last_key = row0 + 127 + diag_off;
      const int nc = last_key < 0 ? 1 : last_key / C::BN + 1;
      n = nc < n ? nc : n;
    }
    return n;
  };
  const int n_t0 = tiles_for(0), n_t1 = tiles_for(1);
  auto n_of = [&](int t) -> int { return t == 0 ? n_t0 : n_t1; };
  const int n_kv = n_t0 > n_t1 ? n_t0 : n_t1;

  // A launch that finds the status word already set does nothing: once one wait has given up, the
  // rest of the grid (and later launches) must not each spend their own time limit.
  if (cta_should_skip(p.status)) return;

  // ---- set-up ----
  if (tid == 0) {
    mbar_init(bar_q_full, 1);
    for (int i = 0; i < C::NSLOT; ++i) {
      mbar_init(bar_kv_full + 8 * i, 1);
      mbar_init(bar_kv_empty + 8 * i, 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar_s_full + 8 * t, 1);
      mbar_init(bar_p_full + 8 * t, 128);
      mbar_init(bar_o_full + 8 * t, 1);
      mbar_init(bar_o_staged + 8 * t, 128);
    }
    *s_abort = 0u;
    fence_barrier_init();
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(s_tmem_base)), C::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 9 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_o);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *s_tmem_base;

  // bf16 only: rows that see few keys get P as a two-term sum (hi + lo), see the P store below.
  bool split = false;
  if constexpr (PT == kDtBF16) {
    int visible = p.Skv;
    if (p.causal) { const int v0 = qblk * 256 + diag_off + 1; visible = v0 < visible ? v0 : visible; }
    split = visible < p.split_keys;
  }

  if (warp >= 8) {
   // Third warpgroup: hands most of its registers to the softmax warpgroups.
   setmaxnreg_dec<C::AUX_REGS>();
   if (warp == 9) {
    // =========================== TMA producer ===========================
    if (lane == 0 && n_kv > 0) {
      const uint32_t q_bytes = (n_t0 > 0 ? C::TILEB : 0) + (n_t1 > 0 ? C::TILEB : 0);
      mbar_arrive_expect_tx(bar_q_full, q_bytes);
      for (int t = 0; t < 2; ++t)
        if (n_of(t) > 0) tma_load_5d(sQ + t * C::TILEB, &tm_q, bar_q_full, 0, qblk * 256 + t * 128, 0, head, batch);
      int idx = 0;
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        for (int which = 0; which < 2; ++which, ++idx) {
          const int slot = idx % C::NSLOT;
          const uint32_t ph = (idx / C::NSLOT) & 1;
          if (!mbar_wait(bar_kv_empty + 8 * slot, ph ^ 1u, actx, kErrFmhaKvEmpty)) { ok = false; break; }
          mbar_arrive_expect_tx(bar_kv_full + 8 * slot, C::TILEB);
          tma_load_5d(sRing + slot * C::TILEB, which == 0 ? &tm_k : &tm_v, bar_kv_full + 8 * slot, 0, j * C::BN, 0,
                      head, batch);
        }
      }
    }
   } else if (warp == 8) {
    // =========================== UMMA issuer ===========================
    if (lane == 0 && n_kv > 0) {
      bool ok = true;
      auto issue_qk = [&](int t, int slot) {
        const uint64_t a0 = make_smem_desc(sQ + t * C::TILEB, 16, 1024, kSwizzle128B);
        const uint64_t b0 = make_smem_desc(sRing + slot * C::TILEB, 16, 1024, kSwizzle128B);
        const uint32_t d = tmem_base + t * 128;
#pragma unroll
        for (int kk = 0; kk < C::QK_KSTEPS; ++kk) {
          const uint32_t off = (kk >> 2) * C::SUBB + (kk & 3) * 32;
          umma_ss<C::KIND8>(d, desc_advance(a0, off), desc_advance(b0, off), C::IDESC_QK, kk > 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int t, int slot, uint32_t accumulate) {
        // V tile: [NSUB][128 keys][128 B]; N (= d) contiguous.  LBO = distance between the 64-element
        // column groups (one sub-tile), SBO = distance between groups of 8 keys.
        const uint64_t b0 = make_smem_desc(sRing + slot * C::TILEB, C::SUBB, 1024, kSwizzle128B);
        const uint32_t d = tmem_base + C::O_COL0 + t * HD;
        const uint32_t a = tmem_base + t * 128;
#pragma unroll
        for (int kk = 0; kk < C::PV_KSTEPS; ++kk)
          umma_ts<C::KIND8>(d, a + kk * 8, desc_advance(b0, kk * C::V_STEPB), C::IDESC_PV,
                            (accumulate | (uint32_t)(kk > 0)) ? 1u : 0u);
        if (split) {   // second term of P lives in the upper half of the S_t columns
#pragma unroll
          for (int kk = 0; kk < C::PV_KSTEPS; ++kk)
            umma_ts<C::KIND8>(d, a + 64 + kk * 8, desc_advance(b0, kk * C::V_STEPB), C::IDESC_PV, 1u);
        }
      };

      CFK_PROF_DECL(4)
      ok = mbar_wait(bar_q_full, 0, actx, kErrFmhaQFull);
      if (ok) ok = mbar_wait(bar_kv_full + 0, 0, actx, kErrFmhaKvFull);   // K_0 is ring index 0
      CFK_PROF_MARK(0)
      if (ok) {
        tc_fence_after_sync();
        for (int t = 0; t < 2; ++t)
          if (n_of(t) > 0) {
            issue_qk(t, 0);
            umma_commit(bar_s_full + 8 * t);
          }
        umma_commit(bar_kv_empty + 0);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int vidx = 2 * j + 1, kidx = 2 * j + 2;
        const int vslot = vidx % C::NSLOT, kslot = kidx % C::NSLOT;
        CFK_PROF_MARK(3)
        ok = mbar_wait(bar_kv_full + 8 * vslot, (vidx / C::NSLOT) & 1, actx, kErrFmhaKvFull);
        CFK_PROF_MARK(1)
        bool k_ready = false;
        for (int t = 0; t < 2 && ok; ++t) {
          if (j >= n_of(t)) continue;
          CFK_PROF_MARK(3)
          ok = mbar_wait(bar_p_full + 8 * t, j & 1, actx, kErrFmhaPFull);
          CFK_PROF_MARK(2)
          if (!ok) break;
          tc_fence_after_sync();
          issue_pv(t, vslot, j > 0 ? 1u : 0u);
          if (j + 1 < n_of(t)) {
            if (!k_ready) {
              ok = mbar_wait(bar_kv_full + 8 * kslot, (kidx / C::NSLOT) & 1, actx, kErrFmhaKvFull);
              if (!ok) break;
              tc_fence_after_sync();
              k_ready = true;
            }
            issue_qk(t, kslot);
            umma_commit(bar_s_full + 8 * t);
          } else {
            umma_commit(bar_o_full + 8 * t);
          }
        }
        if (ok) {
          umma_commit(bar_kv_empty + 8 * vslot);
          if (j + 1 < n_kv) umma_commit(bar_kv_empty + 8 * kslot);
        }
      }
      CFK_PROF_MARK(3)
      CFK_PROF_FLUSH(8, 4, true)
    }
   }
  } else {
    // =========================== softmax + epilogue ===========================
    setmaxnreg_inc<C::SOFTMAX_REGS>();
    const int t = warp >> 2;               // query tile of this warpgroup
    const int r = tid & 127;               // row within the tile == TMEM lane
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + t * 128;
    const uint32_t tO = tmem_base + lane_base + C::O_COL0 + t * HD;
    const int row_g = qblk * 256 + t * 128 + r;     // global query row
    const int n_my = n_of(t);
    // smallest last-visible-key index over the rows of this tile
    const int tile_min_lim = p.causal ? min(p.Skv - 1, qblk * 256 + t * 128 + diag_off) : p.Skv - 1;
    const float sl = p.scale_log2;

    float m_ref = 0.f;       // maximum in use (raw score units)
    float m_true = -INFINITY;
    float l = 0.f;
    bool ok = true;
    uint32_t sreg[128];

    CFK_PROF_DECL(8)
    for (int j = 0; j < n_my; ++j) {
      CFK_PROF_MARK(7)
      ok = mbar_wait_warp(bar_s_full + 8 * t, j & 1, actx, kErrFmhaSFull);
      CFK_PROF_MARK(0)
      if (!ok) break;
      tc_fence_after_sync();
      tmem_ld_x32(tS + 0, sreg + 0);
      tmem_ld_x32(tS + 32, sreg + 32);
      tmem_ld_x32(tS + 64, sreg + 64);
      tmem_ld_x32(tS + 96, sreg + 96);
      tmem_wait_ld();
      CFK_PROF_MARK(1)

      // masking: columns beyond the causal limit of this row or beyond the key length.  Whether a tile
      // needs it at all depends only on the tile, so the test costs no vote.
      if (j * C::BN + 127 > tile_min_lim) {
        int lim = p.Skv - 1;
        if (p.causal) { const int cl = row_g + diag_off; lim = cl < lim ? cl : lim; }
        lim -= j * C::BN;     // last visible local column
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (i > lim) sreg[i] = 0xff800000u;  // -inf
      }

      // row maximum: sixteen independent chains of two-input max, then a tree
      float mx[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) mx[i] = __uint_as_float(sreg[i]);
#pragma unroll
      for (int i = 16; i < 128; ++i) mx[i & 15] = fmaxf(mx[i & 15], __uint_as_float(sreg[i]));
#pragma unroll
      for (int w = 8; w >= 1; w >>= 1)
#pragma unroll
        for (int i = 0; i < w; ++i) mx[i] = fmaxf(mx[i], mx[i + w]);
      const float rowmax = mx[0];
      m_true = fmaxf(m_true, rowmax);

      if (j == 0) {
        m_ref = (rowmax == -INFINITY) ? 0.f : rowmax;
      } else {
        const bool need = (rowmax - m_ref) * sl > C::TAU;
        if (__any_sync(0xffffffffu, need)) {
          float alpha = 1.f;
          if (need) {
            alpha = ex2_approx((m_ref - rowmax) * sl);
            m_ref = rowmax;
            l *= alpha;
          }
          // O_t is complete up to tile j-1 here: the commit that released S_t(j) was issued after it.
          uint32_t oreg[32];
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            tmem_ld_x32(tO + c * 32, oreg);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
            tmem_st_x32(tO + c * 32, oreg);
          }
          tmem_wait_st();
        }
      }
      CFK_PROF_MARK(2)
      const float negm = C::PSHIFT - m_ref * sl;
      const float2 sl2 = make_float2(sl, sl), negm2 = make_float2(negm, negm);
      float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
      auto gen_p = [&](auto split_c) {
        constexpr bool SPLIT = decltype(split_c)::value;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float2 pr[16];   // the 32 probabilities of this chunk, as pairs
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float2 x = __ffma2_rn(make_float2(__uint_as_float(sreg[32 * c + 2 * j]),
                                                  __uint_as_float(sreg[32 * c + 2 * j + 1])), sl2, negm2);
          pr[j] = ((j & 3) < EMU) ? exp2_pair_fma(x) : exp2_pair_sfu(x);
          if (j & 1) acc1 = __fadd2_rn(acc1, pr[j]); else acc0 = __fadd2_rn(acc0, pr[j]);
        }
        if constexpr (C::PESZ == 2) {
          uint32_t hi[16], lo[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if constexpr (PT == kDtBF16) {
              hi[j] = pack_bf16x2(pr[j].x, pr[j].y);
              if constexpr (SPLIT)
                lo[j] = pack_bf16x2(pr[j].x - __uint_as_float(hi[j] << 16), pr[j].y - __uint_as_float(hi[j] & 0xffff0000u));
            } else {
              hi[j] = pack_f16x2(pr[j].x, pr[j].y);
            }
          }
          tmem_st_x16(tS + 16 * c, hi);
          if constexpr (PT == kDtBF16) {
            if constexpr (SPLIT) tmem_st_x16(tS + 64 + 16 * c, lo);
          }
        } else {
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) w[j] = pack_e4m3x4(pr[2 * j].x, pr[2 * j].y, pr[2 * j + 1].x, pr[2 * j + 1].y);
          tmem_st_x8(tS + 8 * c, w);
        }
      }
      };
      if constexpr (PT == kDtBF16) {
        if (split) gen_p(std::true_type{}); else gen_p(std::false_type{});
      } else {
        gen_p(std::false_type{});
      }
      l += (acc0.x + acc0.y) + (acc1.x + acc1.y);
      CFK_PROF_MARK(3)
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar_p_full + 8 * t);
      CFK_PROF_MARK(4)
    }
    CFK_PROF_MARK(7)

    if (ok && n_my > 0) {
      ok = mbar_wait_warp(bar_o_full + 8 * t, 0, actx, kErrFmhaOFull);
      if (ok) {
        tc_fence_after_sync();
        const float inv = p.out_scale / l;
        const uint32_t stage = C::O_SEPARATE ? (sOst + t * C::OTILEB) : (sQ + t * C::TILEB);
        uint32_t oreg[32];
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          tmem_ld_x32(tO + c * 32, oreg);
          tmem_wait_ld();
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float a = __uint_as_float(oreg[2 * i]) * inv, b = __uint_as_float(oreg[2 * i + 1]) * inv;
            pk[i] = p.out_bf16 ? pack_bf16x2(a, b) : pack_f16x2(a, b);
          }
          // 32 output columns = 64 bytes = four 16-byte chunks of sub-tile c/2, 128-byte swizzled
          const uint32_t row_addr = stage + (c >> 1) * C::SUBB + r * 128;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t chunk = (uint32_t)((c & 1) * 4 + i) ^ (uint32_t)(r & 7);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + chunk * 16), "r"(pk[4 * i]),
                         "r"(pk[4 * i + 1]), "r"(pk[4 * i + 2]), "r"(pk[4 * i + 3])
                         : "memory");
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(bar_o_staged + 8 * t);
        if (r == 0) {
          if (mbar_wait(bar_o_staged + 8 * t, 0, actx, kErrFmhaOStaged)) {
            tma_store_5d(&tm_o, stage, 0, qblk * 256 + t * 128, 0, head, batch);
            tma_store_commit();
            tma_store_wait_read0();
          }
        }
        if (row_g < p.Sq) {
          const size_t so = ((size_t)batch * p.H + head) * p.Sq + row_g;
          const float mref2 = m_ref * sl - C::PSHIFT;      // exponent origin of l, log2 domain
          if (p.lse) p.lse[so] = 0.69314718055994531f * (mref2 + log2f(l));
          if (p.mi) p.mi[so] = m_true * sl;
          if (p.sprime) p.sprime[so] = l * exp2f(mref2 - m_true * sl);
        }
      }
    }
    CFK_PROF_MARK(5)
    CFK_PROF_FLUSH(0, 8, (tid == 0))
  }

  // ---- tear-down ----
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

}  // namespace cfk
