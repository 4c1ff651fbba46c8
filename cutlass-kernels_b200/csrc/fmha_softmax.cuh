// Pieces shared by the FMHA forward kernels (single-CTA and CTA-pair): tile configuration, the exp2
// variants, the per-tile softmax step of a row-owning thread, and the staging of an output tile.
// Reference counterparts: online_softmax.h:87-207 (onlineSoftmaxAndRescale), fmha_consumer.h:54 (P is
// rounded to the GEMM-II operand type, unnormalised), fmha_epilogue.h:120-177 (normalise, stage, TMA store).
#pragma once
#include <type_traits>

#include "common.cuh"
#include "fmha_params.h"

namespace cfk {

template <int DT, int PT, int HD>
struct FmhaCfg {
  // DT: element type of Q and K; PT: element type of P and of V (they meet in the second GEMM and must be of one MMA
  // kind).  PT == DT everywhere except the hybrid mode DT = e4m3, PT = fp16, which is what the reference runs for
  // --prec-type=2 unless it is built with GEMM2FP8 (src/fmha-pipeline/fmha_forward.cu:446-450).
  static constexpr int ESZ = (DT == kDtE4M3) ? 1 : 2;
  static constexpr int PESZ = (PT == kDtE4M3) ? 1 : 2;
  static_assert(ESZ == PESZ || (DT == kDtE4M3 && PT == kDtF16), "unsupported mix of operand types");
  static constexpr bool KIND8 = (ESZ == 1);        // MMA kind of Q K^T
  static constexpr bool KIND8_PV = (PESZ == 1);    // MMA kind of P V
  static constexpr int BM = 128, BN = 128;
  static constexpr int ROWB = HD * ESZ;            // bytes per row of a Q/K/V tile
  static constexpr int SPANB = ROWB < 128 ? ROWB : 128;   // swizzle span: 128 bytes, or the whole 64-byte row (e4m3, d = 64)
  static_assert(ROWB % SPANB == 0 && (SPANB == 128 || SPANB == 64), "rows must be whole swizzle spans");
  static constexpr uint32_t SWZ = SPANB == 128 ? kSwizzle128B : kSwizzle64B;
  static constexpr int SBO = 8 * SPANB;            // bytes between groups of 8 rows of a sub-tile
  static constexpr int KSPS = SPANB / 32;          // UMMA k-steps (32 bytes of reduction) per span
  static constexpr int NSUB = ROWB / SPANB;        // span-wide sub-tiles per tile
  static constexpr int SUBB = 128 * SPANB;         // bytes per sub-tile (128 rows x one span)
  static constexpr int TILEB = NSUB * SUBB;        // bytes per Q/K tile
  // V tile: same quantities for rows of HD * PESZ bytes
  static constexpr int VROWB = HD * PESZ;
  static constexpr int VSPANB = VROWB < 128 ? VROWB : 128;
  static constexpr uint32_t VSWZ = VSPANB == 128 ? kSwizzle128B : kSwizzle64B;
  static constexpr int VSBO = 8 * VSPANB;
  static constexpr int VSUBB = 128 * VSPANB;
  static constexpr int VTILEB = (VROWB / VSPANB) * VSUBB;
  static constexpr int SLOTB = VTILEB > TILEB ? VTILEB : TILEB;   // ring slot: holds a K tile or a V tile
  static constexpr int ONSUB = HD * 2 / 128;       // output is always 16 bit, in 128-byte spans
  static constexpr int OSUBB = 128 * 128;
  static constexpr int OTILEB = ONSUB * OSUBB;
  static constexpr bool O_SEPARATE = (OTILEB > TILEB);  // else O is staged over the Q tile
  static constexpr int SMEM_LIMIT = 232448;
  static constexpr int FIXEDB = 2 * TILEB + (O_SEPARATE ? 2 * OTILEB : 0);
  static constexpr int BARB = 512;
  static constexpr int NSLOT_FIT = (SMEM_LIMIT - 1024 - BARB - FIXEDB) / SLOTB;
  static constexpr int NSLOT = NSLOT_FIT > 8 ? 8 : NSLOT_FIT;
  static_assert(NSLOT >= 3, "ring too small");
  static constexpr int SMEM_BYTES = 1024 + FIXEDB + NSLOT * SLOTB + BARB;
  static constexpr int QK_KSTEPS = ROWB / 32;      // each UMMA consumes 32 bytes of K extent
  static constexpr int PV_KSTEPS = BN * PESZ / 32;
  static constexpr int V_STEPB = (32 / PESZ) * VSPANB;   // bytes between the key groups of successive UMMAs of P V
  static constexpr int PCOLS = BN * PESZ / 4;      // TMEM columns taken by P
  static constexpr int TMEM_COLS = 512;
  static constexpr int O_COL0 = 256;
  // Head dimension 64 leaves 128 columns of tensor memory free (2 x S + 2 x O = 384): P gets buffers of its own
  // there instead of being written over S, so the next Q K^T of a tile does not have to wait for its P V.
  static constexpr bool SEP_P = (HD == 64);
  static constexpr int P_COL0 = 384;               // P_t at P_COL0 + 64 t (SEP_P only)
  static constexpr uint32_t FMT_IN = (DT == kDtBF16) ? kFmtBF16 : 0u;   // f16 / e4m3 are both code 0
  static constexpr uint32_t FMT_P = (PT == kDtBF16) ? kFmtBF16 : 0u;
  static constexpr uint32_t IDESC_QK = make_idesc(1, FMT_IN, FMT_IN, 0, 0, BM, BN);
  static constexpr uint32_t IDESC_PV = make_idesc(1, FMT_P, FMT_P, 0, 1, BM, HD);   // A = P and B = V share PT
  static constexpr int NTHREADS = 384;
  // Register budget after setmaxnreg.  The pool is what the CTA was launched with: 384 threads at the
  // 168 registers a 384-thread launch bound allows.  setmaxnreg.inc blocks until the registers it asks
  // for are free, with no time limit, so the sum below must never exceed that pool.
  static constexpr int LAUNCH_REGS = 168, SOFTMAX_REGS = 216, AUX_REGS = 72;
  static_assert(2 * 128 * SOFTMAX_REGS + 128 * AUX_REGS <= NTHREADS * LAUNCH_REGS, "setmaxnreg would block forever");
  // log2-domain slack before the running maximum is moved, and a constant exponent offset that puts
  // P into the well-represented range of its type (it cancels in O / l).  For e4m3 the two share the head-room
  // below the format's largest value (448): 2^(PSHIFT + TAU) = 256.  An even split moves the maximum far less
  // often than PSHIFT = 6, TAU = 2 did (then one row group in six asked for a rescale on N(0,1) inputs), and values
  // down to 2^-10 of the row's reference maximum still fall into the normal range of the format.
  static constexpr float TAU = (PT == kDtE4M3) ? 4.0f : 8.0f;
  static constexpr float PSHIFT = (PT == kDtE4M3) ? 4.0f : 0.0f;
};

// exp2 of a pair of log2-domain scores on the special-function unit ...
__device__ __forceinline__ float2 exp2_pair_sfu(float2 x) { return make_float2(ex2_approx(x.x), ex2_approx(x.y)); }
// ... or on the FMA pipe: x = n + f with n = round(x), f in [-0.5, 0.5]; 2^f by a cubic whose relative
// error (7.5e-5) is below the rounding step of every P format; 2^n by adding n to the exponent bits.
// The special-function unit delivers 16 results per clock per SM, exactly what the tensor core consumes
// at D=128, so a share of the exponentials is moved here (packed two-wide FMA instructions).
// QUAD: a quadratic instead (minimax on [-0.5, 0.5], relative error 1.7e-3) for a P format whose rounding step is
// far above that (e4m3: 6e-2); one instruction less per pair where the softmax warps are the bound.
constexpr float kExp2Q0 = 1.00044314f, kExp2Q1 = 0.70344801f, kExp2Q2 = 0.23842894f;
template <bool QUAD = false>
__device__ __forceinline__ float2 exp2_pair_fma(float2 x) {
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 t = __fadd2_rn(x, make_float2(12582912.f, 12582912.f));      // 1.5 * 2^23: n sits in the low bits
  const float2 nf = __fadd2_rn(t, make_float2(-12582912.f, -12582912.f));
  const float2 f = __ffma2_rn(nf, make_float2(-1.f, -1.f), x);
  float2 q;
  if constexpr (QUAD) {
    q = __ffma2_rn(make_float2(kExp2Q2, kExp2Q2), f, make_float2(kExp2Q1, kExp2Q1));
    q = __ffma2_rn(q, f, make_float2(kExp2Q0, kExp2Q0));
  } else {
    q = __ffma2_rn(make_float2(0.0551716648f, 0.0551716648f), f, make_float2(0.2426111251f, 0.2426111251f));
    q = __ffma2_rn(q, f, make_float2(0.6932609677f, 0.6932609677f));
    q = __ffma2_rn(q, f, make_float2(0.9999280572f, 0.9999280572f));
  }
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

// Row maximum of the N scores a thread holds: eight independent chains of three-input maxima, then a tree.  The
// three-input form runs at half the rate of the two-input one, so the pipe time is the same, but it takes half the
// issue slots, which the two softmax warps of a scheduler share with everything else they do.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
template <int N>
__device__ __forceinline__ float row_max_n(const uint32_t (&sreg)[N]) {
  static_assert(N >= 24 && N % 8 == 0, "row_max_n: unsupported width");
  float mx[8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
    mx[i] = max3(__uint_as_float(sreg[i]), __uint_as_float(sreg[8 + i]), __uint_as_float(sreg[16 + i]));
  constexpr int REST = (N - 24) / 16 * 16;
#pragma unroll
  for (int i = 24; i < 24 + REST; i += 16)
#pragma unroll
    for (int k = 0; k < 8; ++k) mx[k] = max3(mx[k], __uint_as_float(sreg[i + k]), __uint_as_float(sreg[i + 8 + k]));
  if constexpr (24 + REST < N) {
#pragma unroll
    for (int k = 0; k < 8; ++k) mx[k] = fmaxf(mx[k], __uint_as_float(sreg[24 + REST + k]));
  }
  const float a = max3(mx[0], mx[1], mx[2]), b = max3(mx[3], mx[4], mx[5]);
  return max3(a, b, fmaxf(mx[6], mx[7]));
}
__device__ __forceinline__ float row_max128(const uint32_t (&sreg)[128]) { return row_max_n<128>(sreg); }

// P = 2^(s * sl + negm) for the N scores a thread holds of a row (N = 128: the whole key tile; 64: one half of it),
// rounded to the operand type and stored to tensor memory at tP (N/2 columns, N/4 for e4m3); with SPLIT (bf16) the
// rounding remainder goes to tLo as a second bf16 term.  Returns the sum of the N probabilities.
// With HALF_ARRIVE the first half of P is released on its own: once its stores have had the time of the next
// chunk's exponentials to land, the warp arrives on `bar_half`, and the UMMA thread starts P V on those keys while the
// second half is still being computed.
template <int N, int PT, int EMU, bool SPLIT, bool HALF_ARRIVE = false>
__device__ __forceinline__ float emit_p(const uint32_t (&sreg)[N], uint32_t tP, uint32_t tLo, float sl, float negm,
                                        uint32_t bar_half = 0u) {
  const float2 sl2 = make_float2(sl, sl), negm2 = make_float2(negm, negm);
  float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
  for (int c = 0; c < N / 32; ++c) {
    float2 pr[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float2 x = __ffma2_rn(make_float2(__uint_as_float(sreg[32 * c + 2 * j]),
                                              __uint_as_float(sreg[32 * c + 2 * j + 1])), sl2, negm2);
      pr[j] = ((j & 3) < EMU) ? exp2_pair_fma<(PT == kDtE4M3)>(x) : exp2_pair_sfu(x);
      if (j & 1) acc1 = __fadd2_rn(acc1, pr[j]); else acc0 = __fadd2_rn(acc0, pr[j]);
    }
    if constexpr (HALF_ARRIVE) {
      if (c == N / 64) {   // the stores of the first half have had the time of this chunk's exponentials to land
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive_warp(bar_half);
      }
    }
    if constexpr (PT == kDtE4M3) {   // 32 probabilities = 8 words = 8 columns
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) w[j] = pack_e4m3x4(pr[2 * j].x, pr[2 * j].y, pr[2 * j + 1].x, pr[2 * j + 1].y);
      tmem_st_x8(tP + 8 * c, w);
    } else {
      uint32_t hi[16];
      [[maybe_unused]] uint32_t lo[16];
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
      tmem_st_x16(tP + 16 * c, hi);
      if constexpr (SPLIT) tmem_st_x16(tLo + 16 * c, lo);
    }
  }
  return (acc0.x + acc0.y) + (acc1.x + acc1.y);
}
template <int PT, int EMU, bool SPLIT>
__device__ __forceinline__ float emit_p128(const uint32_t (&sreg)[128], uint32_t tP, uint32_t tLo, float sl, float negm) {
  return emit_p<128, PT, EMU, SPLIT>(sreg, tP, tLo, sl, negm);
}

// Debugging only: the `n` raw scores of query row `row_g` against keys key0 .. key0+n-1 (held by the calling thread,
// before scale and mask) go to S[b][h][row][key], rounded to fp16 / bf16.  The reference writes the same tile from its
// GEMM-I accumulator fragment (fmha_consumer.h:31-42).
template <int N>
__device__ __forceinline__ void dump_scores(const FmhaParams& p, const uint32_t (&sreg)[N], int batch, int head,
                                            int row_g, int key0) {
  if (row_g >= p.Sq) return;
  uint16_t* dst = reinterpret_cast<uint16_t*>(p.s_dump) + (((size_t)batch * p.H + head) * p.Sq + row_g) * (size_t)p.Skv + key0;
  const int left = p.Skv - key0;
  // fully unrolled with constant indices: the score registers must not be addressed dynamically
#pragma unroll
  for (int i = 0; i < N; ++i) {
    if (i < left) {
      const float v = __uint_as_float(sreg[i]);
      dst[i] = p.s_dump_bf16 ? (uint16_t)(pack_bf16x2(v, 0.f) & 0xffffu) : (uint16_t)(pack_f16x2(v, 0.f) & 0xffffu);
    }
  }
}

// O row (fp32, `HD` columns at tO) *= alpha, in chunks of 32 columns.
template <int HD>
__device__ __forceinline__ void rescale_o_row(uint32_t tO, float alpha) {
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

// One key tile of the online softmax for the thread that owns a query row.  On entry sreg[0..127] holds
// the row's raw scores (S_t, fp32 bits); on exit P has been written to tensor memory at tP (over S_t, or a buffer
// of its own; tcgen05.st issued, not yet waited for) and m_ref / m_true / l are updated.  `first`: first
// key tile of the row; `mask_tile`: this tile contains masked columns for some row, `lim` is this row's last visible
// column.  `bar_half`: barrier that gets one arrival per warp once P of the first 64 keys is in tensor memory; not
// used with the two-term P (SPLIT, bf16 only), whose second term goes to the upper half of S_t.
// When P has a buffer of its own (`bar_pv_done` != 0) the S buffer no longer says that P V of the previous key tile
// has run (the next Q K^T was issued before it), so the thread waits for `bar_pv_done` before it touches O_t or the
// P buffer again.  Returns false if
// that wait gave up.  A look at a barrier costs one to several hundred clocks even when the barrier is complete
// (the tensor core's operand reads keep the shared-memory port busy), so the caller looks early, with a test that
// cannot put the warp to sleep, and hands the answer in.
template <class CFG, int PT, int HD, int EMU, bool SPLIT>
__device__ __forceinline__ bool softmax_step(uint32_t (&sreg)[128], uint32_t tS, uint32_t tP, uint32_t tO, float sl,
                                             bool first, bool mask_tile, int lim, uint32_t bar_half,
                                             uint32_t bar_pv_done, uint32_t pv_parity, uint32_t pv_seen,
                                             const AbortCtx& actx, float& m_ref, float& m_true, float& l) {
  // masking: columns beyond the causal limit of this row or beyond the key length.  Whether a tile
  // needs it at all depends only on the tile, so the test costs no vote.
  if (mask_tile) {   // lim: last visible local column of this row
#pragma unroll
    for (int i = 0; i < 128; ++i)
      if (i > lim) sreg[i] = 0xff800000u;  // -inf
  }
  const float rowmax = row_max_n<128>(sreg);
  m_true = fmaxf(m_true, rowmax);
  if (bar_pv_done != 0u && !first) {   // `pv_seen`: an early look (issued before the row maximum) found it complete
    if (!__all_sync(0xffffffffu, pv_seen) && !mbar_wait_warp(bar_pv_done, pv_parity, actx, kErrFmhaPvDone)) return false;
    tc_fence_after_sync();
  }
  if (first) {
    m_ref = (rowmax == -INFINITY) ? 0.f : rowmax;
  } else {
    const bool need = (rowmax - m_ref) * sl > CFG::TAU;
    if (__any_sync(0xffffffffu, need)) {
      float alpha = 1.f;
      if (need) {
        alpha = ex2_approx((m_ref - rowmax) * sl);
        m_ref = rowmax;
        l *= alpha;
      }
      // O_t is complete up to tile j-1 here: the commit that released S_t(j) was issued after it (P over S), or
      // the wait above has seen it.
      rescale_o_row<HD>(tO, alpha);
    }
  }
  const float negm = CFG::PSHIFT - m_ref * sl;
  if constexpr (SPLIT) l += emit_p<128, PT, EMU, true>(sreg, tP, tS + 64, sl, negm);
  else l += emit_p<128, PT, EMU, false, true>(sreg, tP, 0u, sl, negm, bar_half);
  return true;
}

// O_t (fp32, tensor memory) * inv -> 16 bit -> shared-memory tile in the 128-byte swizzled layout the TMA
// store reads ([64-column span][row][128 B]); `r` is this thread's row.
template <class CFG, int HD>
__device__ __forceinline__ void stage_output(uint32_t tO, uint32_t stage, int r, float inv, bool out_bf16) {
  uint32_t oreg[32];
#pragma unroll
  for (int c = 0; c < HD / 32; ++c) {
    tmem_ld_x32(tO + c * 32, oreg);
    tmem_wait_ld();
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float a = __uint_as_float(oreg[2 * i]) * inv, b = __uint_as_float(oreg[2 * i + 1]) * inv;
      pk[i] = out_bf16 ? pack_bf16x2(a, b) : pack_f16x2(a, b);
    }
    // 32 output columns = 64 bytes = four 16-byte chunks of sub-tile c/2, 128-byte swizzled
    const uint32_t row_addr = stage + (c >> 1) * CFG::OSUBB + r * 128;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t chunk = (uint32_t)((c & 1) * 4 + i) ^ (uint32_t)(r & 7);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + chunk * 16), "r"(pk[4 * i]),
                   "r"(pk[4 * i + 1]), "r"(pk[4 * i + 2]), "r"(pk[4 * i + 3])
                   : "memory");
    }
  }
}

}  // namespace cfk
