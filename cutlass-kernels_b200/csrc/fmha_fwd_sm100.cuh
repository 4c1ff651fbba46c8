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
// as fmha_consumer.h:54 does) is written to TMEM - over S, or into a buffer of its own where the columns
// allow it (the three schedules are described where `mode` is set) - and consumed from there; V is used in
// its natural [key][d] layout through an MN-major operand descriptor, so neither the host-side V
// transpose (src/fmha-pipeline/fmha_forward.cu:514-532) nor the register shuffle of reg2reg.h:45-108
// exists here.  The running maximum is only moved (and O only rescaled) when the new maximum exceeds
// the one in use by more than kTau in the log2 domain; the reference rescales on every tile
// (online_softmax.h:144-165).  Both carry the same factor into O and the row sum, so O / l is
// unchanged.
#pragma once
#include <type_traits>

#include "fmha_softmax.cuh"

namespace cfk {

// EMU: of every four pairs of probabilities, how many are computed on the FMA pipe (0..3).  DUMP: the debugging
// build that also writes the raw scores (FmhaParams::s_dump); a separate instantiation keeps the test out of the loop.
template <int DT, int PT, int HD, int EMU, bool DUMP = false>
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
  const uint32_t sBar = sRing + C::NSLOT * C::SLOTB;
  uint8_t* gBar = smem_gen + (sBar - smem_base);
  // barrier map (8 bytes each)
  const uint32_t bar_q_full = sBar;
  const uint32_t bar_kv_full = sBar + 8;                   // [NSLOT]
  const uint32_t bar_kv_empty = bar_kv_full + 8 * C::NSLOT;  // [NSLOT]
  const uint32_t bar_s_full = bar_kv_empty + 8 * C::NSLOT;   // [2]
  const uint32_t bar_p_full = bar_s_full + 16;               // [2][2]: per tile, P of keys 0-63 / of keys 64-127
  const uint32_t bar_o_full = bar_p_full + 32;               // [2]
  const uint32_t bar_o_staged = bar_o_full + 16;             // [2]
  const uint32_t bar_pv_done = bar_o_staged + 16;            // [2] P in its own buffer: O_t += P_t V_j is complete
  const uint32_t bar_s_read = bar_pv_done + 16;              // [2] shared S buffer: tile t's scores are in registers (4 warps)
  const uint32_t off_misc = (bar_s_read + 16) - sBar;
  static_assert(8 + 16 * C::NSLOT + 16 + 32 + 16 + 16 + 16 + 16 + 16 <= C::BARB, "barrier block overflows");
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
      mbar_init(bar_p_full + 16 * t, 4);
      mbar_init(bar_p_full + 16 * t + 8, 4);
      mbar_init(bar_o_full + 8 * t, 1);
      mbar_init(bar_o_staged + 8 * t, 128);
      mbar_init(bar_pv_done + 8 * t, 1);
      mbar_init(bar_s_read + 8 * t, 4);
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
  // Three schedules, one per CTA:
  //  kOverS   P_t is written over S_t; Q_t K_{j+1}^T is issued after P_t(j) V_j has consumed P.  The two-term bf16 P
  //           (second term in the upper half of S_t) needs this one.
  //  kSepP    d = 64 leaves 128 columns of tensor memory free: P_t has a buffer of its own, and Q_t K_{j+1}^T is
  //           issued as soon as the first half of P_t(j) has arrived (S_t(j) has then long been read into registers),
  //           so S_t(j+1) is complete before the softmax warps have finished tile j.
  //  kSharedS d = 128 has no column to spare, but one S buffer is enough for both query tiles if the tiles take
  //           turns: S lives in it only from the Q K^T to the tcgen05.ld of the softmax warps, P_0 and P_1 take the
  //           columns of the second S buffer, and again no Q K^T waits for a P V.  Entries (tile, key tile) pass
  //           through the buffer in the order (0,0) (1,0) (0,1) (1,1) ..; the UMMA warp runs three entries ahead
  //           of the P V it issues.
  constexpr int kOverS = 0, kSepP = 1, kSharedS = 2;
  int mode = kOverS;
  if (!split) {
    if (C::SEP_P) mode = kSepP;
    else if (p.sched == 1 && n_t0 > 0 && n_t1 > 0) mode = kSharedS;
  }
  const uint32_t p_col0 = mode == kSepP ? C::P_COL0 : 128u;        // P_t at p_col0 + 64 t (kSepP, kSharedS)

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
      // Tiles enter the ring in the order the UMMA warp first uses them: K_0, then V_j, K_{j+1}.
      int idx = 0;
      bool ok = true;
      auto load_tile = [&](bool is_v, int j) {
        const int slot = idx % C::NSLOT;
        const uint32_t ph = (idx / C::NSLOT) & 1;
        ++idx;
        if (!mbar_wait(bar_kv_empty + 8 * slot, ph ^ 1u, actx, kErrFmhaKvEmpty)) { ok = false; return; }
        mbar_arrive_expect_tx(bar_kv_full + 8 * slot, is_v ? C::VTILEB : C::TILEB);
        tma_load_5d(sRing + slot * C::SLOTB, is_v ? &tm_v : &tm_k, bar_kv_full + 8 * slot, 0, j * C::BN, 0, head, batch);
      };
      if (mode != kSharedS) {
        load_tile(false, 0);
        for (int j = 0; j < n_kv && ok; ++j) {
          load_tile(true, j);
          if (j + 1 < n_kv && ok) load_tile(false, j + 1);
        }
      } else {   // K_0, K_1, then V_j, K_{j+2}
        load_tile(false, 0);
        if (n_kv > 1 && ok) load_tile(false, 1);
        for (int j = 0; j < n_kv && ok; ++j) {
          load_tile(true, j);
          if (j + 2 < n_kv && ok) load_tile(false, j + 2);
        }
      }
    }
   } else if (warp == 8) {
    // =========================== UMMA issuer ===========================
    // All 32 lanes run the loop (uniform control flow); one elected lane executes the tcgen05 instructions.
    if (n_kv > 0) {
      const uint32_t leader = elect_one();
      bool ok = true;
      // Descriptor words that do not change: Q_0 and Q_1 (K-major), and ring slot 0 seen as a K tile
      // (K-major) and as a V tile (MN-major: LBO = distance between the 64-element column groups, i.e. one
      // sub-tile; SBO = distance between groups of 8 keys).  A slot or a k-step adds a constant to the low word.
      const uint64_t aq0 = make_smem_desc(sQ, 16, C::SBO, C::SWZ);
      const uint64_t bk0 = make_smem_desc(sRing, 16, C::SBO, C::SWZ);
      const uint64_t bv0 = make_smem_desc(sRing, C::VSUBB, C::VSBO, C::VSWZ);
      auto issue_qk = [&](int t, int slot) {
        const uint64_t a0 = desc_advance_lo(aq0, t * C::TILEB);
        const uint64_t b0 = desc_advance_lo(bk0, slot * C::SLOTB);
        const uint32_t d = tmem_base + (mode == kSharedS ? 0 : t * 128);
#pragma unroll
        for (int kk = 0; kk < C::QK_KSTEPS; ++kk) {
          const uint32_t off = (kk / C::KSPS) * C::SUBB + (kk % C::KSPS) * 32;
          umma_ss_e<C::KIND8, false>(d, desc_advance_lo(a0, off), desc_advance_lo(b0, off), C::IDESC_QK, kk > 0 ? 1u : 0u,
                                     leader);
        }
      };
      // half 0: keys 0-63 of the tile, half 1: keys 64-127
      auto issue_pv_half = [&](int t, int slot, int half, uint32_t accumulate) {
        const uint64_t b0 = desc_advance_lo(bv0, slot * C::SLOTB);
        const uint32_t d = tmem_base + C::O_COL0 + t * HD;
        const uint32_t a = tmem_base + (mode == kOverS ? t * 128 : p_col0 + t * 64);
#pragma unroll
        for (int k2 = 0; k2 < C::PV_KSTEPS / 2; ++k2) {
          const int kk = half * (C::PV_KSTEPS / 2) + k2;
          umma_ts_e<C::KIND8_PV, false>(d, a + kk * 8, desc_advance_lo(b0, kk * C::V_STEPB), C::IDESC_PV,
                                     k2 > 0 ? 1u : accumulate, leader);
        }
      };
      auto issue_pv_lo = [&](int t, int slot) {
        const uint64_t b0 = desc_advance_lo(bv0, slot * C::SLOTB);
        const uint32_t d = tmem_base + C::O_COL0 + t * HD;
        const uint32_t a = tmem_base + t * 128;
        {   // second term of P lives in the upper half of the S_t columns
#pragma unroll
          for (int kk = 0; kk < C::PV_KSTEPS; ++kk)
            umma_ts_e<C::KIND8_PV, false>(d, a + 64 + kk * 8, desc_advance_lo(b0, kk * C::V_STEPB), C::IDESC_PV, 1u, leader);
        }
      };

      CFK_PROF_DECL(4)
      ok = mbar_wait_warp(bar_q_full, 0, actx, kErrFmhaQFull);
      if (mode == kSharedS) {
        // Entry k of the S buffer is (tile, key tile) = (k & 1, k >> 1) while both tiles have key tiles left, then the
        // rest of the longer one.  Ring index of K_j and V_j in the producer's order K_0 K_1 V_0 K_2 V_1 ..
        const int n_lo = n_t0 < n_t1 ? n_t0 : n_t1, total = n_t0 + n_t1;
        auto entry = [&](int k, int& t, int& j) {
          if (k < 2 * n_lo) { t = k & 1; j = k >> 1; }
          else { t = n_t0 > n_t1 ? 0 : 1; j = n_lo + (k - 2 * n_lo); }
        };
        auto idx_k = [&](int j) { return j < 2 ? j : 2 * j - 1; };
        auto idx_v = [&](int j) { return j + 2 <= n_kv ? 2 * j + 2 : (n_kv == 1 ? 1 : 2 * n_kv - 1); };
        // first / last entry that uses key tile j: tile 0's, tile 1's - or the only one
        auto first_of = [&](int t, int j) { return t == 0 || j >= n_t0; };
        auto last_of = [&](int t, int j) { return t == 1 || j >= n_t1; };
        auto do_qk = [&](int k) -> bool {
          int t, j;
          entry(k, t, j);
          const int idx = idx_k(j), slot = idx % C::NSLOT;
          if (first_of(t, j) && !mbar_wait_warp(bar_kv_full + 8 * slot, (idx / C::NSLOT) & 1, actx, kErrFmhaKvFull))
            return false;
          if (k > 0) {   // the scores of the previous entry are in its owner's registers
            int tp, jp;
            entry(k - 1, tp, jp);
            if (!mbar_wait_warp(bar_s_read + 8 * tp, (uint32_t)jp & 1u, actx, kErrFmhaSRead)) return false;
          }
          tc_fence_after_sync();
          issue_qk(t, slot);
          umma_commit_e<false>(bar_s_full + 8 * t, leader);
          if (last_of(t, j)) umma_commit_e<false>(bar_kv_empty + 8 * slot, leader);
          return true;
        };
        auto do_pv = [&](int k) -> bool {
          int t, j;
          entry(k, t, j);
          const int idx = idx_v(j), slot = idx % C::NSLOT;
          if (first_of(t, j) && !mbar_wait_warp(bar_kv_full + 8 * slot, (idx / C::NSLOT) & 1, actx, kErrFmhaKvFull))
            return false;
          if (!mbar_wait_warp(bar_p_full + 16 * t, j & 1, actx, kErrFmhaPFull)) return false;
          tc_fence_after_sync();
          issue_pv_half(t, slot, 0, j > 0 ? 1u : 0u);
          if (!mbar_wait_warp(bar_p_full + 16 * t + 8, j & 1, actx, kErrFmhaPFull)) return false;
          tc_fence_after_sync();
          issue_pv_half(t, slot, 1, 1u);
          umma_commit_e<false>(bar_pv_done + 8 * t, leader);
          if (j == n_of(t) - 1) umma_commit_e<false>(bar_o_full + 8 * t, leader);
          if (last_of(t, j)) umma_commit_e<false>(bar_kv_empty + 8 * slot, leader);
          return true;
        };
        for (int k = 0; k < 3 && k < total && ok; ++k) ok = do_qk(k);
        for (int k = 0; k < total && ok; ++k) {
          ok = do_pv(k);
          if (ok && k + 3 < total) ok = do_qk(k + 3);
        }
      } else {
      if (ok) ok = mbar_wait_warp(bar_kv_full + 0, 0, actx, kErrFmhaKvFull);   // K_0 is ring index 0
      CFK_PROF_MARK(0)
      if (ok) {
        tc_fence_after_sync();
        for (int t = 0; t < 2; ++t)
          if (n_of(t) > 0) {
            issue_qk(t, 0);
            umma_commit_e<false>(bar_s_full + 8 * t, leader);
          }
        umma_commit_e<false>(bar_kv_empty + 0, leader);
      }
      auto pv_qk_loop = [&](auto split_c, auto early_c) {     // one copy per case, as for the softmax warps
      constexpr bool SPLIT = decltype(split_c)::value;
      constexpr bool qk_early = decltype(early_c)::value;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int vidx = 2 * j + 1, kidx = 2 * j + 2;
        const int vslot = vidx % C::NSLOT, kslot = kidx % C::NSLOT;
        CFK_PROF_MARK(3)
        ok = mbar_wait_warp(bar_kv_full + 8 * vslot, (vidx / C::NSLOT) & 1, actx, kErrFmhaKvFull);
        CFK_PROF_MARK(1)
        bool k_ready = false;
        // S_t = Q_t K_{j+1}^T
        auto next_qk = [&](int t) -> bool {
          if (!k_ready) {
            if (!mbar_wait_warp(bar_kv_full + 8 * kslot, (kidx / C::NSLOT) & 1, actx, kErrFmhaKvFull)) return false;
            tc_fence_after_sync();
            k_ready = true;
          }
          issue_qk(t, kslot);
          umma_commit_e<false>(bar_s_full + 8 * t, leader);
          return true;
        };
        for (int t = 0; t < 2 && ok; ++t) {
          if (j >= n_of(t)) continue;
          const bool more = j + 1 < n_of(t);
          CFK_PROF_MARK(3)
          // with the two-term P the first-half barrier is not signalled; everything waits for the second
          if constexpr (!SPLIT) {
            ok = mbar_wait_warp(bar_p_full + 16 * t, j & 1, actx, kErrFmhaPFull);
            if (!ok) break;
            tc_fence_after_sync();
            if (qk_early && more) {   // first: the softmax warps will ask for S before they ask for O
              ok = next_qk(t);
              if (!ok) break;
            }
            issue_pv_half(t, vslot, 0, j > 0 ? 1u : 0u);
          }
          ok = mbar_wait_warp(bar_p_full + 16 * t + 8, j & 1, actx, kErrFmhaPFull);
          CFK_PROF_MARK(2)
          if (!ok) break;
          tc_fence_after_sync();
          if constexpr (SPLIT) {
            issue_pv_half(t, vslot, 0, j > 0 ? 1u : 0u);
            issue_pv_half(t, vslot, 1, 1u);
            issue_pv_lo(t, vslot);
          } else {
            issue_pv_half(t, vslot, 1, 1u);
          }
          if (mode == kSepP) umma_commit_e<false>(bar_pv_done + 8 * t, leader);
          if (!more) umma_commit_e<false>(bar_o_full + 8 * t, leader);
          if (!qk_early && more) {
            ok = next_qk(t);
            if (!ok) break;
          }
        }
        if (ok) {
          umma_commit_e<false>(bar_kv_empty + 8 * vslot, leader);
          if (j + 1 < n_kv) umma_commit_e<false>(bar_kv_empty + 8 * kslot, leader);
        }
      }
      };
      if (mode == kSepP) {
        pv_qk_loop(std::false_type{}, std::true_type{});
      } else {
        if constexpr (PT == kDtBF16) {
          if (split) pv_qk_loop(std::true_type{}, std::false_type{});
          else pv_qk_loop(std::false_type{}, std::false_type{});
        } else {
          pv_qk_loop(std::false_type{}, std::false_type{});
        }
      }
      }
      CFK_PROF_MARK(3)
      CFK_PROF_FLUSH(8, 4, (leader != 0))
    }
   }
  } else {
    // =========================== softmax + epilogue ===========================
    setmaxnreg_inc<C::SOFTMAX_REGS>();
    const int t = warp >> 2;               // query tile of this warpgroup
    const int r = tid & 127;               // row within the tile == TMEM lane
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
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
    [[maybe_unused]] uint32_t s_seen = 0u;

    CFK_PROF_DECL(8)
    // The loop over the key tiles exists once per form of the P store (two-term or plain) and per schedule: with both
    // forms of the store in one loop body every bf16 launch ran 4-7 % slower, also where no CTA used the second form,
    // and the schedule as a run-time value cost the 16-bit shapes at d = 128 another 2 %.
    auto key_tile_loop = [&](auto split_c, auto mode_c) {
    constexpr bool SPLIT = decltype(split_c)::value;
    constexpr int MODE = decltype(mode_c)::value;
    constexpr bool own_p = MODE != kOverS;     // P has a buffer of its own
    const uint32_t tS = tmem_base + lane_base + (MODE == kSharedS ? 0 : t * 128);
    const uint32_t tP = MODE == kOverS ? tS : tmem_base + lane_base + (MODE == kSepP ? C::P_COL0 : 128) + t * 64;
    for (int j = 0; j < n_my; ++j) {
      CFK_PROF_MARK(7)
      if (!(own_p && __all_sync(0xffffffffu, s_seen)))   // own_p: looked at while the previous tile's P was on its way
        ok = mbar_wait_warp(bar_s_full + 8 * t, j & 1, actx, kErrFmhaSFull);
      CFK_PROF_MARK(0)
      if (!ok) break;
      tc_fence_after_sync();
      tmem_ld_x32(tS + 0, sreg + 0);
      tmem_ld_x32(tS + 32, sreg + 32);
      tmem_ld_x32(tS + 64, sreg + 64);
      tmem_ld_x32(tS + 96, sreg + 96);
      // own_p: an early look at "P V of the previous key tile is complete", used after the row maximum (measured:
      // looking here, behind the loads, beats looking before them or only when the answer is needed, 824 against
      // 787 TFLOP/s at d = 64 fp16)
      uint32_t pv_seen = 0u;
      if (own_p && j > 0) pv_seen = mbar_test_wait(bar_pv_done + 8 * t, (uint32_t)(j - 1) & 1u);
      tmem_wait_ld();
      if constexpr (MODE == kSharedS) {   // the S buffer may take the other tile's scores
        tc_fence_before_sync();
        mbar_arrive_warp(bar_s_read + 8 * t);
      }
      CFK_PROF_MARK(1)

      if constexpr (DUMP) dump_scores(p, sreg, batch, head, row_g, j * C::BN);
      // mask, row maximum, lazy rescale of O and l, P = 2^(x - m) written over S_t, row sum
      {
        int lim = p.Skv - 1;
        if (p.causal) { const int cl = row_g + diag_off; lim = cl < lim ? cl : lim; }
        ok = softmax_step<C, PT, HD, EMU, SPLIT>(sreg, tS, tP, tO, sl, j == 0, j * C::BN + 127 > tile_min_lim,
                                                 lim - j * C::BN, bar_p_full + 16 * t, own_p ? bar_pv_done + 8 * t : 0u,
                                                 (uint32_t)(j - 1) & 1u, pv_seen, actx, m_ref, m_true, l);
        if (!ok) break;
      }
      CFK_PROF_MARK(3)
      // own_p: the scores of the next key tile are as a rule complete by now; the look overlaps the wait for the stores
      if (own_p) s_seen = mbar_test_wait(bar_s_full + 8 * t, (uint32_t)(j + 1) & 1u);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive_warp(bar_p_full + 16 * t + 8);
      CFK_PROF_MARK(4)
    }
    };
    using OverS = std::integral_constant<int, kOverS>;
    using OwnP = std::integral_constant<int, C::SEP_P ? kSepP : kSharedS>;
    if (mode != kOverS) {
      key_tile_loop(std::false_type{}, OwnP{});
    } else {
      if constexpr (PT == kDtBF16) {
        if (split) key_tile_loop(std::true_type{}, OverS{});
        else key_tile_loop(std::false_type{}, OverS{});
      } else {
        key_tile_loop(std::false_type{}, OverS{});
      }
    }
    CFK_PROF_MARK(7)

    if (ok && n_my > 0) {
      ok = mbar_wait_warp(bar_o_full + 8 * t, 0, actx, kErrFmhaOFull);
      if (ok) {
        tc_fence_after_sync();
        const uint32_t stage = C::O_SEPARATE ? (sOst + t * C::OTILEB) : (sQ + t * C::TILEB);
        stage_output<C, HD>(tO, stage, r, p.out_scale / l, p.out_bf16 != 0);
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
  settle_if_aborted(s_abort);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

}  // namespace cfk
