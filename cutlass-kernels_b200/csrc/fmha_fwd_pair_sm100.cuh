// Flash-attention forward for sm_100a on CTA pairs (tcgen05 cta_group::2): 16-bit inputs, head dimension 128.
//
// A pair of CTAs (two SMs) owns 256 consecutive query rows of one head; each CTA owns one 128-row tile.
// One thread of the leader CTA issues M = 256 UMMAs for both:
//
//   S[256 x 128 keys] = [Q of CTA 0; Q of CTA 1] K_j^T     each CTA holds 64 of the 128 keys of K_j
//   O[256 x 128]     += [P of CTA 0; P of CTA 1] V_j       each CTA holds 64 of the 128 columns of V_j
//
// so each SM fetches half of every K/V tile and reads half of the B operand from its shared memory.
// With a single query tile per CTA, tensor memory has room for what the single-CTA kernel
// (fmha_fwd_sm100.cuh) lacks: two S buffers and P buffers that do not alias them,
//
//   columns   0-127  S_A (key tiles j = 0, 2, 4, ...)      384-447  P_A
//           128-255  S_B (key tiles j = 1, 3, 5, ...)      448-511  P_B
//           256-383  O
//
// and the two softmax warpgroups take alternate KEY tiles of the same rows instead of different rows.
// Q K_{j+2}^T is issued as soon as warpgroup X has copied S_X(j) into registers, so it runs while P(j) is
// still being computed: the chain "softmax -> P V -> next Q K^T -> softmax" of the single-CTA kernel is
// gone, and a warpgroup has two UMMA periods for one tile's softmax.  The price is that the running
// maximum of a row is shared by two threads: thread r of each warpgroup hands the maximum in use to the
// other through shared memory (`mpub` barriers), keeps its own partial row sum, and the two are combined
// once at the end.  Reference counterparts: the kernels of src/fmha-pipeline (fmha_pipe_ws.h:69-365),
// online_softmax.h:87-207, fmha_epilogue.h:120-177.  Neither CTA multicasts: each loads its own halves
// with ordinary TMA copies that signal the leader's barrier.
#pragma once
#include "fmha_softmax.cuh"

namespace cfk {


template <int DT>
struct FmhaPairCfg {
  static_assert(DT == kDtF16 || DT == kDtBF16, "16-bit inputs only");
  static constexpr int HD = 128, ESZ = 2, PESZ = 2;
  static constexpr bool KIND8 = false;
  static constexpr int BM = 128, BN = 128;
  static constexpr int SUBB = 128 * 128;              // Q sub-tile: 128 rows x 128 B
  static constexpr int TILEB = 2 * SUBB;              // Q tile (and staged O tile): 32 KB
  static constexpr int KHALF_SUBB = 64 * 128;         // this CTA's 64 keys x 128 B, per 64-column span
  static constexpr int SLOTB = 16384;                 // half a K tile, or half a V tile (128 keys x 64 columns)
  static constexpr int SMEM_LIMIT = 232448;
  static constexpr int MISCB = 8192;                  // barriers (512 B) + per-row exchange arrays
  static constexpr int NSLOT = (SMEM_LIMIT - 1024 - MISCB - TILEB) / SLOTB;   // 11
  static_assert(NSLOT >= 6, "ring too small");
  static constexpr int SMEM_BYTES = 1024 + TILEB + NSLOT * SLOTB + MISCB;
  static constexpr int QK_KSTEPS = 8, PV_KSTEPS = 8;
  static constexpr int V_STEPB = 16 * 128;
  static constexpr int TMEM_COLS = 512, O_COL0 = 256, P_COL0 = 384, PCOLS = 64;
  static constexpr uint32_t FMT = (DT == kDtBF16) ? kFmtBF16 : kFmtF16;
  static constexpr uint32_t IDESC_QK = make_idesc(1, FMT, FMT, 0, 0, 256, 128);
  static constexpr uint32_t IDESC_PV = make_idesc(1, FMT, FMT, 0, 1, 256, 128);
  static constexpr int NTHREADS = 384;
  static constexpr int LAUNCH_REGS = 168, SOFTMAX_REGS = 216, AUX_REGS = 72;
  static_assert(2 * 128 * SOFTMAX_REGS + 128 * AUX_REGS <= NTHREADS * LAUNCH_REGS, "setmaxnreg would block forever");
  static constexpr float TAU = 8.0f;
  static constexpr float PSHIFT = 0.0f;
};

// tm_q / tm_o: boxes of 128 rows x all columns; tm_k: 64 keys x all columns; tm_v: 128 keys x one 64-column span.
template <int DT, int EMU, bool DUMP = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(384, 1)
fmha_fwd_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                     const FmhaParams p) {
  using C = FmhaPairCfg<DT>;
  constexpr int PT = DT;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t sQ = smem_base;                          // this CTA's Q tile; reused to stage O
  const uint32_t sRing = smem_base + C::TILEB;
  const uint32_t sBar = sRing + C::NSLOT * C::SLOTB;
  uint8_t* gBar = smem_gen + (sBar - smem_base);
  const uint32_t bar_q_full = sBar;                          // leader: Q tiles of both CTAs landed (2 arrivals)
  const uint32_t bar_kv_full = sBar + 8;                     // [NSLOT] leader: both halves of a tile landed
  const uint32_t bar_kv_empty = bar_kv_full + 8 * C::NSLOT;  // [NSLOT] each CTA: its half was consumed
  const uint32_t bar_s_full = bar_kv_empty + 8 * C::NSLOT;   // [2] each CTA: S_X ready
  const uint32_t bar_s_free = bar_s_full + 16;               // [2] leader: S_X copied to registers by both CTAs (8 warps)
  const uint32_t bar_p_full = bar_s_free + 16;               // [2] leader: P_X written by both CTAs (8 warps)
  const uint32_t bar_pv_done = bar_p_full + 16;              // [2] each CTA: O += P_X V done
  const uint32_t bar_mpub = bar_pv_done + 16;                // [2] each CTA: warpgroup X published its maxima (4 warps)
  const uint32_t bar_o_full = bar_mpub + 16;                 // each CTA: O complete
  const uint32_t bar_o_staged = bar_o_full + 8;              // each CTA: O staged in shared memory (256)
  static_assert(8 * (2 * C::NSLOT + 13) <= 448, "barrier block overflows");
  volatile uint32_t* s_tmem_base = reinterpret_cast<volatile uint32_t*>(gBar + 448);
  volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(gBar + 452);
  volatile float* m_sh = reinterpret_cast<volatile float*>(gBar + 512);        // [128] maximum in use per row
  volatile float* x_l = reinterpret_cast<volatile float*>(gBar + 1024);        // [2][128] partial row sums
  volatile float* x_ml = reinterpret_cast<volatile float*>(gBar + 2048);       // [2][128] maximum each sum refers to
  volatile float* x_mt = reinterpret_cast<volatile float*>(gBar + 3072);       // [2][128] true maxima
  const AbortCtx actx{s_abort, p.status};

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const uint32_t rank = cluster_ctarank();

  // Work item of this pair: same ordering as the single-CTA kernel (groups of heads that share L2, heaviest
  // query blocks first).
  int qblk, head, batch;
  {
    const int item = (int)(blockIdx.x >> 1);
    const int bh_total = p.B * p.H;
    const int per_group = p.group * p.nqblk;
    const int g = item / per_group;
    const int rr = item - g * per_group;
    const int left = bh_total - g * p.group;
    const int gsz = left < p.group ? left : p.group;
    qblk = p.nqblk - 1 - rr / gsz;
    const int bh = g * p.group + rr % gsz;
    batch = bh / p.H;
    head = bh - batch * p.H;
  }
  const int nkv_total = (p.Skv + C::BN - 1) / C::BN;
  const int diag_off = p.Skv - p.Sq;
  auto tiles_for = [&](int r0) -> int {
    if (r0 >= p.Sq) return 0;
    int n = nkv_total;
    if (p.causal) {
      const int last_key = r0 + 127 + diag_off;
      const int nc = last_key < 0 ? 1 : last_key / C::BN + 1;
      n = nc < n ? nc : n;
    }
    return n;
  };
  // Key tiles the pair runs: the larger need of its two query tiles.  The CTA that needs one fewer sees a fully
  // masked last tile (all probabilities zero).
  const int n_kv = max(tiles_for(qblk * 256), tiles_for(qblk * 256 + 128));
  const int row0 = qblk * 256 + (int)rank * 128;

  if (pair_should_skip(p.status)) return;   // one decision for the pair: both CTAs skip or both run

  if (tid == 0) {
    mbar_init(bar_q_full, 2);
    for (int i = 0; i < C::NSLOT; ++i) {
      mbar_init(bar_kv_full + 8 * i, 2);
      mbar_init(bar_kv_empty + 8 * i, 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(bar_s_full + 8 * x, 1);
      mbar_init(bar_s_free + 8 * x, 8);
      mbar_init(bar_p_full + 8 * x, 8);
      mbar_init(bar_pv_done + 8 * x, 1);
      mbar_init(bar_mpub + 8 * x, 4);
    }
    mbar_init(bar_o_full, 1);
    mbar_init(bar_o_staged, 256);
    *s_abort = 0u;
    fence_barrier_init();
  }
  if (warp == 8) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(s_tmem_base)), C::TMEM_COLS);
    tmem_relinquish_pair();
  }
  if (warp == 9 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_o);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();           // the peer's barriers exist before anything is signalled on them
  tc_fence_after_sync();
  const uint32_t tmem_base = *s_tmem_base;

  // bf16 only: pairs whose first row sees few keys keep P as a two-term sum (hi + lo); the second term goes
  // into the S buffer the scores came from, so for these pairs Q K_{j+2}^T waits for P_j V_j.
  bool split = false;
  if constexpr (PT == kDtBF16) {
    int visible = p.Skv;
    if (p.causal) { const int v0 = qblk * 256 + diag_off + 1; visible = v0 < visible ? v0 : visible; }
    split = visible < p.split_keys;
  }

  if (warp >= 8) {
   setmaxnreg_dec<C::AUX_REGS>();
   if (warp == 9) {
    // =========================== TMA producer (both CTAs) ===========================
    // Tiles are loaded in the order the UMMA thread uses them: K_0, K_1, then K_{j+2}, V_j for j = 0, 1, ...
    if (lane == 0 && n_kv > 0) {
      const uint32_t leader_q_full = map_to_cta(bar_q_full, 0);
      mbar_arrive_expect_tx_cluster(leader_q_full, C::TILEB);
      tma_load_5d_pair(sQ, &tm_q, leader_q_full, 0, row0, 0, head, batch);
      int idx = 0;
      auto load = [&](int which, int j) -> bool {
        const int slot = idx % C::NSLOT;
        const uint32_t ph = (idx / C::NSLOT) & 1;
        if (!mbar_wait(bar_kv_empty + 8 * slot, ph ^ 1u, actx, kErrFmhaKvEmpty)) return false;
        const uint32_t leader_full = map_to_cta(bar_kv_full + 8 * slot, 0);
        mbar_arrive_expect_tx_cluster(leader_full, C::SLOTB);
        if (which == 0)   // this CTA's 64 keys of K_j, all 128 columns
          tma_load_5d_pair(sRing + slot * C::SLOTB, &tm_k, leader_full, 0, j * C::BN + (int)rank * 64, 0, head, batch);
        else              // all 128 keys of V_j, this CTA's 64 columns
          tma_load_5d_pair(sRing + slot * C::SLOTB, &tm_v, leader_full, 0, j * C::BN, (int)rank, head, batch);
        ++idx;
        return true;
      };
      bool ok = load(0, 0);
      if (ok && n_kv > 1) ok = load(0, 1);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 2 < n_kv) ok = load(0, j + 2);
        if (ok) ok = load(1, j);
      }
    }
   } else if (warp == 8) {
    // =========================== UMMA issuer (leader CTA only) ===========================
    // All 32 lanes run the loop (uniform control flow); one elected lane executes the tcgen05 instructions.
    if (rank == 0 && n_kv > 0) {
      const uint32_t leader = elect_one();
      bool ok = true;
      const uint32_t peer_delta = map_to_cta(sBar, 1) - sBar;
      auto commit_both = [&](uint32_t bar) {
        umma_commit_e<true>(bar, leader);
        umma_commit_e<true>(bar + peer_delta, leader);
      };
      const uint64_t aq0 = make_smem_desc(sQ, 16, 1024, kSwizzle128B);
      const uint64_t bk0 = make_smem_desc(sRing, 16, 1024, kSwizzle128B);
      const uint64_t bv0 = make_smem_desc(sRing, C::SLOTB, 1024, kSwizzle128B);   // one 64-column group per CTA
      auto issue_qk = [&](int x, int slot) {
        const uint64_t b0 = desc_advance_lo(bk0, slot * C::SLOTB);
        const uint32_t d = tmem_base + x * 128;
#pragma unroll
        for (int kk = 0; kk < C::QK_KSTEPS; ++kk)
          umma_ss_e<false, true>(d, desc_advance_lo(aq0, (kk >> 2) * C::SUBB + (kk & 3) * 32),
                                 desc_advance_lo(b0, (kk >> 2) * C::KHALF_SUBB + (kk & 3) * 32), C::IDESC_QK, kk > 0 ? 1u : 0u, leader);
      };
      auto issue_pv = [&](int x, int slot, uint32_t accumulate) {
        const uint64_t b0 = desc_advance_lo(bv0, slot * C::SLOTB);
        const uint32_t d = tmem_base + C::O_COL0;
        const uint32_t a = tmem_base + C::P_COL0 + x * C::PCOLS;
#pragma unroll
        for (int kk = 0; kk < C::PV_KSTEPS; ++kk)
          umma_ts_e<false, true>(d, a + kk * 8, desc_advance_lo(b0, kk * C::V_STEPB), C::IDESC_PV, kk > 0 ? 1u : accumulate, leader);
        if (split) {   // second term of P: columns 0-63 of S_X
          const uint32_t a2 = tmem_base + x * 128;
#pragma unroll
          for (int kk = 0; kk < C::PV_KSTEPS; ++kk)
            umma_ts_e<false, true>(d, a2 + kk * 8, desc_advance_lo(b0, kk * C::V_STEPB), C::IDESC_PV, 1u, leader);
        }
      };
      auto slot_wait = [&](int i) -> bool {
        return mbar_wait_warp(bar_kv_full + 8 * (i % C::NSLOT), (i / C::NSLOT) & 1, actx, kErrFmhaKvFull);
      };
      auto qk_step = [&](int x, int i) {   // Q K^T from ring entry i into S_x, then release the entry
        tc_fence_after_sync();
        issue_qk(x, i % C::NSLOT);
        commit_both(bar_s_full + 8 * x);
        commit_both(bar_kv_empty + 8 * (i % C::NSLOT));
      };

      int idx = 0;
      CFK_PROF_DECL(8)
      ok = mbar_wait_warp(bar_q_full, 0, actx, kErrFmhaQFull);
      if (ok) ok = slot_wait(0);
      if (ok) { qk_step(0, 0); idx = 1; }
      if (ok && n_kv > 1) {
        ok = slot_wait(1);
        if (ok) { qk_step(1, 1); idx = 2; }
      }
      CFK_PROF_MARK(0)
      for (int j = 0; j < n_kv && ok; ++j) {
        const int x = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const bool has_k = j + 2 < n_kv;
        const int kidx = idx, vidx = idx + (has_k ? 1 : 0);
        if (has_k && !split) {
          ok = mbar_wait_warp(bar_s_free + 8 * x, ph, actx, kErrFmhaSFree);
          CFK_PROF_MARK(1)
          if (ok) ok = slot_wait(kidx);
          CFK_PROF_MARK(2)
          if (!ok) break;
          qk_step(x, kidx);
          CFK_PROF_MARK(3)
        }
        ok = slot_wait(vidx);
        CFK_PROF_MARK(4)
        if (ok) ok = mbar_wait_warp(bar_p_full + 8 * x, ph, actx, kErrFmhaPFull);
        CFK_PROF_MARK(5)
        if (!ok) break;
        tc_fence_after_sync();
        issue_pv(x, vidx % C::NSLOT, j > 0 ? 1u : 0u);
        commit_both(bar_pv_done + 8 * x);
        commit_both(bar_kv_empty + 8 * (vidx % C::NSLOT));
        CFK_PROF_MARK(6)
        if (has_k && split) {
          ok = slot_wait(kidx);
          if (!ok) break;
          qk_step(x, kidx);
        }
        idx = vidx + 1;
      }
      if (ok) commit_both(bar_o_full);
      CFK_PROF_MARK(7)
      CFK_PROF_FLUSH(8, 8, (leader != 0))
    }
   }
  } else {
    // =========================== softmax + epilogue (both CTAs) ===========================
    setmaxnreg_inc<C::SOFTMAX_REGS>();
    const int x = warp >> 2;               // warpgroup X takes key tiles j = X, X + 2, ...
    const int r = tid & 127;               // row within the tile == TMEM lane
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + x * 128;
    const uint32_t tP = tmem_base + lane_base + C::P_COL0 + x * C::PCOLS;
    const uint32_t tO = tmem_base + lane_base + C::O_COL0;
    const int row_g = row0 + r;
    const int tile_min_lim = p.causal ? min(p.Skv - 1, row0 + diag_off) : p.Skv - 1;
    const float sl = p.scale_log2;
    const uint32_t leader_s_free = map_to_cta(bar_s_free + 8 * x, 0);
    const uint32_t leader_p_full = map_to_cta(bar_p_full + 8 * x, 0);
    const uint32_t my_mpub = bar_mpub + 8 * x, other_mpub = bar_mpub + 8 * (x ^ 1);
    const uint32_t my_pv_done = bar_pv_done + 8 * x, other_pv_done = bar_pv_done + 8 * (x ^ 1);

    float m_ref = 0.f;        // maximum in use (raw score units), shared with the other warpgroup's thread r
    float m_l = 0.f;          // the maximum this thread's partial sum refers to
    float m_true = -INFINITY;
    float l = 0.f;
    bool ok = true;
    uint32_t sreg[128];

    CFK_PROF_DECL(8)
    for (int j = x; j < n_kv; j += 2) {
      const uint32_t ph = (j >> 1) & 1;
      CFK_PROF_MARK(7)
      ok = mbar_wait_warp(bar_s_full + 8 * x, ph, actx, kErrFmhaSFull);
      CFK_PROF_MARK(0)
      if (!ok) break;
      tc_fence_after_sync();
      tmem_ld_x32(tS + 0, sreg + 0);
      tmem_ld_x32(tS + 32, sreg + 32);
      tmem_ld_x32(tS + 64, sreg + 64);
      tmem_ld_x32(tS + 96, sreg + 96);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive_cluster_warp(leader_s_free);     // S_X may be overwritten by Q K_{j+2}^T
      CFK_PROF_MARK(1)

      if (DUMP && j < tiles_for(row0)) dump_scores(p, sreg, batch, head, row_g, j * C::BN);   // not the peer's extra tile
      if (j * C::BN + 127 > tile_min_lim) {   // this tile has masked columns for some row of the CTA
        int lim = p.Skv - 1;
        if (p.causal) { const int cl = row_g + diag_off; lim = cl < lim ? cl : lim; }
        lim -= j * C::BN;
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (i > lim) sreg[i] = 0xff800000u;  // -inf
      }
      const float rowmax = row_max128(sreg);
      m_true = fmaxf(m_true, rowmax);

      CFK_PROF_MARK(2)
      if (j == 0) {
        m_ref = (rowmax == -INFINITY) ? 0.f : rowmax;
        m_l = m_ref;
      } else {
        // the maximum in use after tile j-1, from the thread that owns this row in the other warpgroup
        ok = mbar_wait_warp(other_mpub, ((j - 1) >> 1) & 1, actx, kErrFmhaMaxPub);
        if (!ok) break;
        const float m_prev = m_sh[r];
        if (m_prev != m_l) {
          if (l != 0.f) l *= ex2_approx((m_l - m_prev) * sl);
          m_l = m_prev;
        }
        m_ref = m_prev;
        const bool need = (rowmax - m_prev) * sl > C::TAU;
        if (__any_sync(0xffffffffu, need)) {
          // O holds tiles 0..j-1 once P_{j-1} V_{j-1} is done; P_j V_j cannot start before this thread's P_j.
          ok = mbar_wait_warp(other_pv_done, ((j - 1) >> 1) & 1, actx, kErrFmhaPvDone);
          if (!ok) break;
          tc_fence_after_sync();
          float alpha = 1.f;
          if (need) {
            alpha = ex2_approx((m_prev - rowmax) * sl);
            m_ref = rowmax;
            l *= alpha;
            m_l = m_ref;
          }
          uint32_t oreg[32];
#pragma unroll 1
          for (int c = 0; c < C::HD / 32; ++c) {
            tmem_ld_x32(tO + c * 32, oreg);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
            tmem_st_x32(tO + c * 32, oreg);
          }
          tmem_wait_st();
        }
      }
      m_sh[r] = m_ref;
      mbar_arrive_warp(my_mpub);
      CFK_PROF_MARK(3)

      // P_X was last read by P_{j-2} V_{j-2}
      if (j >= 2) {
        ok = mbar_wait_warp(my_pv_done, ((j >> 1) - 1) & 1, actx, kErrFmhaPvDone);
        if (!ok) break;
      }
      CFK_PROF_MARK(4)
      const float negm = C::PSHIFT - m_ref * sl;
      if constexpr (PT == kDtBF16) {
        if (split) l += emit_p128<PT, EMU, true>(sreg, tP, tS, sl, negm);
        else l += emit_p128<PT, EMU, false>(sreg, tP, tS, sl, negm);
      } else {
        l += emit_p128<PT, EMU, false>(sreg, tP, tS, sl, negm);
      }
      CFK_PROF_MARK(5)
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive_cluster_warp(leader_p_full);
      CFK_PROF_MARK(6)
    }
    CFK_PROF_MARK(7)
    CFK_PROF_FLUSH(0, 8, (tid == 0 && rank == 0))

    // combine the two partial sums of each row (every softmax thread gets here, also after an abandoned wait)
    x_l[x * 128 + r] = l;
    x_ml[x * 128 + r] = m_l;
    x_mt[x * 128 + r] = m_true;
    named_bar_sync(1, 256);
    const float m_fin = m_sh[r];
    float l_tot = 0.f;
#pragma unroll
    for (int y = 0; y < 2; ++y) {
      const float ly = x_l[y * 128 + r];
      if (ly != 0.f) l_tot += ly * ex2_approx((x_ml[y * 128 + r] - m_fin) * sl);
    }
    m_true = fmaxf(x_mt[r], x_mt[128 + r]);

    if (ok && n_kv > 0) {
      ok = mbar_wait_warp(bar_o_full, 0, actx, kErrFmhaOFull);
      if (ok) {
        tc_fence_after_sync();
        // warpgroup X normalises and stages columns 64 X .. 64 X + 63 (one 128-byte span of the output tile)
        const float inv = p.out_scale / l_tot;
        uint32_t oreg[32];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int c = 2 * x + cc;
          tmem_ld_x32(tO + c * 32, oreg);
          tmem_wait_ld();
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float a = __uint_as_float(oreg[2 * i]) * inv, b = __uint_as_float(oreg[2 * i + 1]) * inv;
            pk[i] = p.out_bf16 ? pack_bf16x2(a, b) : pack_f16x2(a, b);
          }
          const uint32_t row_addr = sQ + x * C::SUBB + r * 128;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t chunk = (uint32_t)(cc * 4 + i) ^ (uint32_t)(r & 7);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + chunk * 16), "r"(pk[4 * i]),
                         "r"(pk[4 * i + 1]), "r"(pk[4 * i + 2]), "r"(pk[4 * i + 3])
                         : "memory");
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(bar_o_staged);
        if (tid == 0 && row0 < p.Sq) {
          if (mbar_wait(bar_o_staged, 0, actx, kErrFmhaOStaged)) {
            tma_store_5d(&tm_o, sQ, 0, row0, 0, head, batch);
            tma_store_commit();
            tma_store_wait_read0();
          }
        }
        if (x == 0 && row_g < p.Sq) {
          const size_t so = ((size_t)batch * p.H + head) * p.Sq + row_g;
          const float mref2 = m_fin * sl - C::PSHIFT;
          if (p.lse) p.lse[so] = 0.69314718055994531f * (mref2 + log2f(l_tot));
          if (p.mi) p.mi[so] = m_true * sl;
          if (p.sprime) p.sprime[so] = l_tot * exp2f(mref2 - m_true * sl);
        }
      }
    }
  }

  // ---- tear-down: no CTA leaves while its peer may still read its shared memory or signal its barriers
  settle_if_aborted(s_abort);
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 8) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
  }
}

}  // namespace cfk
