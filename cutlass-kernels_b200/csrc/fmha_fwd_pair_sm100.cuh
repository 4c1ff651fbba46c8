// Flash-attention forward for sm_100a on CTA pairs (tcgen05 cta_group::2): 16-bit inputs, head dimension 128.
//
// Same algorithm, roles and tensor-memory plan as fmha_fwd_sm100.cuh, but two CTAs on two SMs share every
// key/value tile.  A pair owns 512 consecutive query rows = four 128-row tiles g = 4i + 2t + r (r: CTA rank,
// t: which of the CTA's two tiles), so the tiles of one UMMA (t fixed, r = 0/1) are neighbours and, under a
// causal mask, differ by at most one key tile.  One thread of the leader CTA issues M = 256 UMMAs:
//
//   S_t[256 x 128 keys] = [Q_t of CTA 0; Q_t of CTA 1] K_j^T     each CTA holds 64 of the 128 keys of K_j
//   O_t[256 x 128]     += [P_t of CTA 0; P_t of CTA 1] V_j       each CTA holds 64 of the 128 columns of V_j
//
// so every SM reads half of the B operand from its shared memory and fetches half of every K/V tile from
// L2.  With both operands of Q K^T in shared memory the single-CTA kernel is limited by the operand read
// rate of the tensor core (its 128 x 128 x 16 instruction reads 8 KB per 64 clocks); the pair's
// instruction reads 6 KB per SM for the same work.  Rows of S_t and O_t stay inside the CTA that owns the
// query rows, so the softmax is unchanged; the softmax threads of both CTAs arrive on the leader's barriers.
// Neither CTA multicasts: each one loads its own half with an ordinary TMA copy that signals the leader.
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
  static constexpr bool O_SEPARATE = false;
  static constexpr int SMEM_LIMIT = 232448;
  static constexpr int BARB = 512;
  static constexpr int NSLOT = (SMEM_LIMIT - 1024 - BARB - 2 * TILEB) / SLOTB;   // 10
  static_assert(NSLOT >= 4, "ring too small");
  static constexpr int SMEM_BYTES = 1024 + 2 * TILEB + NSLOT * SLOTB + BARB;
  static constexpr int QK_KSTEPS = 8, PV_KSTEPS = 8;
  static constexpr int V_STEPB = 16 * 128;
  static constexpr int TMEM_COLS = 512, O_COL0 = 256;
  static constexpr uint32_t FMT = (DT == kDtBF16) ? kFmtBF16 : kFmtF16;
  static constexpr uint32_t IDESC_QK = make_idesc(1, FMT, FMT, 0, 0, 256, 128);
  static constexpr uint32_t IDESC_PV = make_idesc(1, FMT, FMT, 0, 1, 256, 128);
  static constexpr int NTHREADS = 384;
  static constexpr int LAUNCH_REGS = 168, SOFTMAX_REGS = 216, AUX_REGS = 72;
  static_assert(2 * 128 * SOFTMAX_REGS + 128 * AUX_REGS <= NTHREADS * LAUNCH_REGS, "setmaxnreg would block forever");
  static constexpr float TAU = 8.0f;
  static constexpr float PSHIFT = 0.0f;
};

// tm_k: box of 64 keys x all columns; tm_v: box of 128 keys x one 64-column span.
template <int DT, int EMU>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(384, 1)
fmha_fwd_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                     const FmhaParams p) {
  using C = FmhaPairCfg<DT>;
  constexpr int HD = C::HD;
  constexpr int PT = DT;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t sQ = smem_base;                          // 2 tiles; reused to stage O
  const uint32_t sRing = smem_base + 2 * C::TILEB;
  const uint32_t sBar = sRing + C::NSLOT * C::SLOTB;
  uint8_t* gBar = smem_gen + (sBar - smem_base);
  const uint32_t bar_q_full = sBar;                          // leader: Q tiles of both CTAs landed
  const uint32_t bar_kv_full = sBar + 8;                     // [NSLOT] leader: both halves of a tile landed
  const uint32_t bar_kv_empty = bar_kv_full + 8 * C::NSLOT;  // [NSLOT] each CTA: its half was consumed
  const uint32_t bar_s_full = bar_kv_empty + 8 * C::NSLOT;   // [2] each CTA: S_t ready
  const uint32_t bar_p_full = bar_s_full + 16;               // [2] leader: P_t written by both CTAs (256 arrivals)
  const uint32_t bar_o_full = bar_p_full + 16;               // [2] each CTA: O_t complete
  const uint32_t bar_o_staged = bar_o_full + 16;             // [2] each CTA: O_t staged in shared memory
  const uint32_t off_misc = (bar_o_staged + 16) - sBar;
  volatile uint32_t* s_tmem_base = reinterpret_cast<volatile uint32_t*>(gBar + off_misc);
  volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(gBar + off_misc + 4);
  const AbortCtx actx{s_abort, p.status};

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const uint32_t rank = cluster_ctarank();

  // Work item of this pair (p.nqblk counts 512-row blocks here); same ordering as the single-CTA kernel.
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
  auto tiles_for = [&](int row0) -> int {
    if (row0 >= p.Sq) return 0;
    int n = nkv_total;
    if (p.causal) {
      const int last_key = row0 + 127 + diag_off;
      const int nc = last_key < 0 ? 1 : last_key / C::BN + 1;
      n = nc < n ? nc : n;
    }
    return n;
  };
  // Key tiles the pair runs for tile t: the larger need of the two neighbouring query tiles.  The CTA whose
  // own tile needs one fewer sees a fully masked last tile (all probabilities zero).
  auto pair_tiles = [&](int t) -> int {
    const int a = tiles_for((qblk * 4 + 2 * t) * 128), b = tiles_for((qblk * 4 + 2 * t + 1) * 128);
    return a > b ? a : b;
  };
  const int n_t0 = pair_tiles(0), n_t1 = pair_tiles(1);
  auto n_of = [&](int t) -> int { return t == 0 ? n_t0 : n_t1; };
  const int n_kv = n_t0 > n_t1 ? n_t0 : n_t1;
  auto row0_of = [&](int t) -> int { return (qblk * 4 + 2 * t + (int)rank) * 128; };

  if (cta_should_skip(p.status)) return;   // both CTAs of a pair read the same word

  if (tid == 0) {
    mbar_init(bar_q_full, 2);
    for (int i = 0; i < C::NSLOT; ++i) {
      mbar_init(bar_kv_full + 8 * i, 2);
      mbar_init(bar_kv_empty + 8 * i, 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar_s_full + 8 * t, 1);
      mbar_init(bar_p_full + 8 * t, 256);
      mbar_init(bar_o_full + 8 * t, 1);
      mbar_init(bar_o_staged + 8 * t, 128);
    }
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

  // bf16 only: pairs whose first row sees few keys keep P as a two-term sum (hi + lo).
  bool split = false;
  if constexpr (PT == kDtBF16) {
    int visible = p.Skv;
    if (p.causal) { const int v0 = qblk * 512 + diag_off + 1; visible = v0 < visible ? v0 : visible; }
    split = visible < p.split_keys;
  }

  if (warp >= 8) {
   setmaxnreg_dec<C::AUX_REGS>();
   if (warp == 9) {
    // =========================== TMA producer (both CTAs) ===========================
    if (lane == 0 && n_kv > 0) {
      const uint32_t leader_q_full = map_to_cta(bar_q_full, 0);
      const uint32_t q_bytes = (n_t0 > 0 ? C::TILEB : 0) + (n_t1 > 0 ? C::TILEB : 0);
      mbar_arrive_expect_tx_cluster(leader_q_full, q_bytes);
      for (int t = 0; t < 2; ++t)
        if (n_of(t) > 0) tma_load_5d_pair(sQ + t * C::TILEB, &tm_q, leader_q_full, 0, row0_of(t), 0, head, batch);
      int idx = 0;
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        for (int which = 0; which < 2; ++which, ++idx) {
          const int slot = idx % C::NSLOT;
          const uint32_t ph = (idx / C::NSLOT) & 1;
          if (!mbar_wait(bar_kv_empty + 8 * slot, ph ^ 1u, actx, kErrFmhaKvEmpty)) { ok = false; break; }
          const uint32_t leader_full = map_to_cta(bar_kv_full + 8 * slot, 0);
          mbar_arrive_expect_tx_cluster(leader_full, C::SLOTB);
          if (which == 0)   // this CTA's 64 keys of K_j, all 128 columns
            tma_load_5d_pair(sRing + slot * C::SLOTB, &tm_k, leader_full, 0, j * C::BN + (int)rank * 64, 0, head, batch);
          else              // all 128 keys of V_j, this CTA's 64 columns
            tma_load_5d_pair(sRing + slot * C::SLOTB, &tm_v, leader_full, 0, j * C::BN, (int)rank, head, batch);
        }
      }
    }
   } else if (warp == 8) {
    // =========================== UMMA issuer (leader CTA only) ===========================
    if (lane == 0 && rank == 0 && n_kv > 0) {
      bool ok = true;
      auto commit_both = [&](uint32_t bar) {
        umma_commit_pair(bar);
        umma_commit_pair(map_to_cta(bar, 1));
      };
      auto issue_qk = [&](int t, int slot) {
        const uint64_t a0 = make_smem_desc(sQ + t * C::TILEB, 16, 1024, kSwizzle128B);
        const uint64_t b0 = make_smem_desc(sRing + slot * C::SLOTB, 16, 1024, kSwizzle128B);
        const uint32_t d = tmem_base + t * 128;
#pragma unroll
        for (int kk = 0; kk < C::QK_KSTEPS; ++kk)
          umma_ss_pair<false>(d, desc_advance(a0, (kk >> 2) * C::SUBB + (kk & 3) * 32),
                              desc_advance(b0, (kk >> 2) * C::KHALF_SUBB + (kk & 3) * 32), C::IDESC_QK, kk > 0 ? 1u : 0u);
      };
      auto issue_pv = [&](int t, int slot, uint32_t accumulate) {
        // this CTA's half of V_j: [128 keys][128 B = 64 columns], columns contiguous (MN-major)
        const uint64_t b0 = make_smem_desc(sRing + slot * C::SLOTB, C::SLOTB, 1024, kSwizzle128B);
        const uint32_t d = tmem_base + C::O_COL0 + t * HD;
        const uint32_t a = tmem_base + t * 128;
#pragma unroll
        for (int kk = 0; kk < C::PV_KSTEPS; ++kk)
          umma_ts_pair<false>(d, a + kk * 8, desc_advance(b0, kk * C::V_STEPB), C::IDESC_PV,
                              (accumulate | (uint32_t)(kk > 0)) ? 1u : 0u);
        if (split) {
#pragma unroll
          for (int kk = 0; kk < C::PV_KSTEPS; ++kk)
            umma_ts_pair<false>(d, a + 64 + kk * 8, desc_advance(b0, kk * C::V_STEPB), C::IDESC_PV, 1u);
        }
      };

      ok = mbar_wait(bar_q_full, 0, actx, kErrFmhaQFull);
      if (ok) ok = mbar_wait(bar_kv_full + 0, 0, actx, kErrFmhaKvFull);
      if (ok) {
        tc_fence_after_sync();
        for (int t = 0; t < 2; ++t)
          if (n_of(t) > 0) {
            issue_qk(t, 0);
            commit_both(bar_s_full + 8 * t);
          }
        commit_both(bar_kv_empty + 0);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int vidx = 2 * j + 1, kidx = 2 * j + 2;
        const int vslot = vidx % C::NSLOT, kslot = kidx % C::NSLOT;
        ok = mbar_wait(bar_kv_full + 8 * vslot, (vidx / C::NSLOT) & 1, actx, kErrFmhaKvFull);
        bool k_ready = false;
        for (int t = 0; t < 2 && ok; ++t) {
          if (j >= n_of(t)) continue;
          ok = mbar_wait(bar_p_full + 8 * t, j & 1, actx, kErrFmhaPFull);
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
            commit_both(bar_s_full + 8 * t);
          } else {
            commit_both(bar_o_full + 8 * t);
          }
        }
        if (ok) {
          commit_both(bar_kv_empty + 8 * vslot);
          if (j + 1 < n_kv) commit_both(bar_kv_empty + 8 * kslot);
        }
      }
    }
   }
  } else {
    // =========================== softmax + epilogue (both CTAs) ===========================
    setmaxnreg_inc<C::SOFTMAX_REGS>();
    const int t = warp >> 2;
    const int r = tid & 127;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + t * 128;
    const uint32_t tO = tmem_base + lane_base + C::O_COL0 + t * HD;
    const int row0 = row0_of(t);
    const int row_g = row0 + r;
    const int n_my = n_of(t);
    const int tile_min_lim = p.causal ? min(p.Skv - 1, row0 + diag_off) : p.Skv - 1;
    const float sl = p.scale_log2;
    const uint32_t leader_p_full = map_to_cta(bar_p_full + 8 * t, 0);

    float m_ref = 0.f, m_true = -INFINITY, l = 0.f;
    bool ok = true;
    uint32_t sreg[128];

    for (int j = 0; j < n_my; ++j) {
      ok = mbar_wait_warp(bar_s_full + 8 * t, j & 1, actx, kErrFmhaSFull);
      if (!ok) break;
      tc_fence_after_sync();
      tmem_ld_x32(tS + 0, sreg + 0);
      tmem_ld_x32(tS + 32, sreg + 32);
      tmem_ld_x32(tS + 64, sreg + 64);
      tmem_ld_x32(tS + 96, sreg + 96);
      tmem_wait_ld();
      {
        int lim = p.Skv - 1;
        if (p.causal) { const int cl = row_g + diag_off; lim = cl < lim ? cl : lim; }
        softmax_step<C, PT, HD, EMU>(sreg, tS, tO, sl, j == 0, j * C::BN + 127 > tile_min_lim, lim - j * C::BN, split,
                                     m_ref, m_true, l);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive_cluster(leader_p_full);
    }

    if (ok && n_my > 0) {
      ok = mbar_wait_warp(bar_o_full + 8 * t, 0, actx, kErrFmhaOFull);
      if (ok) {
        tc_fence_after_sync();
        const uint32_t stage = sQ + t * C::TILEB;    // every Q_t K^T of the pair is done by now
        stage_output<C, HD>(tO, stage, r, p.out_scale / l, p.out_bf16 != 0);
        fence_proxy_async_smem();
        mbar_arrive(bar_o_staged + 8 * t);
        if (r == 0) {
          if (mbar_wait(bar_o_staged + 8 * t, 0, actx, kErrFmhaOStaged)) {
            tma_store_5d(&tm_o, stage, 0, row0, 0, head, batch);
            tma_store_commit();
            tma_store_wait_read0();
          }
        }
        if (row_g < p.Sq) {
          const size_t so = ((size_t)batch * p.H + head) * p.Sq + row_g;
          const float mref2 = m_ref * sl - C::PSHIFT;
          if (p.lse) p.lse[so] = 0.69314718055994531f * (mref2 + log2f(l));
          if (p.mi) p.mi[so] = m_true * sl;
          if (p.sprime) p.sprime[so] = l * exp2f(mref2 - m_true * sl);
        }
      }
    }
  }

  // ---- tear-down: no CTA leaves while its peer may still read its shared memory or signal its barriers
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 8) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
  }
}

}  // namespace cfk
