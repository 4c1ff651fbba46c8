// Flash-attention forward for sm_100a, head dimension 256 (fp16, bf16 or e4m3 inputs): one CTA per (128 query rows,
// head, batch).
//
// The reference runs head dimension 256 through the same kernels as 64 and 128 with a smaller key tile
// (src/fmha-pipeline/fmha_forward.cu:746-757, compile_run_all_config.sh:3-6).  On B200 the O accumulator of one
// 128-row query tile alone takes 256 of the 512 tensor-memory columns, so the two-tile plan of fmha_fwd_sm100.cuh
// does not fit; this kernel keeps ONE query tile per CTA and double-buffers the scores instead:
//
//   columns   0-127  S_A (key tiles j = 0, 2, ...), P_j written over its first 64 columns
//           128-255  S_B (key tiles j = 1, 3, ...)
//           256-511  O
//
// At this head dimension the two GEMMs of a key tile take 2048 tensor-core clocks (16 + 16 UMMAs of 128x128x16 /
// 128x128x16-per-half) against about 1700 clocks of softmax for the tile, so a single softmax warpgroup keeps the
// tensor core busy: while P_j V_j and Q K_{j+2}^T run on buffer A, the warpgroup is already working on S_B(j+1).
//   warps 0-3  softmax (thread r owns row r) and epilogue      warp 4  UMMA issue      warp 5  TMA producer
// Shared memory: 64 KB for the Q tile and later the staged O tile, and a ring of 32 KB slots (16 KB for e4m3); K_j and
// V_j each travel as two [128 keys][128 columns] halves (K halves split the reduction of Q K^T, V halves the columns
// of O).  With e4m3 inputs the tensor core runs at twice the rate and the single softmax warpgroup is the bound.
#pragma once
#include "fmha_softmax.cuh"

namespace cfk {


template <int DT>
struct FmhaHd256Cfg {
  static constexpr int HD = 256, BN = 128;
  static constexpr int ESZ = (DT == kDtE4M3) ? 1 : 2;
  static constexpr bool KIND8 = (ESZ == 1);
  static constexpr int SUBB = 128 * 128;              // one 128-byte span of a 128-row tile
  static constexpr int HSPANS = ESZ;                  // spans per half of a K or V tile (128 columns)
  static constexpr int QB = 2 * HSPANS * SUBB;        // bytes of the Q tile
  static constexpr int QTILEB = 4 * SUBB;             // Q tile, later the staged O tile (16-bit, 64 KB)
  static constexpr int SLOTB = HSPANS * SUBB;         // half a K or V tile: 128 keys x 128 columns
  static constexpr int HALF_KSTEPS = 128 * ESZ / 32;  // UMMAs per half tile (32 bytes of reduction each)
  static constexpr int SMEM_LIMIT = 232448;
  static constexpr int BARB = 512;
  static constexpr int NSLOT_FIT = (SMEM_LIMIT - 1024 - BARB - QTILEB) / SLOTB;   // 5 (16-bit) or 10
  static constexpr int NSLOT = NSLOT_FIT > 10 ? 10 : NSLOT_FIT;
  static_assert(NSLOT >= 4, "ring too small");
  static constexpr int SMEM_BYTES = 1024 + QTILEB + NSLOT * SLOTB + BARB;
  static constexpr int V_STEPB = (32 / ESZ) * 128;    // bytes between the key groups of successive UMMAs in a V half
  static constexpr int TMEM_COLS = 512, O_COL0 = 256;
  static constexpr uint32_t FMT = (DT == kDtBF16) ? kFmtBF16 : 0u;   // f16 and e4m3 are both code 0 of their kind
  static constexpr uint32_t IDESC_QK = make_idesc(1, FMT, FMT, 0, 0, 128, 128);
  static constexpr uint32_t IDESC_PV = make_idesc(1, FMT, FMT, 0, 1, 128, 128);
  static constexpr int NTHREADS = 192;
  static constexpr float TAU = (DT == kDtE4M3) ? 4.0f : 8.0f;      // see FmhaCfg
  static constexpr float PSHIFT = (DT == kDtE4M3) ? 4.0f : 0.0f;
};

// tm_q / tm_o: boxes of 128 rows x all 128-byte spans of a row; tm_k / tm_v: 128 keys x 128 columns (HSPANS spans).
template <int DT, int EMU, bool DUMP = false>
__global__ void __launch_bounds__(192, 1)
fmha_fwd_hd256_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                      const FmhaParams p) {
  using C = FmhaHd256Cfg<DT>;
  constexpr int PT = DT;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t sQ = smem_base;
  const uint32_t sRing = smem_base + C::QTILEB;
  const uint32_t sBar = sRing + C::NSLOT * C::SLOTB;
  uint8_t* gBar = smem_gen + (sBar - smem_base);
  const uint32_t bar_q_full = sBar;
  const uint32_t bar_kv_full = sBar + 8;                     // [NSLOT]
  const uint32_t bar_kv_empty = bar_kv_full + 8 * C::NSLOT;  // [NSLOT]
  const uint32_t bar_s_full = bar_kv_empty + 8 * C::NSLOT;   // [2]
  const uint32_t bar_p_full = bar_s_full + 16;               // [2] one arrival per softmax warp
  const uint32_t bar_pv_done = bar_p_full + 16;              // O += P_j V_j finished (completion j)
  const uint32_t bar_o_full = bar_pv_done + 8;
  const uint32_t bar_o_staged = bar_o_full + 8;              // one arrival per softmax warp
  const uint32_t off_misc = (bar_o_staged + 8) - sBar;
  static_assert(8 * (2 * C::NSLOT + 8) + 8 <= C::BARB, "barrier block overflows");
  volatile uint32_t* s_tmem_base = reinterpret_cast<volatile uint32_t*>(gBar + off_misc);
  volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(gBar + off_misc + 4);
  const AbortCtx actx{s_abort, p.status};

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // Work item: p.nqblk counts 128-row query blocks here; same grouped, heaviest-first order as the other kernels.
  int qblk, head, batch;
  {
    const int bh_total = p.B * p.H;
    const int per_group = p.group * p.nqblk;
    const int g = (int)blockIdx.x / per_group;
    const int rr = (int)blockIdx.x - g * per_group;
    const int left = bh_total - g * p.group;
    const int gsz = left < p.group ? left : p.group;
    qblk = p.nqblk - 1 - rr / gsz;
    const int bh = g * p.group + rr % gsz;
    batch = bh / p.H;
    head = bh - batch * p.H;
  }
  const int row0 = qblk * 128;
  const int diag_off = p.Skv - p.Sq;
  int n_kv = (p.Skv + C::BN - 1) / C::BN;
  if (p.causal) {
    const int last_key = row0 + 127 + diag_off;
    const int nc = last_key < 0 ? 1 : last_key / C::BN + 1;
    n_kv = nc < n_kv ? nc : n_kv;
  }

  if (cta_should_skip(p.status)) return;

  if (tid == 0) {
    mbar_init(bar_q_full, 1);
    for (int i = 0; i < C::NSLOT; ++i) {
      mbar_init(bar_kv_full + 8 * i, 1);
      mbar_init(bar_kv_empty + 8 * i, 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(bar_s_full + 8 * x, 1);
      mbar_init(bar_p_full + 8 * x, 4);
    }
    mbar_init(bar_pv_done, 1);
    mbar_init(bar_o_full, 1);
    mbar_init(bar_o_staged, 4);
    *s_abort = 0u;
    fence_barrier_init();
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(s_tmem_base)), C::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 5 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_o);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *s_tmem_base;

  // bf16 only: blocks whose first row sees few keys keep P as a two-term sum (hi + lo, lo in columns 64-127 of S_x)
  bool split = false;
  if constexpr (PT == kDtBF16) {
    int visible = p.Skv;
    if (p.causal) { const int v0 = row0 + diag_off + 1; visible = v0 < visible ? v0 : visible; }
    split = visible < p.split_keys;
  }

  if (warp == 5) {
    // =========================== TMA producer ===========================
    // Ring order = order of use: K_0 (two halves), K_1, then for every j: V_j (two halves), K_{j+2}.
    if (lane == 0) {
      mbar_arrive_expect_tx(bar_q_full, C::QB);
      tma_load_5d(sQ, &tm_q, bar_q_full, 0, row0, 0, head, batch);
      int idx = 0;
      auto load = [&](const CUtensorMap* tm, int j) -> bool {   // both halves of K_j or V_j
        for (int h = 0; h < 2; ++h, ++idx) {
          const int slot = idx % C::NSLOT;
          const uint32_t ph = (idx / C::NSLOT) & 1;
          if (!mbar_wait(bar_kv_empty + 8 * slot, ph ^ 1u, actx, kErrFmhaKvEmpty)) return false;
          mbar_arrive_expect_tx(bar_kv_full + 8 * slot, C::SLOTB);
          tma_load_5d(sRing + slot * C::SLOTB, tm, bar_kv_full + 8 * slot, 0, j * C::BN, C::HSPANS * h, head, batch);
        }
        return true;
      };
      bool ok = load(&tm_k, 0);
      if (ok && n_kv > 1) ok = load(&tm_k, 1);
      for (int j = 0; j < n_kv && ok; ++j) {
        ok = load(&tm_v, j);
        if (ok && j + 2 < n_kv) ok = load(&tm_k, j + 2);
      }
    }
  } else if (warp == 4) {
    // =========================== UMMA issue ===========================
    // All 32 lanes run the loop (uniform control flow); one elected lane executes the tcgen05 instructions.
    const uint32_t leader = elect_one();
    bool ok = true;
    const uint64_t aq0 = make_smem_desc(sQ, 16, 1024, kSwizzle128B);
    const uint64_t bk0 = make_smem_desc(sRing, 16, 1024, kSwizzle128B);
    const uint64_t bv0 = make_smem_desc(sRing, C::SUBB, 1024, kSwizzle128B);   // MN-major: two 64-column groups
    int idx = 0;
    auto slot_wait = [&]() -> bool {
      return mbar_wait_warp(bar_kv_full + 8 * (idx % C::NSLOT), (idx / C::NSLOT) & 1, actx, kErrFmhaKvFull);
    };
    // S_x = Q K_j^T: the two halves of K_j split the reduction over the head dimension
    auto qk = [&](int x) -> bool {
      const uint32_t d = tmem_base + x * 128;
      for (int h = 0; h < 2; ++h, ++idx) {
        if (!slot_wait()) return false;
        tc_fence_after_sync();
        const uint64_t a0 = desc_advance_lo(aq0, h * C::SLOTB);
        const uint64_t b0 = desc_advance_lo(bk0, (idx % C::NSLOT) * C::SLOTB);
#pragma unroll
        for (int kk = 0; kk < C::HALF_KSTEPS; ++kk) {
          const uint32_t off = (kk >> 2) * C::SUBB + (kk & 3) * 32;
          umma_ss_e<C::KIND8, false>(d, desc_advance_lo(a0, off), desc_advance_lo(b0, off), C::IDESC_QK,
                                  (h > 0 || kk > 0) ? 1u : 0u, leader);
        }
        umma_commit_e<false>(bar_kv_empty + 8 * (idx % C::NSLOT), leader);
      }
      umma_commit_e<false>(bar_s_full + 8 * x, leader);
      return true;
    };
    // O += P_x V_j: the two halves of V_j are columns 0-127 and 128-255 of O
    auto pv = [&](int x, uint32_t accumulate) -> bool {
      const uint32_t a = tmem_base + x * 128;
      for (int h = 0; h < 2; ++h, ++idx) {
        if (!slot_wait()) return false;
        tc_fence_after_sync();
        const uint32_t d = tmem_base + C::O_COL0 + h * 128;
        const uint64_t b0 = desc_advance_lo(bv0, (idx % C::NSLOT) * C::SLOTB);
#pragma unroll
        for (int kk = 0; kk < C::HALF_KSTEPS; ++kk)
          umma_ts_e<C::KIND8, false>(d, a + kk * 8, desc_advance_lo(b0, kk * C::V_STEPB), C::IDESC_PV,
                                  kk > 0 ? 1u : accumulate, leader);
        if (split) {
#pragma unroll
          for (int kk = 0; kk < C::HALF_KSTEPS; ++kk)
            umma_ts_e<C::KIND8, false>(d, a + 64 + kk * 8, desc_advance_lo(b0, kk * C::V_STEPB), C::IDESC_PV, 1u, leader);
        }
        umma_commit_e<false>(bar_kv_empty + 8 * (idx % C::NSLOT), leader);
      }
      umma_commit_e<false>(bar_pv_done, leader);
      return true;
    };

    ok = mbar_wait_warp(bar_q_full, 0, actx, kErrFmhaQFull);
    if (ok) ok = qk(0);
    if (ok && n_kv > 1) ok = qk(1);
    for (int j = 0; j < n_kv && ok; ++j) {
      const int x = j & 1;
      ok = mbar_wait_warp(bar_p_full + 8 * x, (j >> 1) & 1, actx, kErrFmhaPFull);
      if (!ok) break;
      tc_fence_after_sync();
      ok = pv(x, j > 0 ? 1u : 0u);
      if (ok && j + 2 < n_kv) ok = qk(x);     // P_j lives in S_x, so S_x(j+2) follows P_j V_j
    }
    if (ok) umma_commit_e<false>(bar_o_full, leader);
  } else {
    // =========================== softmax + epilogue ===========================
    const int r = tid;                     // row within the tile == TMEM lane
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const uint32_t tO = tmem_base + lane_base + C::O_COL0;
    const int row_g = row0 + r;
    const int tile_min_lim = p.causal ? min(p.Skv - 1, row0 + diag_off) : p.Skv - 1;
    const float sl = p.scale_log2;

    float m_ref = 0.f, m_true = -INFINITY, l = 0.f;
    bool ok = true;
    uint32_t sreg[128];

    // One copy of the loop per form of the P store (two-term or plain): with both forms in one loop body a bf16
    // launch runs slower also where no CTA uses the second form.
    auto key_tile_loop = [&](auto split_c) {
    constexpr bool SPLIT = decltype(split_c)::value;
    for (int j = 0; j < n_kv; ++j) {
      const int x = j & 1;
      const uint32_t tS = tmem_base + lane_base + x * 128;
      ok = mbar_wait_warp(bar_s_full + 8 * x, (j >> 1) & 1, actx, kErrFmhaSFull);
      if (!ok) break;
      tc_fence_after_sync();
      tmem_ld_x32(tS + 0, sreg + 0);
      tmem_ld_x32(tS + 32, sreg + 32);
      tmem_ld_x32(tS + 64, sreg + 64);
      tmem_ld_x32(tS + 96, sreg + 96);
      tmem_wait_ld();

      if constexpr (DUMP) dump_scores(p, sreg, batch, head, row_g, j * C::BN);
      if (j * C::BN + 127 > tile_min_lim) {   // this tile has masked columns for some row
        int lim = p.Skv - 1;
        if (p.causal) { const int cl = row_g + diag_off; lim = cl < lim ? cl : lim; }
        lim -= j * C::BN;
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (i > lim) sreg[i] = 0xff800000u;  // -inf
      }
      const float rowmax = row_max128(sreg);
      m_true = fmaxf(m_true, rowmax);
      if (j == 0) {
        m_ref = (rowmax == -INFINITY) ? 0.f : rowmax;
      } else {
        const bool need = (rowmax - m_ref) * sl > C::TAU;
        if (__any_sync(0xffffffffu, need)) {
          // O must hold tiles 0..j-1: P_{j-1} V_{j-1} was issued after this warpgroup's previous step and may still run
          ok = mbar_wait_warp(bar_pv_done, (j - 1) & 1, actx, kErrFmhaPvDone256);
          if (!ok) break;
          tc_fence_after_sync();
          float alpha = 1.f;
          if (need) {
            alpha = ex2_approx((m_ref - rowmax) * sl);
            m_ref = rowmax;
            l *= alpha;
          }
          rescale_o_row<C::HD>(tO, alpha);
        }
      }
      const float negm = C::PSHIFT - m_ref * sl;
      l += emit_p128<PT, EMU, SPLIT>(sreg, tS, tS + 64, sl, negm);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive_warp(bar_p_full + 8 * x);
    }
    };
    if constexpr (PT == kDtBF16) {
      if (split) key_tile_loop(std::true_type{});
      else key_tile_loop(std::false_type{});
    } else {
      key_tile_loop(std::false_type{});
    }

    if (ok && n_kv > 0) {
      ok = mbar_wait_warp(bar_o_full, 0, actx, kErrFmhaOFull);
      if (ok) {
        tc_fence_after_sync();
        const float inv = p.out_scale / l;
        uint32_t oreg[32];
#pragma unroll 1
        for (int c = 0; c < C::HD / 32; ++c) {   // 32 output columns = half a 128-byte span
          tmem_ld_x32(tO + c * 32, oreg);
          tmem_wait_ld();
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float a = __uint_as_float(oreg[2 * i]) * inv, b = __uint_as_float(oreg[2 * i + 1]) * inv;
            pk[i] = p.out_bf16 ? pack_bf16x2(a, b) : pack_f16x2(a, b);
          }
          const uint32_t row_addr = sQ + (c >> 1) * C::SUBB + r * 128;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t chunk = (uint32_t)((c & 1) * 4 + i) ^ (uint32_t)(r & 7);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + chunk * 16), "r"(pk[4 * i]),
                         "r"(pk[4 * i + 1]), "r"(pk[4 * i + 2]), "r"(pk[4 * i + 3])
                         : "memory");
          }
        }
        fence_proxy_async_smem();
        mbar_arrive_warp(bar_o_staged);
        if (tid == 0) {
          if (mbar_wait(bar_o_staged, 0, actx, kErrFmhaOStaged)) {
            tma_store_5d(&tm_o, sQ, 0, row0, 0, head, batch);
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

  // ---- tear-down ----
  settle_if_aborted(s_abort);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

}  // namespace cfk
