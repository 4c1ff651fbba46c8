// Flash-attention forward for sm_100a, head dimensions 64 and 128: a persistent kernel with one 128-row query tile
// in flight per CTA and six roles.  It stands where the reference has fmhaForwardPipelinedWspl
// (src/fmha-pipeline/fmha_pipe_ws.h:69-365: producer warpgroup :245-290, consumer warpgroups :292-364) with
// fmhaForwardProducer / fmhaForwardConsumer (fmha_producer.h:4-79, fmha_consumer.h:8-73), the online softmax
// (online_softmax.h:87-207) and the TMA-store epilogue (fmha_epilogue.h:120-177).
//
//   warps 0-3   softmax A: thread r owns query row r (== TMEM lane r) for the even key tiles of the CTA's tile sequence
//   warps 4-7   softmax B: the same rows for the odd key tiles
//   warps 8-11  correction: the final correction of an item's accumulator and its epilogue (O / l -> 16 bit -> shared
//               memory -> TMA store, LSE), and the load of the Q tile that takes over the freed buffer, while the
//               other roles are already on the next item
//   warp 12     UMMA issue for O += P_g V_g        (one elected lane each; two warps because what a single warp has
//   warp 13     UMMA issue for S = Q K_g^T          to do per key tile besides the UMMAs - a barrier wait costs it 250
//                                                   clocks even when the barrier is complete, a commit 100 - was
//                                                   measured at twice the tensor time of the tile)
//   warp 14     TMA producer for the K tiles (a ring of shared-memory slots) and the first two Q tiles
//   warp 15     TMA producer for the V tiles (a ring of their own)
//
// Tensor memory: S_0, S_1 (scores of the even / odd key tiles, 128 columns each), O from column 256, P_0, P_1 from
// column 384.  P has buffers of its own, so Q K_{g+2}^T only waits until the softmax warpgroup has READ S_g, not
// until P_g V_g has run: the scores of a warpgroup's next tile are there long before it has finished the present
// one, and neither warpgroup ever waits for the tensor core.  The two of them work half a tile apart and keep the
// special-function unit and the other pipes busy in turns.  (When P is written over S, as in the two-tile kernel, a
// warpgroup has to wait for "P_g V_g, then Q K_{g+2}^T" before its next tile.)
//
// Barriers are keyed by key tile (index modulo the ring depth), and each UMMA warp waits on ONE barrier per tile:
// kq_ready(t) completes when the softmax warps have read S of tile t-2 (4 arrivals) and K_t has landed (the
// producer's arrive.expect_tx and the TMA bytes); pv_ready(g) when P_g is in tensor memory (4 arrivals) and V_g has
// landed.  s_full(t) / pv_done(g), signalled by tcgen05.commit, double as the "slot free" signal for the producer.
//
// The two warpgroups share a row's running maximum without meeting: the reference maximum of a row is a chain over
// the key tiles.  The owner of tile g takes its row maximum, looks up (normally without waiting) the reference
// maximum the owner of tile g-1 has published, keeps it unless its own maximum exceeds it by more than TAU in the
// log2 domain, and publishes the result before it starts on the exponentials.  Only when the maximum moves does it
// wait for P_{g-1} V_{g-1} and rescale the row of O.  Each warpgroup sums its own tiles' probabilities; the two
// partial sums are brought to one scale at the end of the item.  The reference rescales on every tile
// (online_softmax.h:144-165).
//
// Work items ((128 query rows, head, batch), heaviest first) are dealt to the CTAs of a persistent grid in rounds
// whose direction alternates, so that with a causal mask every CTA gets the same mix of long and short items.  All
// barrier waits are bounded; a wait that gives up raises the CTA's abort flag and every role falls through to the
// common tear-down.
#pragma once
#include "fmha_softmax.cuh"

// Sleep between two looks at a barrier (ns) for the roles that wait long; see mbar_wait.
#ifndef CFK_BACKOFF_EPILOGUE
#define CFK_BACKOFF_EPILOGUE 256
#endif
#ifndef CFK_BACKOFF_PRODUCER
#define CFK_BACKOFF_PRODUCER 64
#endif
#ifndef CFK_BACKOFF_UMMA
#define CFK_BACKOFF_UMMA 0
#endif

namespace cfk {

template <int DT, int PT, int HD>
struct FmhaPersistCfg : FmhaCfg<DT, PT, HD> {
  using Base = FmhaCfg<DT, PT, HD>;
  static constexpr int NTHREADS = 512;
  static constexpr int QBUFB = Base::TILEB > Base::OTILEB ? Base::TILEB : Base::OTILEB;   // a Q tile, later the staged O tile
  static constexpr int CHAINB = 128 * 8;            // per row: {tile index + 1, reference maximum after that tile}
  static constexpr int STATSB = 3 * 128 * 4;        // row sum, reference maximum, true maximum of a finished item
  static constexpr int BARB = 384;
  static constexpr int SMEM_LIMIT = 232448;
  // K ring and V ring, filled alternately while both fit; two slots each at least, four at most
  static constexpr int RINGB = SMEM_LIMIT - 2 * QBUFB - CHAINB - STATSB - BARB;
  static constexpr int PAIRS = RINGB / (Base::TILEB + Base::VTILEB);
  static constexpr int NV = PAIRS > 4 ? 4 : PAIRS;
  static constexpr int NK_FIT = (RINGB - NV * Base::VTILEB) / Base::TILEB;
  static constexpr int NK = NK_FIT > 4 ? 4 : NK_FIT;
  static_assert(NK >= 2 && NV >= 2, "rings too small");
  static constexpr int SMEM_BYTES = 2 * QBUFB + NK * Base::TILEB + NV * Base::VTILEB + CHAINB + STATSB + BARB;
  static constexpr int O_COL0 = 256, P_COL0 = 384, P_COLS = 64;   // tensor-memory columns: S_0 0, S_1 128, O, P_0, P_1
  // Registers after setmaxnreg; the pool is 512 threads x 128 (the launch bound).  setmaxnreg.inc waits without a
  // time limit for the registers it asks for, so the sum must stay inside the pool.
  static constexpr int LAUNCH_REGS = 128, SOFTMAX_REGS = 200, CORR_REGS = 56, AUX_REGS = 56;
  static_assert(2 * 128 * SOFTMAX_REGS + 128 * CORR_REGS + 128 * AUX_REGS <= NTHREADS * LAUNCH_REGS,
                "setmaxnreg would block forever");
};

// One work item of a CTA and the position inside it; every role walks the same sequence.
struct FmhaItem {
  int k;                    // items this CTA started before this one
  int j, n;                 // key tile inside the item, key tiles of the item
  int qblk, head, batch;
  bool split;               // bf16: P as hi + lo terms (rows that see few keys)
  bool valid;
};

template <int DT, int PT, int HD, int EMU, bool DUMP = false>
__global__ void __launch_bounds__(512, 1)
fmha_fwd_persist_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                        const FmhaParams p) {
  using C = FmhaPersistCfg<DT, PT, HD>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = smem_u32(smem_raw);

  const uint32_t sQ = smem_base;                          // [2] Q tile of item k in buffer k & 1
  const uint32_t sK = smem_base + 2 * C::QBUFB;           // [NK] K of tile t in slot t % NK
  const uint32_t sV = sK + C::NK * C::TILEB;              // [NV] V of tile g in slot g % NV
  const uint32_t sChain = sV + C::NV * C::VTILEB;
  const uint32_t sStats = sChain + C::CHAINB;
  const uint32_t sBar = sStats + C::STATSB;
  uint8_t* gBar = smem_raw + (sBar - smem_base);
  const uint32_t chain_row = sChain + 8u * (threadIdx.x & 127u);   // this thread's row (softmax threads)
  volatile float* g_stats = reinterpret_cast<volatile float*>(smem_raw + (sStats - smem_base));
  // barrier map (8 bytes each); "tile" is the index in the CTA's sequence of key tiles, which runs on across items
  const uint32_t bar_q_full = sBar;                           // [2]
  const uint32_t bar_kq_ready = bar_q_full + 16;              // [NK] tile t: S of tile t-2 has been read (4 warps) + K_t landed
  const uint32_t bar_s_full = bar_kq_ready + 8 * C::NK;       // [NK] tile t: S = Q K_t^T is complete (also: K slot free)
  const uint32_t bar_pv_ready = bar_s_full + 8 * C::NK;       // [NV] tile g: P_g is in tensor memory (4 warps) + V_g landed
  const uint32_t bar_pv_done = bar_pv_ready + 8 * C::NV;      // [NV] tile g: O += P_g V_g is complete (also: V slot, P buffer free)
  const uint32_t bar_o_full = bar_pv_done + 8 * C::NV;        // one completion per item
  const uint32_t bar_o_free = bar_o_full + 8;                 // O and the statistics of the item have been read (4 warps)
  const uint32_t bar_o_staged = bar_o_free + 8;               // 4 warps
  const uint32_t bar_stats = bar_o_staged + 8;                // 4 warps: the warpgroup that owns the item's last tile
  const uint32_t bar_fin = bar_stats + 8;                     // [4] the other warpgroup's partial statistics are out
  const uint32_t off_misc = (bar_fin + 32) - sBar;
  static_assert(8 * (2 + 4 * 4 + 4 + 4) + 16 <= C::BARB, "barrier block overflows");
  volatile uint32_t* s_tmem_base = reinterpret_cast<volatile uint32_t*>(gBar + off_misc);
  volatile uint32_t* s_abort = reinterpret_cast<volatile uint32_t*>(gBar + off_misc + 4);
  volatile uint32_t* s_skip = reinterpret_cast<volatile uint32_t*>(gBar + off_misc + 8);
  const AbortCtx actx{s_abort, p.status};

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  const int n_items = p.nqblk * p.B * p.H;
  const int nkv_total = (p.Skv + C::BN - 1) / C::BN;
  const int diag_off = p.Skv - p.Sq;

  // Item k of this CTA: rounds of gridDim.x items, even rounds dealt forwards, odd rounds backwards.  The item index
  // orders (batch, head) pairs in groups whose K and V fit in L2 together and, inside a group, the query blocks from
  // the last (heaviest when causal) to the first.
  auto item_at = [&](FmhaItem& it, int k) {
    it.k = k;
    it.j = 0;
    const long long base = (long long)k * gridDim.x;
    const int pos = (k & 1) ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
    it.valid = base + pos < n_items;
    if (!it.valid) return;
    const int idx = (int)(base + pos);
    const int per_group = p.group * p.nqblk;
    const int g = idx / per_group;
    const int rr = idx - g * per_group;
    const int left = p.B * p.H - g * p.group;
    const int gsz = left < p.group ? left : p.group;
    it.qblk = p.nqblk - 1 - rr / gsz;
    const int bh = g * p.group + rr % gsz;
    it.batch = bh / p.H;
    it.head = bh - it.batch * p.H;
    const int row0 = it.qblk * 128;
    int n = nkv_total;
    if (p.causal) {
      const int last_key = row0 + 127 + diag_off;
      const int nc = last_key < 0 ? 1 : last_key / C::BN + 1;
      n = nc < n ? nc : n;
    }
    it.n = n;
    it.split = false;
    if constexpr (PT == kDtBF16) {
      int visible = p.Skv;
      if (p.causal) { const int v0 = row0 + diag_off + 1; visible = v0 < visible ? v0 : visible; }
      it.split = visible < p.split_keys;
    }
  };
  auto item_next_tile = [&](FmhaItem& it) {
    if (++it.j == it.n) item_at(it, it.k + 1);
  };
  auto load_q = [&](const FmhaItem& it) {
    const int b = it.k & 1;
    mbar_arrive_expect_tx(bar_q_full + 8 * b, C::TILEB);
    tma_load_5d(sQ + b * C::QBUFB, &tm_q, bar_q_full + 8 * b, 0, it.qblk * 128, 0, it.head, it.batch);
  };
  // position of a tile in a ring of N: slot and the parity of the slot's current use
  struct RingPos {
    int i;
    uint32_t ph;
  };
  auto ring_next = [](RingPos& r, int n) {
    if (++r.i == n) { r.i = 0; r.ph ^= 1u; }
  };

  // A launch that finds the status word already set does nothing (see fmha_fwd_sm100.cuh).
  if (tid == 0) *s_skip = (uint32_t)(*reinterpret_cast<const volatile int*>(p.status) != 0);
  __syncthreads();
  if (*s_skip) return;

  // ---- set-up ----
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) mbar_init(bar_q_full + 8 * i, 1);
    for (int i = 0; i < C::NK; ++i) {
      mbar_init(bar_kq_ready + 8 * i, 5);
      mbar_init(bar_s_full + 8 * i, 1);
    }
    for (int i = 0; i < C::NV; ++i) {
      mbar_init(bar_pv_ready + 8 * i, 5);
      mbar_init(bar_pv_done + 8 * i, 1);
    }
    mbar_init(bar_o_full, 1);
    mbar_init(bar_o_free, 4);
    mbar_init(bar_o_staged, 4);
    mbar_init(bar_stats, 4);
    for (int i = 0; i < 4; ++i) mbar_init(bar_fin + 8 * i, 1);
    *s_abort = 0u;
    fence_barrier_init();
  }
  if (tid < 128) {   // the chain starts at "no tile decided"
    asm volatile("st.shared.v2.b32 [%0], {%1, %1};" ::"r"(chain_row), "r"(0u) : "memory");
  }
  if (warp == 12) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(s_tmem_base)), 512);
    tmem_relinquish();
  }
  if (warp == 14 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_o);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *s_tmem_base;

  if (warp >= 12) {
    setmaxnreg_dec<C::AUX_REGS>();
    if (warp == 14 || warp == 15) {
      // =========================== TMA producers ===========================
      // Warp 14 loads the K tiles (and the first two Q tiles), warp 15 the V tiles, each into its own ring: one
      // lane doing both in turn would hold a K load back while it waits for a V slot, and the two rings drain at
      // different times.  A slot is free once the UMMAs that read it have completed, which the s_full / pv_done
      // barrier of the tile that held it says; the load then signals the kq_ready / pv_ready barrier of its own tile.
      if (lane == 0) {
        FmhaItem c;
        item_at(c, 0);
        RingPos r{0, 0};
        uint32_t n = 0;     // tiles issued
        CFK_PROF_DECL(4)
        if (warp == 14) {
          while (c.valid) {
            if (c.j == 0 && c.k < 2) load_q(c);   // later Q tiles are loaded by the epilogue that frees their buffer
            CFK_PROF_MARK(1)
            if (n >= (uint32_t)C::NK &&
                !mbar_wait(bar_s_full + 8 * r.i, r.ph ^ 1u, actx, kErrFmhaKvEmpty, kWaitLimitNs, CFK_BACKOFF_PRODUCER)) break;
            CFK_PROF_MARK(0)
            mbar_arrive_expect_tx(bar_kq_ready + 8 * r.i, C::TILEB);
            tma_load_5d(sK + r.i * C::TILEB, &tm_k, bar_kq_ready + 8 * r.i, 0, c.j * C::BN, 0, c.head, c.batch);
            ring_next(r, C::NK);
            ++n;
            item_next_tile(c);
          }
          CFK_PROF_FLUSH(20, 4, true)
        } else {
          while (c.valid) {
            if (n >= (uint32_t)C::NV &&
                !mbar_wait(bar_pv_done + 8 * r.i, r.ph ^ 1u, actx, kErrFmhaKvEmpty, kWaitLimitNs, CFK_BACKOFF_PRODUCER)) break;
            mbar_arrive_expect_tx(bar_pv_ready + 8 * r.i, C::VTILEB);
            tma_load_5d(sV + r.i * C::VTILEB, &tm_v, bar_pv_ready + 8 * r.i, 0, c.j * C::BN, 0, c.head, c.batch);
            ring_next(r, C::NV);
            ++n;
            item_next_tile(c);
          }
        }
      }
    } else if (warp == 13) {
      // =========================== UMMA issue: S = Q K^T ===========================
      // All 32 lanes run the loop (uniform control flow); one elected lane executes the tcgen05 instructions.
      const uint32_t leader = elect_one();
      bool ok = true;
      const uint64_t aq0 = make_smem_desc(sQ, 16, C::SBO, C::SWZ);
      const uint64_t bk0 = make_smem_desc(sK, 16, C::SBO, C::SWZ);
      FmhaItem kc;
      item_at(kc, 0);
      RingPos kr{0, 0};
      uint32_t t = 0;                 // tile
      bool split1 = false, split2 = false;   // tiles t-1 and t-2 belong to items with a two-term P
      RingPos d1{0, 0}, d2{0, 0};     // pv_done positions of tiles t-1 and t-2
      CFK_PROF_DECL(4)
      while (ok && kc.valid) {
        CFK_PROF_MARK(3)
        if (kc.j == 0) {
          ok = mbar_wait_warp(bar_q_full + 8 * (kc.k & 1), (kc.k >> 1) & 1, actx, kErrFmhaQFull);
          if (!ok) break;
        }
        ok = mbar_wait_warp(bar_kq_ready + 8 * kr.i, kr.ph, actx, kErrFmhaKvFull, CFK_BACKOFF_UMMA);
        if (!ok) break;
        if constexpr (PT == kDtBF16) {
          if (split2) {   // the second term of that tile's P was left in the S buffer: its P V must have run
            ok = mbar_wait_warp(bar_pv_done + 8 * d2.i, d2.ph, actx, kErrFmhaCorrPv);
            if (!ok) break;
          }
        }
        CFK_PROF_MARK(0)
        tc_fence_after_sync();
        const uint64_t a0 = desc_advance_lo(aq0, (kc.k & 1) * C::QBUFB);
        const uint64_t b0 = desc_advance_lo(bk0, kr.i * C::TILEB);
        const uint32_t d = tmem_base + (t & 1u) * 128;
#pragma unroll
        for (int kk = 0; kk < C::QK_KSTEPS; ++kk) {
          const uint32_t off = (kk / C::KSPS) * C::SUBB + (kk % C::KSPS) * 32;
          umma_ss_e<C::KIND8, false>(d, desc_advance_lo(a0, off), desc_advance_lo(b0, off), C::IDESC_QK, kk > 0 ? 1u : 0u,
                                     leader);
        }
        CFK_PROF_MARK(1)
        umma_commit_e<false>(bar_s_full + 8 * kr.i, leader);
        CFK_PROF_MARK(2)
        ring_next(kr, C::NK);
        if constexpr (PT == kDtBF16) {
          split2 = split1; split1 = kc.split;
          d2 = d1;
          if (t > 0) ring_next(d1, C::NV);   // d1 follows tile t-1: position of tile 0 is {0, 0}
        }
        ++t;
        item_next_tile(kc);
      }
      CFK_PROF_FLUSH(12, 4, (leader != 0))
    } else if (warp == 12) {
      // =========================== UMMA issue: O += P V ===========================
      const uint32_t leader = elect_one();
      bool ok = true;
      const uint64_t bv0 = make_smem_desc(sV, C::VSUBB, C::VSBO, C::VSWZ);
      FmhaItem pc;
      item_at(pc, 0);
      RingPos vr{0, 0};
      uint32_t g = 0;
      CFK_PROF_DECL(4)
      while (ok && pc.valid) {
        CFK_PROF_MARK(3)
        ok = mbar_wait_warp(bar_pv_ready + 8 * vr.i, vr.ph, actx, kErrFmhaPFull, CFK_BACKOFF_UMMA);
        if (!ok) break;
        if (pc.j == 0 && pc.k > 0) {   // O still holds the previous item until the correction warps have read it
          ok = mbar_wait_warp(bar_o_free, (uint32_t)(pc.k - 1) & 1u, actx, kErrFmhaOFree);
          if (!ok) break;
        }
        CFK_PROF_MARK(0)
        tc_fence_after_sync();
        const uint64_t b0 = desc_advance_lo(bv0, vr.i * C::VTILEB);
        const uint32_t d = tmem_base + C::O_COL0;
        const uint32_t a = tmem_base + C::P_COL0 + (g & 1u) * C::P_COLS;
#pragma unroll
        for (int kk = 0; kk < C::PV_KSTEPS; ++kk)
          umma_ts_e<C::KIND8_PV, false>(d, a + kk * 8, desc_advance_lo(b0, kk * C::V_STEPB), C::IDESC_PV,
                                        (kk > 0 || pc.j > 0) ? 1u : 0u, leader);
        if constexpr (PT == kDtBF16) {
          if (pc.split) {   // second term of P: the first 64 columns of the tile's S buffer
            const uint32_t a2 = tmem_base + (g & 1u) * 128;
#pragma unroll
            for (int kk = 0; kk < C::PV_KSTEPS; ++kk)
              umma_ts_e<C::KIND8_PV, false>(d, a2 + kk * 8, desc_advance_lo(b0, kk * C::V_STEPB), C::IDESC_PV, 1u, leader);
          }
        }
        CFK_PROF_MARK(1)
        umma_commit_e<false>(bar_pv_done + 8 * vr.i, leader);
        if (pc.j == pc.n - 1) umma_commit_e<false>(bar_o_full, leader);
        CFK_PROF_MARK(2)
        ring_next(vr, C::NV);
        ++g;
        item_next_tile(pc);
      }
      CFK_PROF_FLUSH(8, 4, (leader != 0))
    }
  } else if (warp >= 8) {
    // =========================== correction + epilogue ===========================
    setmaxnreg_dec<C::CORR_REGS>();
    const int q = warp & 3;
    const int r = q * 32 + lane;                     // row within the tile == TMEM lane
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    const uint32_t tO = tmem_base + lane_base + C::O_COL0;
    const float sl = p.scale_log2;
    bool ok = true;
    FmhaItem it;
    CFK_PROF_DECL(4)
    for (item_at(it, 0); ok && it.valid; item_at(it, it.k + 1)) {
      ok = mbar_wait_warp(bar_o_full, (uint32_t)it.k & 1u, actx, kErrFmhaOFull, CFK_BACKOFF_EPILOGUE);   // the item's last P V has completed
      if (!ok) break;
      CFK_PROF_MARK(0)
      ok = mbar_wait_warp(bar_stats, (uint32_t)it.k & 1u, actx, kErrFmhaStats);
      if (!ok) break;
      tc_fence_after_sync();
      const float l = g_stats[r], m_ref = g_stats[128 + r], m_true = g_stats[256 + r];
      const uint32_t stage = sQ + (it.k & 1) * C::QBUFB;      // every Q K^T of the item is done: its Q tile is free
      stage_output<C, HD>(tO, stage, r, p.out_scale / l, p.out_bf16 != 0);
      tc_fence_before_sync();
      mbar_arrive_warp(bar_o_free);
      fence_proxy_async_smem();
      mbar_arrive_warp(bar_o_staged);
      if (warp == 8 && lane == 0) {
        if (mbar_wait(bar_o_staged, (uint32_t)it.k & 1u, actx, kErrFmhaOStaged)) {
          tma_store_5d(&tm_o, stage, 0, it.qblk * 128, 0, it.head, it.batch);
          tma_store_commit();
          tma_store_wait_read0();
          FmhaItem nx;                                        // the buffer is free: the item after next moves in
          item_at(nx, it.k + 2);
          if (nx.valid) load_q(nx);
        }
      }
      const int row_g = it.qblk * 128 + r;
      if (row_g < p.Sq) {
        const size_t so = ((size_t)it.batch * p.H + it.head) * p.Sq + row_g;
        const float mref2 = m_ref * sl - C::PSHIFT;      // exponent origin of l, log2 domain
        if (p.lse) p.lse[so] = 0.69314718055994531f * (mref2 + log2f(l));
        if (p.mi) p.mi[so] = m_true * sl;
        if (p.sprime) p.sprime[so] = l * exp2f(mref2 - m_true * sl);
      }
      CFK_PROF_MARK(2)
    }
    CFK_PROF_FLUSH(16, 4, (warp == 8 && lane == 0))
  } else {
    // =========================== softmax ===========================
    setmaxnreg_inc<C::SOFTMAX_REGS>();
    const uint32_t w = (uint32_t)warp >> 2;          // this warpgroup owns the key tiles g with g % 2 == w; S_w, P_w
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    const uint32_t tO = tmem_base + lane_base + C::O_COL0;
    const uint32_t tS = tmem_base + lane_base + w * 128;
    const uint32_t tP = tmem_base + lane_base + C::P_COL0 + w * C::P_COLS;
    const float sl = p.scale_log2;
    uint32_t g = 0;                                  // key tiles of this CTA so far (both warpgroups')
    uint32_t fins = 0;                               // items with two or more key tiles so far
    bool ok = true;
    uint32_t sreg[128];
    FmhaItem it;
    CFK_PROF_DECL(8)
    // S_w is free for this warpgroup's first tile
    mbar_arrive_warp(bar_kq_ready + 8 * (w % C::NK));
    uint32_t s_ready = 0u;                           // an early look found the scores of the next tile complete
    for (item_at(it, 0); ok && it.valid; item_at(it, it.k + 1)) {
      const int row_g = it.qblk * 128 + r;
      int lim = p.Skv - 1;                           // last key this row may see
      if (p.causal) { const int cl = row_g + diag_off; lim = cl < lim ? cl : lim; }
      const int tile_min_lim = p.causal ? min(p.Skv - 1, it.qblk * 128 + diag_off) : p.Skv - 1;
      // own running state of the item: sum of this warpgroup's probabilities, the reference maximum they are
      // relative to, and the largest score seen in this warpgroup's tiles
      float l = 0.f, m_l = 0.f, m_true = -INFINITY;
      for (int j = 0; j < it.n; ++j, ++g) {
        if ((g & 1u) != w) continue;
        CFK_PROF_MARK(7)
        // The looks at barriers and at shared memory of this step are issued early and their results used late:
        // each costs one to several hundred clocks even when it finds what it looks for (the tensor core's operand
        // reads keep the shared-memory port busy), which the loads and the maximum pass in between hide.
        if (!__all_sync(0xffffffffu, s_ready)) {   // looked at during the previous tile of this warpgroup
          ok = mbar_wait_warp(bar_s_full + 8 * (g % C::NK), (g / C::NK) & 1u, actx, kErrFmhaSFull);
        }
        CFK_PROF_MARK(0)
        if (!ok) break;
        tc_fence_after_sync();
        tmem_ld_x32(tS + 0, sreg + 0);
        tmem_ld_x32(tS + 32, sreg + 32);
        tmem_ld_x32(tS + 64, sreg + 64);
        tmem_ld_x32(tS + 96, sreg + 96);
        // P_w still holds this warpgroup's previous tile until its P V has run (it has, long ago)
        uint32_t p_free = 1u;
        if (g >= 2u) p_free = mbar_test_wait(bar_pv_done + 8 * ((g - 2u) % C::NV), ((g - 2u) / C::NV) & 1u);
        // the chain word of this row: {tile index + 1, reference maximum after that tile}
        uint32_t tag = 0u, val = 0u;
        if (g > 0)
          asm volatile("ld.volatile.shared.v2.b32 {%0, %1}, [%2];" : "=r"(tag), "=r"(val) : "r"(chain_row) : "memory");
        tmem_wait_ld();
        // S_w may take the scores of this warpgroup's next tile - unless a second term of P goes there (below)
        tc_fence_before_sync();
        mbar_arrive_warp(bar_kq_ready + 8 * ((g + 2u) % C::NK));
        CFK_PROF_MARK(1)
        if constexpr (DUMP) dump_scores(p, sreg, it.batch, it.head, row_g, j * C::BN);
        if (j * C::BN + 127 > tile_min_lim) {   // this tile has masked columns for some row
          const int ll = lim - j * C::BN;
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (i > ll) sreg[i] = 0xff800000u;  // -inf
        }
        const float rowmax = row_max_n<128>(sreg);
        m_true = fmaxf(m_true, rowmax);
        CFK_PROF_MARK(2)
        // the chain: reference maximum after tile g-1 (the other warpgroup's), decision for tile g, publication.
        // The two threads of a row are the only users of its 8-byte word, so neither a barrier nor a fence is
        // involved: a thread looks at the word until it names tile g-1 (as a rule the early look above did), and
        // writes the word for tile g with one store.  The first tile of an item starts a new chain but still takes
        // its turn, which keeps the word's history in tile order.
        float m_prev = 0.f;
        if (g > 0) {
          uint32_t spins = 0;
          while (tag != g) {
            asm volatile("ld.volatile.shared.v2.b32 {%0, %1}, [%2];" : "=r"(tag), "=r"(val) : "r"(chain_row) : "memory");
            if ((++spins & 0x3ffu) == 0 && (*s_abort || spins > (1u << 24))) {
              if (!*s_abort) { *s_abort = 1u; atomicCAS(p.status, kDevOk, kErrFmhaRowMax); }
              break;
            }
          }
          ok = __all_sync(0xffffffffu, tag == g);
          if (!ok) break;
          m_prev = __uint_as_float(val);
        }
        CFK_PROF_MARK(3)
        bool need = false;
        float m_new;
        if (j == 0) {
          m_new = (rowmax == -INFINITY) ? 0.f : rowmax;
        } else {
          need = (rowmax - m_prev) * sl > C::TAU;
          m_new = need ? rowmax : m_prev;
        }
        asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(chain_row), "r"(g + 1u), "r"(__float_as_uint(m_new)) : "memory");
        // this warpgroup's partial sum follows the reference maximum (which the other warpgroup may have moved)
        if (__any_sync(0xffffffffu, l != 0.f && m_l != m_new)) {
          if (l != 0.f && m_l != m_new) l *= ex2_approx((m_l - m_new) * sl);
        }
        m_l = m_new;
        // P V of this warpgroup's previous tile: complete before P_w is written again.  This also keeps the wait
        // below honest: a parity wait is only meaningful for the barrier's current phase, and P V of tile g-2
        // being complete says that the earlier uses of the barrier of tile g-1 are complete too.
        if (!__all_sync(0xffffffffu, p_free)) {
          ok = mbar_wait_warp(bar_pv_done + 8 * ((g - 2u) % C::NV), ((g - 2u) / C::NV) & 1u, actx, kErrFmhaCorrPv);
          if (!ok) break;
        }
        tc_fence_after_sync();
        if (j > 0 && __any_sync(0xffffffffu, need)) {
          // O holds the tiles before this one at the scale of m_prev: P V of the previous tile may still be running
          ok = mbar_wait_warp(bar_pv_done + 8 * ((g - 1u) % C::NV), ((g - 1u) / C::NV) & 1u, actx, kErrFmhaCorrPv);
          if (!ok) break;
          tc_fence_after_sync();
          rescale_o_row<HD>(tO, need ? ex2_approx((m_prev - m_new) * sl) : 1.f);
        }
        CFK_PROF_MARK(4)
        const float negm = C::PSHIFT - m_new * sl;
        if constexpr (PT == kDtBF16) {
          if (it.split) l += emit_p<128, PT, EMU, true>(sreg, tP, tS, sl, negm);
          else l += emit_p<128, PT, EMU, false>(sreg, tP, 0u, sl, negm);
        } else {
          l += emit_p<128, PT, EMU, false>(sreg, tP, 0u, sl, negm);
        }
        CFK_PROF_MARK(5)
        // an early look at the scores of this warpgroup's next tile (if the CTA has none, nobody asks for the answer);
        // test_wait, because try_wait may put the warp to sleep until the phase completes
        s_ready = mbar_test_wait(bar_s_full + 8 * ((g + 2u) % C::NK), ((g + 2u) / C::NK) & 1u);
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive_warp(bar_pv_ready + 8 * (g % C::NV));
        CFK_PROF_MARK(6)
      }
      if (!ok) break;
      // End of the item.  The statistics slot is free once the previous item's O has been read (o_free).  The
      // warpgroup that owns the item's last tile finishes last: the other one leaves its partial sum (with the
      // maximum it refers to) and its true maximum in the slot, the last one folds its own into them.
      const uint32_t g_last = g - 1u;                  // the item's last tile
      const bool two = it.n >= 2;
      if (it.k > 0) {   // every warpgroup looks at every phase of this barrier: a parity wait must not skip one
        ok = mbar_wait_warp(bar_o_free, (uint32_t)(it.k - 1) & 1u, actx, kErrFmhaOFree);
        if (!ok) break;
      }
      if ((g_last & 1u) != w && !two) continue;       // a one-tile item of the other warpgroup
      if ((g_last & 1u) != w) {
        g_stats[r] = l; g_stats[128 + r] = m_l; g_stats[256 + r] = m_true;
        mbar_arrive_warp(bar_fin + 8 * q);
      } else {
        float lt = l, mt = m_true;
        if (two) {
          ok = mbar_wait_warp(bar_fin + 8 * q, fins & 1u, actx, kErrFmhaStats);
          if (!ok) break;
          const float l_o = g_stats[r], m_o = g_stats[128 + r];
          mt = fmaxf(mt, g_stats[256 + r]);
          // the chain never decreases and this warpgroup decided last, so m_l >= m_o
          lt += l_o * ex2_approx((m_o - m_l) * sl);
        }
        g_stats[r] = lt; g_stats[128 + r] = m_l; g_stats[256 + r] = mt;
        mbar_arrive_warp(bar_stats);
      }
      if (two) ++fins;
    }
    CFK_PROF_MARK(7)
    CFK_PROF_FLUSH(0, 8, (warp == 0 && lane == 0))
  }

  // ---- tear-down ----
  settle_if_aborted(s_abort);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 12) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace cfk
