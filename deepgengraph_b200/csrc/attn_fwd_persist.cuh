// Persistent variant of the attention forward kernel (head_dim 128: two CTAs per SM; head_dim 256: one).
//
// Same tiling, TMEM plan and warp roles as attn_fwd_kernel<D, 64, 1, 2> (one 128-row query tile at a time, two
// S buffers), but the grid is CTAS_PER_SM x #SM CTAs that each walk a sequence of query tiles:
//   * tiles are handed out by an atomic counter, (batch, head) units in L2-sized groups and tile-major,
//     heaviest tile first inside a group (see decode_item), so the SMs drain evenly;
//   * every barrier, the K/V ring and the TMEM buffers run continuously across tile boundaries (phases follow
//     CTA-global counters), so the next tile's Q/K loads and its first S = Q K^T MMAs overlap the current tile's
//     epilogue.  A non-persistent launch pays ~6 us of un-overlapped set-up, pipeline fill and epilogue per
//     tile and leaves the slot idle between CTAs.
// Per-CTA roles: warps 0-3 softmax warpgroup, warp 4 TMA producer + tile scheduler, warp 5 MMA issuer.
#pragma once

#include "attn_fwd.cuh"

namespace b200 {

#ifndef B200_PERSIST_MIDBATCH_WAITS
#define B200_PERSIST_MIDBATCH_WAITS 1
#endif

struct SchedParams {
  unsigned int* counter;   // [2]: next item, CTAs finished; both return to 0 when the last CTA leaves
  int n_q_tiles;           // query tiles per (batch, head)
  int total_items;         // batch * heads * n_q_tiles
  int group_heads;         // (batch, head) units per scheduling group
};

struct TileInfo {
  int q0, h, hk, b, lo, hi;
};

// Work order: the (batch, head) units are taken in groups of `group_heads`; inside a group the items run
// tile-major, heaviest query tile first (all heads' last tile, then all heads' second-to-last tile, ...).
// The K/V of one group (group_heads x 2 x kv_len x D x 2 bytes; 32 MB for 16 heads at 4096 keys) stay
// L2-resident while ~2 x #SM CTAs walk it, and the launch ends on the LIGHTEST tiles, so that the CTAs drain
// within a few key blocks of each other (longest-processing-time-first order).
__device__ __forceinline__ TileInfo decode_item(int item, const FwdParams& p, const SchedParams& sp, int bn) {
  TileInfo t;
  const int per_group = sp.group_heads * sp.n_q_tiles;
  const int grp = item / per_group;
  const int r = item - grp * per_group;
  const int units = p.batch * p.heads;
  const int in_group = min(sp.group_heads, units - grp * sp.group_heads);   // the last group may be smaller
  const int rank = r / in_group;                                            // 0 = heaviest tile
  const int bh = grp * sp.group_heads + (r - rank * in_group);
  const int qt = sp.n_q_tiles - 1 - rank;
  t.b = bh / p.heads;
  t.h = bh - t.b * p.heads;
  t.hk = t.h / (p.heads / p.kv_heads);
  t.q0 = qt * 128;
  const TileRange rg = tile_range(t.q0, bn, p);
  t.lo = rg.lo;
  t.hi = rg.hi;
  return t;
}

// Q as the TMEM-resident A operand of S = Q K^T (0 = both operands in shared memory) and the S buffers that
// then fit: head_dim 128 shares the SM between two CTAs (256 columns each: S 64 + Q 64 + O 128), head_dim 256
// has the SM to itself (S 2 x 64 + Q 128 + O 256 = 512).
#ifndef B200_FWD_QT128
#define B200_FWD_QT128 0
#endif
#ifndef B200_FWD_QT256
#define B200_FWD_QT256 1
#endif

template <int D_, bool QT_ = (D_ == 128 ? B200_FWD_QT128 : B200_FWD_QT256) != 0>
struct PersistCfg : FwdCfg<D_, 64, 1, (QT_ && D_ == 128) ? 1 : 2> {
  using Base = FwdCfg<D_, 64, 1, (QT_ && D_ == 128) ? 1 : 2>;
  static constexpr bool QT = QT_;
  static constexpr int Q_COL = Base::SB * Base::BN;   // first TMEM column of the Q operand
  static_assert(!QT || (Q_COL + D_ / 2 <= Base::O_BASE && Base::TMEM_USED <= Base::TMEM_COLS), "TMEM plan");
  static constexpr int SOFTMAX_WARPS = 4;
  static constexpr int THREADS_P = (SOFTMAX_WARPS + 2) * 32;
  static constexpr int BAR_SCHED = Base::NUM_BARS;        // [2] tile descriptor slot k % 2 published
  static constexpr int BAR_Q_FREE = BAR_SCHED + 2;        // last S MMA of a tile retired: Q buffer reusable
  static constexpr int BAR_SCHED_FREE = BAR_Q_FREE + 1;   // [2] descriptor slot read by all its consumers
  static constexpr int BAR_QT_FULL = BAR_SCHED_FREE + 2;  // Q operand of the tile is in TMEM
  static constexpr int NUM_BARS_P = BAR_QT_FULL + 1;
  static constexpr int SMEM_BYTES_P = Base::SMEM_TILES + NUM_BARS_P * 8 + 64 + 1024;
  static_assert(SMEM_BYTES_P <= Base::SMEM_BUDGET, "shared memory budget exceeded");
};

template <int D_, bool BF16, bool SOFTCAP>
__global__ void __launch_bounds__(PersistCfg<D_>::THREADS_P, PersistCfg<D_>::CTAS_PER_SM)
attn_fwd_persist_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_v, const FwdParams p, const SchedParams sp) {
  using Cfg = PersistCfg<D_>;
  constexpr int SL = Cfg::SLOTS, D = Cfg::D, BN = Cfg::BN, BM = Cfg::BM, SB = Cfg::SB;
  constexpr int PRODUCER_WARP = Cfg::SOFTMAX_WARPS;
  constexpr bool QT = Cfg::QT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

  // A launch that follows an expired wait on this device drains immediately (the status word stays set until the
  // host reads it).  The word is loaded here and looked at after the set-up below, whose barrier it shares: a
  // global load of its own before anything else costs every launch most of a microsecond.
  __shared__ int s_skip;
  int status_now = 0;
  if (threadIdx.x == 0) status_now = *reinterpret_cast<volatile int*>(&g_device_status);

  [[maybe_unused]] const uint64_t cta_start_ns = global_timer_ns();
  [[maybe_unused]] const long long cta_start_clk = clock64();
  [[maybe_unused]] int blocks_done = 0;
  B200_TL_INIT();
  FwdCtx<Cfg, BF16> c;
  c.sQ = smem;
  c.sKV = c.sQ + Cfg::Q_TILE_BYTES;
  c.bars = reinterpret_cast<uint64_t*>(c.sKV + SL * Cfg::KV_STAGE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(c.bars + Cfg::NUM_BARS_P);
  c.abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* sched = reinterpret_cast<volatile int*>(tmem_slot + 2);   // [2] item index or -1

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < Cfg::NUM_BARS_P; ++i) {
      const bool is_p_full = (i >= Cfg::BAR_P_FULL && i < Cfg::BAR_P_FULL + SB);   // every softmax warp
      const bool is_sched_free = (i >= Cfg::BAR_SCHED_FREE && i < Cfg::BAR_SCHED_FREE + 2);   // + the MMA issuer
      // with Q in TMEM the softmax warps fill it from the shared-memory tile and release that tile themselves
      const bool is_q_copy = QT && (i == Cfg::BAR_QT_FULL || i == Cfg::BAR_Q_FREE);
      mbar_init(&c.bars[i], is_sched_free ? (uint32_t)Cfg::SOFTMAX_WARPS + 1u
                                          : (is_p_full || is_q_copy) ? (uint32_t)Cfg::SOFTMAX_WARPS : 1u);
    }
    *c.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == PRODUCER_WARP && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if (threadIdx.x == 0) s_skip = status_now;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  c.tmem_base = *tmem_slot;
  if (s_skip != 0) {   // (the tile counter is untouched: the host zeroes it when it clears the status word)
    if (warp == 0) tmem_dealloc(c.tmem_base, Cfg::TMEM_COLS);
    return;
  }

  if (warp < PRODUCER_WARP) {
    // ------------------------------ softmax warps ------------------------------
    const int warp_q = warp & 3;
    const uint32_t lane_addr = c.tmem_base + ((uint32_t)(warp_q * 32) << 16);
    const uint32_t o_addr = lane_addr + Cfg::O_BASE;
    uint64_t* o_full = &c.bars[Cfg::BAR_O_FULL];
    const float cmul = SOFTCAP ? p.cap_out : p.scale_log2;
    int g = 0;   // blocks processed by this CTA so far (S / P buffer = g % SB, barrier phases follow g)
    // Q in TMEM: thread r moves row r of tile k2's Q from the (swizzled) shared-memory tile into TMEM lane r.  Every S MMA of the previous tile has completed by then (its last S tile was
    // awaited before that tile's last softmax step), so the columns are free.
    [[maybe_unused]] auto stage_q = [&](int k2) -> bool {
      if (!mbar_wait(&c.bars[Cfg::BAR_Q_FULL], k2 & 1, c.abort_flag, WAIT_Q_FULL)) return false;
      constexpr int NCH = D / 8;   // 16-byte pieces of the row
      const int r = warp_q * 32 + lane;
      const uint8_t* qrow = c.sQ + r * 128;
#pragma unroll
      for (int cc = 0; cc < NCH; cc += 8) {
        uint32_t w[32];
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          const int piece = cc + v, ks = piece >> 3, ci = piece & 7;
          const uint4 x = *reinterpret_cast<const uint4*>(qrow + ks * (BM * 128) + ((ci ^ (r & 7)) << 4));
          w[4 * v] = x.x;
          w[4 * v + 1] = x.y;
          w[4 * v + 2] = x.z;
          w[4 * v + 3] = x.w;
        }
        tmem_st32(lane_addr + Cfg::Q_COL + cc * 4, w);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&c.bars[Cfg::BAR_QT_FULL]);
        mbar_arrive(&c.bars[Cfg::BAR_Q_FREE]);
      }
      return true;
    };
    bool q_staged = false;   // the coming tile's Q was moved before the previous tile's epilogue
    for (int k = 0;; ++k) {
      if (!mbar_wait(&c.bars[Cfg::BAR_SCHED + (k & 1)], (k >> 1) & 1, c.abort_flag, WAIT_SCHED)) break;
      const int item = sched[k & 1];
      __syncwarp();
      if (lane == 0) mbar_arrive(&c.bars[Cfg::BAR_SCHED_FREE + (k & 1)]);   // slot may be rewritten for tile k + 2
      if (item < 0) break;
      if constexpr (QT) {
        if (!q_staged && !stage_q(k)) break;
        q_staged = false;
      }
      const TileInfo t = decode_item(item, p, sp, BN);
      const int row = t.q0 + warp_q * 32 + lane;
      float m = -1.0e30f, l = 0.f;
      const int hi_key = p.causal ? min(row + p.delta, p.kv_len - 1) : p.kv_len - 1;
      const int lo_key = (p.causal && p.window > 0) ? (row + p.delta - p.window + 1) : -(1 << 28);
      const int hi_first = p.causal ? min(t.q0 + p.delta, p.kv_len - 1) : p.kv_len - 1;
      const int lo_last = (p.causal && p.window > 0) ? (t.q0 + 127 + p.delta - p.window + 1) : -(1 << 28);
      bool ok = true;
      for (int j = t.lo; j < t.hi && ok; ++j, ++g) {
        const int n = j - t.lo, buf = g % SB;
        const uint32_t s_addr = lane_addr + buf * BN;
        uint64_t* p_full = &c.bars[Cfg::BAR_P_FULL + buf];
        if (threadIdx.x == 0 && g < 64) B200_TL((g & 63) * 8 + 5);
        ok = mbar_wait(&c.bars[Cfg::BAR_S_FULL + buf], (g / SB) & 1, c.abort_flag, WAIT_S_FULL);
        if (!ok) break;
        if (threadIdx.x == 0 && g < 64) B200_TL((g & 63) * 8 + 6);
        tc_fence_after();
        const bool need_mask = (hi_first - j * BN < BN - 1) || (lo_last - j * BN > 0);
        if (need_mask) {
          ok = fwd_softmax_block<Cfg, BF16, SOFTCAP, true>(c, p, s_addr, o_addr, o_full, p_full, n, g, lo_key - j * BN,
                                                           hi_key - j * BN, cmul, m, l, nullptr, 0, nullptr);
        } else {
          ok = fwd_softmax_block<Cfg, BF16, SOFTCAP, false>(c, p, s_addr, o_addr, o_full, p_full, n, g, 0, 0, cmul, m, l,
                                                            nullptr, 0, nullptr);
        }
      }
      if (!ok) break;
      // epilogue of this tile; the MMA issuer is already computing the next tile's first S tiles meanwhile.
      // The next tile's first P V (which overwrites O) is issued only after this warpgroup has delivered that
      // tile's first P, i.e. after the loads below have completed.
      if constexpr (QT) {
        // Next tile's Q first if it has landed (its first S MMAs then run under this tile's epilogue); otherwise
        // the epilogue goes first and the move happens at the top of the loop.
        if (mbar_test_wait(&c.bars[Cfg::BAR_SCHED + ((k + 1) & 1)], ((k + 1) >> 1) & 1) && sched[(k + 1) & 1] >= 0 &&
            mbar_test_wait(&c.bars[Cfg::BAR_Q_FULL], (k + 1) & 1)) {
          if (!stage_q(k + 1)) break;
          q_staged = true;
        }
      }
      const int last = g - 1;
      // (tuning builds: slots (3 * 64 + 48 + tile) * 8 + {0: last P delivered, 1: last P V complete, 2: output stored})
      if (threadIdx.x == 0 && k < 8) B200_TL((3 * 64 + 48 + k) * 8 + 0);
      if (!mbar_wait(o_full + (last & 1), (last >> 1) & 1, c.abort_flag, WAIT_O_FULL)) break;
      tc_fence_after();
      if (threadIdx.x == 0 && k < 8) B200_TL((3 * 64 + 48 + k) * 8 + 1);
      const float inv_l = 1.0f / l;
      const bool in_range = row < p.q_len;
      const bool wide_stores = (reinterpret_cast<uintptr_t>(p.out) & 31) == 0;
      uint4* out_row = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.out) +
                                                (((int64_t)t.b * p.q_len + row) * p.heads + t.h) * (int64_t)D);
#pragma unroll
      for (int ch = 0; ch < D / 32; ++ch) {
        uint32_t o[32];
        tmem_ld32(o_addr + ch * 32, o);
        tmem_ld_wait();
        if (threadIdx.x == 0 && k < 8 && ch < 4) B200_TL((3 * 64 + 48 + k) * 8 + 3 + ch);   // chunk ch loaded
        if (in_range) {
          // every lane writes its own row (rows are heads * D elements apart), so a store instruction costs one
          // memory transaction per lane whatever its width: 32-byte stores halve the count
#pragma unroll
          for (int v = 0; v < 2; ++v) {
            uint32_t w[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)
              w[e] = pack2<BF16>(__uint_as_float(o[v * 16 + 2 * e]) * inv_l, __uint_as_float(o[v * 16 + 2 * e + 1]) * inv_l);
            if (wide_stores) {
              st_global_v8(out_row + ch * 4 + v * 2, w);
            } else {
              out_row[ch * 4 + v * 2] = make_uint4(w[0], w[1], w[2], w[3]);
              out_row[ch * 4 + v * 2 + 1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
          }
        }
      }
      if (p.lse != nullptr && in_range) p.lse[((int64_t)t.b * p.heads + t.h) * p.lse_stride + row] = m + log2f(l);
      if (threadIdx.x == 0 && k < 8) B200_TL((3 * 64 + 48 + k) * 8 + 2);
      blocks_done = g;
    }
  } else if (warp == PRODUCER_WARP) {
    // --------------------------- TMA producer + tile scheduler ---------------------------
    if (lane == 0) {
      int ring_i = 0;   // K/V ring items issued so far (continuous across tiles)
      bool ok = true;
      for (int k = 0; ok; ++k) {
        // the first tile of a CTA is its own index (no round trip to the counter before the first load is issued)
        const int item = k == 0 ? (int)blockIdx.x : (int)(gridDim.x + atomicAdd(&sp.counter[0], 1u));
        const bool valid = item < sp.total_items;
        // Slot k % 2 still holds the descriptor of tile k-2 until the four softmax warps and the issuer have all
        // read it (with tiles of one or two key blocks the issuer can finish a tile's S MMAs, and this thread
        // its loads, before the softmax warpgroup has even left the previous tile's epilogue).
        if (k >= 2 && !mbar_wait(&c.bars[Cfg::BAR_SCHED_FREE + (k & 1)], ((k >> 1) - 1) & 1, c.abort_flag, WAIT_SCHED)) {
          ok = false;
          break;
        }
        sched[k & 1] = valid ? item : -1;
        mbar_arrive(&c.bars[Cfg::BAR_SCHED + (k & 1)]);
        if (!valid) {
          // last CTA out resets the counters for the next launch that uses this pair
          __threadfence();
          const unsigned done = atomicAdd(&sp.counter[1], 1u);
          if (done == gridDim.x - 1) {
            sp.counter[0] = 0;
            sp.counter[1] = 0;
            __threadfence();
          }
          break;
        }
        const TileInfo t = decode_item(item, p, sp, BN);
        if (k > 0) ok = mbar_wait(&c.bars[Cfg::BAR_Q_FREE], (k - 1) & 1, c.abort_flag, WAIT_Q_FREE);
        if (!ok) break;
        mbar_expect_tx(&c.bars[Cfg::BAR_Q_FULL], Cfg::Q_TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < Cfg::KSUB; ++ks)
          tma_load_4d(c.sQ + ks * (BM * 128), &tm_q, &c.bars[Cfg::BAR_Q_FULL], ks * 64, t.h, t.q0, t.b);
        const int nb = t.hi - t.lo;
        auto load = [&](bool is_v, int n) {
          const int slot = ring_i % SL, use = ring_i / SL;
          if (use > 0 && !mbar_wait(&c.bars[Cfg::BAR_EMPTY + slot], (use - 1) & 1, c.abort_flag, WAIT_K_EMPTY)) {
            ok = false;
            return;
          }
          uint64_t* full = &c.bars[Cfg::BAR_FULL + slot];
          uint8_t* dst = c.sKV + slot * Cfg::KV_STAGE_BYTES;
          mbar_expect_tx(full, Cfg::KV_STAGE_BYTES);
#pragma unroll
          for (int ks = 0; ks < Cfg::KSUB; ++ks)
            tma_load_4d(dst + ks * (BN * 128), is_v ? &tm_v : &tm_k, full, ks * 64, t.hk, (t.lo + n) * BN, t.b);
          ++ring_i;
        };
        for (int n = 0; n < SB && n < nb && ok; ++n) load(false, n);
        for (int n = 0; n < nb && ok; ++n) {
          load(true, n);
          if (ok && n + SB < nb) load(false, n + SB);
        }
      }
      if (!ok || *c.abort_flag != 0) {
        // abort path: let our own bulk copies land before the CTA exits (bounded, 20 ms)
        const uint64_t t0 = global_timer_ns();
        for (int slot = 0; slot < SL; ++slot) {
          if (ring_i <= slot) continue;
          const int last = slot + ((ring_i - 1 - slot) / SL) * SL;
          while (!mbar_try_wait(&c.bars[Cfg::BAR_FULL + slot], (last / SL) & 1) &&
                 global_timer_ns() - t0 < 20000000ull) {
          }
        }
      }
    }
  } else {
    // ---------------------------------- MMA issuer ----------------------------------
    constexpr uint32_t IDESC_S = make_idesc(BF16, BM, BN, false, false);
    constexpr uint32_t IDESC_PV = make_idesc(BF16, BM, D, false, true);
    const uint32_t desc_hi = smem_desc_hi(1024);
    const uint32_t q_lo = smem_desc_lo(smem_u32(c.sQ), 16);
    const uint32_t k_lo = smem_desc_lo(smem_u32(c.sKV), 16);
    const uint32_t v_lo = smem_desc_lo(smem_u32(c.sKV), BN * 128);
    const uint32_t o_tmem = c.tmem_base + Cfg::O_BASE;
    auto issue_s = [&](int slot, int gb, bool last_of_tile) {
      const uint32_t b0 = k_lo + (uint32_t)(slot * (Cfg::KV_STAGE_BYTES >> 4));
      const uint32_t s_tmem = c.tmem_base + (gb % SB) * BN;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t a_off = (uint32_t)(((kk / 4) * (BM * 128) + (kk % 4) * 32) >> 4);
        const uint32_t b_off = (uint32_t)(((kk / 4) * (BN * 128) + (kk % 4) * 32) >> 4);
        if constexpr (QT) {
          // 16 dims (one K step) = 8 TMEM columns of packed 16-bit pairs
          const uint32_t a_tmem = c.tmem_base + Cfg::Q_COL + kk * 8;
          if (kk == 0)
            umma_ts_c<IDESC_S, 0>(s_tmem, a_tmem, b0 + b_off, desc_hi);
          else
            umma_ts_c<IDESC_S, 1>(s_tmem, a_tmem, b0 + b_off, desc_hi);
        } else {
          if (kk == 0)
            umma_ss_c<IDESC_S, 0>(s_tmem, q_lo + a_off, b0 + b_off, desc_hi);
          else
            umma_ss_c<IDESC_S, 1>(s_tmem, q_lo + a_off, b0 + b_off, desc_hi);
        }
      }
      umma_commit(&c.bars[Cfg::BAR_S_FULL + (gb % SB)]);
      if (!QT && last_of_tile) umma_commit(&c.bars[Cfg::BAR_Q_FREE]);   // no later MMA reads this tile's Q
    };
    auto issue_pv = [&](int slot, int gb, bool first_of_tile) {
      const uint32_t b0 = v_lo + (uint32_t)(slot * (Cfg::KV_STAGE_BYTES >> 4));
      const uint32_t s_tmem = c.tmem_base + (gb % SB) * BN;
      if (first_of_tile)
        umma_ts_c<IDESC_PV, 0>(o_tmem, s_tmem, b0, desc_hi);
      else
        umma_ts_c<IDESC_PV, 1>(o_tmem, s_tmem, b0, desc_hi);
#pragma unroll
      for (int kk = 1; kk < BN / 16; ++kk)
        umma_ts_c<IDESC_PV, 1>(o_tmem, s_tmem + kk * 8, b0 + (uint32_t)(kk * (2048 >> 4)), desc_hi);
      umma_commit(&c.bars[Cfg::BAR_O_FULL + (gb & 1)]);
    };
    int ring_i = 0, g0 = 0;   // ring items consumed, blocks issued before this tile
    bool ok = true;
    for (int k = 0; ok; ++k) {
      if (!mbar_wait(&c.bars[Cfg::BAR_SCHED + (k & 1)], (k >> 1) & 1, c.abort_flag, WAIT_SCHED)) break;
      const int item = sched[k & 1];
      __syncwarp();
      if (lane == 0) mbar_arrive(&c.bars[Cfg::BAR_SCHED_FREE + (k & 1)]);
      if (item < 0) break;
      const TileInfo t = decode_item(item, p, sp, BN);
      const int nb = t.hi - t.lo;
      ok = mbar_wait(&c.bars[QT ? Cfg::BAR_QT_FULL : Cfg::BAR_Q_FULL], k & 1, c.abort_flag, WAIT_Q_FULL);
      if (QT) tc_fence_after();
      // S of the first SB blocks
      for (int n = 0; n < SB && n < nb && ok; ++n) {
        const int slot = ring_i % SL, ph = (ring_i / SL) & 1;
        ++ring_i;
        ok = mbar_wait(&c.bars[Cfg::BAR_FULL + slot], ph, c.abort_flag, WAIT_K_FULL);
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          issue_s(slot, g0 + n, n == nb - 1);
          umma_commit(&c.bars[Cfg::BAR_EMPTY + slot]);
        }
        __syncwarp();
      }
#if B200_PERSIST_MIDBATCH_WAITS
      // Steady state, one step per key block: [O += P(n) V(n)] then [S(n+SB) = Q K(n+SB)^T].  The tensor pipe
      // accepts only a handful of MMAs ahead of the one it executes, so between the last MMA of one step and the
      // first MMA of the next the issuer has a few hundred clocks before the pipe runs dry -- and every barrier
      // probe costs ~100 of them while the S MMAs saturate the shared-memory port.  Only the wait for P(n)
      // sits in that window: the ring-slot barriers of K(n+SB) and V(n+1) are observed between the two GEMMs,
      // while the four P V MMAs execute.
      int vslot = ring_i % SL, vph = (ring_i / SL) & 1;
      ++ring_i;
      if (ok) ok = mbar_wait(&c.bars[Cfg::BAR_FULL + vslot], vph, c.abort_flag, WAIT_V_FULL);   // V(0)
      for (int n = 0; n < nb && ok; ++n) {
        const bool has_k = n + SB < nb;
        const int kslot = ring_i % SL, kph = (ring_i / SL) & 1;
        if (has_k) ++ring_i;
        const bool has_v = n + 1 < nb;
        const int nvslot = ring_i % SL, nvph = (ring_i / SL) & 1;
        if (has_v) ++ring_i;
        const int gb = g0 + n;
        if (lane == 0 && gb < 64) B200_TL((3 * 64 + (gb & 63)) * 8 + 0);
        ok = mbar_wait(&c.bars[Cfg::BAR_P_FULL + (gb % SB)], (gb / SB) & 1, c.abort_flag, WAIT_P_FULL);
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          if (gb < 64) B200_TL((3 * 64 + (gb & 63)) * 8 + 1);
          issue_pv(vslot, gb, n == 0);
          umma_commit(&c.bars[Cfg::BAR_EMPTY + vslot]);
          if (gb < 64) B200_TL((2 * 64 + (gb & 63)) * 8 + 1);
        }
        __syncwarp();
        if (has_k) ok = mbar_wait(&c.bars[Cfg::BAR_FULL + kslot], kph, c.abort_flag, WAIT_K_FULL);
        if (ok && has_v) ok = mbar_wait(&c.bars[Cfg::BAR_FULL + nvslot], nvph, c.abort_flag, WAIT_V_FULL);
        if (!ok) break;
        tc_fence_after();
        if (has_k) {
          if (elect_one()) {
            if (gb < 64) B200_TL((2 * 64 + (gb & 63)) * 8 + 2);
            issue_s(kslot, gb + SB, n + SB == nb - 1);
            umma_commit(&c.bars[Cfg::BAR_EMPTY + kslot]);
            if (gb < 64) B200_TL((2 * 64 + (gb & 63)) * 8 + 3);
          }
          __syncwarp();
        }
        vslot = nvslot;
      }
#else
      // steady state: [O += P(n) V(n)] [S(n+SB)] back to back; ring slots observed first, P last
      for (int n = 0; n < nb && ok; ++n) {
        const int vslot = ring_i % SL, vph = (ring_i / SL) & 1;
        ++ring_i;
        const bool has_k = n + SB < nb;
        const int kslot = ring_i % SL, kph = (ring_i / SL) & 1;
        if (has_k) ++ring_i;
        const int gb = g0 + n;
        ok = mbar_wait(&c.bars[Cfg::BAR_FULL + vslot], vph, c.abort_flag, WAIT_V_FULL);
        if (ok && has_k) ok = mbar_wait(&c.bars[Cfg::BAR_FULL + kslot], kph, c.abort_flag, WAIT_K_FULL);
        if (ok) ok = mbar_wait(&c.bars[Cfg::BAR_P_FULL + (gb % SB)], (gb / SB) & 1, c.abort_flag, WAIT_P_FULL);
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          issue_pv(vslot, gb, n == 0);
          if (has_k) issue_s(kslot, gb + SB, n + SB == nb - 1);
          umma_commit(&c.bars[Cfg::BAR_EMPTY + vslot]);
          if (has_k) umma_commit(&c.bars[Cfg::BAR_EMPTY + kslot]);
        }
        __syncwarp();
      }
#endif
      g0 += nb;
    }
    // every MMA issued above has retired before the CTA tears TMEM down
    if (elect_one()) umma_commit(&c.bars[Cfg::BAR_DRAIN]);
    __syncwarp();
    mbar_wait(&c.bars[Cfg::BAR_DRAIN], 0, c.abort_flag, WAIT_DRAIN);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(c.tmem_base, Cfg::TMEM_COLS);
  B200_TL_FLUSH();
  B200_TL_CTA(cta_start_ns, cta_start_clk, blocks_done);
}

// Pool of scheduler counter pairs in the library image: one pair per launch, handed out round-robin, returned
// to zero by the last CTA of the launch that used it.
constexpr int kSchedPool = 256;
__device__ unsigned int g_sched_counters[kSchedPool * 2];

inline int sched_counter_for_launch(unsigned int** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static unsigned int* base[kMaxDevices] = {};
  static unsigned int seq[kMaxDevices] = {};
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return B200_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(mu);
  if (base[dev] == nullptr) {
    void* ptr = nullptr;
    B200_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_sched_counters));
    base[dev] = static_cast<unsigned int*>(ptr);
  }
  *out = base[dev] + 2 * (seq[dev]++ % kSchedPool);
  return B200_OK;
}

template <int D_, bool BF16, bool SOFTCAP>
int launch_attn_fwd_persist(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FwdParams& p,
                            cudaStream_t stream) {
  using Cfg = PersistCfg<D_>;
  auto kern = attn_fwd_persist_kernel<D_, BF16, SOFTCAP>;
  static thread_local int configured_dev = -1;
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    B200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES_P));
    configured_dev = dev;
  }
  SchedParams sp;
  int rc = sched_counter_for_launch(&sp.counter);
  if (rc != B200_OK) return rc;
  sp.n_q_tiles = (p.q_len + 127) / 128;
  sp.total_items = p.batch * p.heads * sp.n_q_tiles;
  // group size: K/V of a group within a quarter of L2 (~32 MB), at least 1 and at most 32 units
  {
    const int64_t kv_bytes_per_unit = (int64_t)2 * p.kv_len * D_ * 2;
    int gh = (int)std::max<int64_t>(1, std::min<int64_t>(32, ((int64_t)32 << 20) / kv_bytes_per_unit));
    static const char* env = std::getenv("B200_ATTN_GROUP_HEADS");
    if (env != nullptr && std::atoi(env) > 0) gh = std::atoi(env);
    sp.group_heads = gh;
  }
  const int grid = std::min(sp.total_items, Cfg::CTAS_PER_SM * sm_count());
  kern<<<grid, Cfg::THREADS_P, Cfg::SMEM_BYTES_P, stream>>>(tq, tk, tv, p, sp);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

}  // namespace b200
