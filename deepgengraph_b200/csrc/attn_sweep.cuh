// Score sweeps for the fine-grained-property variants (H2O / RoCo / KeyFormer).
//
// The per-key statistics need the FINAL softmax normaliser of every query row, so they are a
// second sweep over the logits after the forward kernel has produced the base-2 log-sum-exp of
// each row.  The sweep keeps one 128-row tile stationary (in shared memory for 128-wide streamed
// blocks, in TMEM as the A operand for 64-wide ones) and streams blocks of the other operand
// through a TMA ring; the tile product lands in TMEM (double buffered)
// with the STATIONARY rows on the TMEM lanes, so that every thread of the compute warpgroup
// owns one stationary row and reduces along the streamed dimension in registers:
//
//   SWEEP_COLSUM     stationary = 128 keys,    streamed = query blocks.
//                    thread j accumulates sum_i p_ij (and sum_i p_ij^2): no cross-thread
//                    reduction at all.  Query blocks are split into chunks over CTAs; each CTA
//                    writes one partial vector and a small pass adds the partials in a fixed
//                    order (no atomics, bit-reproducible).
//                    -- H2O.forward kernels/h2o.py:35-38, RoCo.forward kernels/roco.py:42-48
//   SWEEP_KF_COLSUM  same, with p2_ij = exp2((x_ij - log2 e_ij) / tau - Lz_i), e = exp_rand
//                    -- KeyFormer.forward kernels/kf.py:36-42
//   SWEEP_KF_ROWLSE  stationary = 128 queries, streamed = key blocks; thread i runs an online
//                    log-sum-exp of z_ij = (x_ij - log2 e_ij) / tau over the keys -> Lz_i.
//
// x_ij are the scaled (and soft-capped) logits in base-2 units, exactly as in the forward kernel.
#pragma once

#include <type_traits>

#include "common.cuh"
#include "attn_fwd.cuh"

namespace b200 {

enum SweepMode : int { SWEEP_COLSUM = 0, SWEEP_KF_COLSUM = 1, SWEEP_KF_ROWLSE = 2 };
// second per-key statistic of the column-sum sweep: none, sum of p^2 (RoCo), or the Corm flag
enum SweepAux : int { AUX_NONE = 0, AUX_SQUARES = 1, AUX_CORM = 2 };

// Of every 8 groups of 4 columns of an unmasked block, this many take their exponentials from the FMA-pipe
// polynomial instead of the special-function unit (column-sum sweeps).
#ifndef B200_SWEEP_POLY_OF_8
#define B200_SWEEP_POLY_OF_8 0
#endif
constexpr int kSweepPolyOf8 = B200_SWEEP_POLY_OF_8;

// ---------------------------------------------------------------------------------------------
// In-kernel noise for the KeyFormer sweeps (no counterpart in the reference, whose modules take the noise as a
// [B, H, Sq, Skv] fp32 tensor, kernels/kf.py:19,36-37, drawn by the caller, kf.py:48 / models/kf.py:44).
// Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11), a counter-based
// generator: the four 32-bit outputs of counter (j >> 2, i, b * heads + h, 0) under key (seed_lo, seed_hi) belong to
// query i and keys 4 * (j >> 2) .. + 3, so any (query, key) element can be produced anywhere, in any order.
// Output word r maps to u = ((r >> 9) + 1/2) * 2^-23 in (0, 1) and exp_rand = -ln(u), which makes -ln(exp_rand) an
// exact Gumbel(0, 1) variate; deepgengraph_b200.attention.kf_noise materialises the same tensor on the host side.
// ---------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0, n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
    c[1] = (uint32_t)p1;
    c[3] = (uint32_t)p0;
    c[0] = n0;
    c[2] = n2;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

// log2(exp_rand) of one Philox output word.  exp_rand = -ln(u): for u within 2^-8 of one the logarithm comes from the
// series -ln(1 - v) = v + v^2/2 + v^3/3 (lg2.approx has an ABSOLUTE error of 2^-22 on (0.5, 2), which near u = 1 is
// as large as the result itself); elsewhere from lg2.approx.  Relative error of exp_rand below 5e-5 everywhere.
__device__ __forceinline__ float kf_gen_log2_exp_rand(uint32_t r) {
  const float t = __uint_as_float(0x3f800000u | (r >> 9)) - 1.0f;      // k * 2^-23, exact
  const float u = t + 5.9604644775390625e-08f;                         // + 2^-24: exact, in (0, 1)
  const float v = 0.99999994039535522461f - t;                         // 1 - u, exact
  const float series = v * fmaf(v, fmaf(v, 0.33333334f, 0.5f), 1.0f);
  const float e = v < 0.00390625f ? series : -lg2_approx(u) * 0.69314718055994530942f;
  return lg2_approx(e);
}

// x[u] <- x[u ^ c] for c in 0..3 (two conditional swap stages)
__device__ __forceinline__ void xor_permute4(uint32_t (&x)[4], uint32_t c) {
  if (c & 1u) {
    uint32_t t = x[0]; x[0] = x[1]; x[1] = t;
    t = x[2]; x[2] = x[3]; x[3] = t;
  }
  if (c & 2u) {
    uint32_t t = x[0]; x[0] = x[2]; x[2] = t;
    t = x[1]; x[1] = x[3]; x[3] = t;
  }
}

struct SweepParams {
  const float* lse;     // [B*H][lse_stride]  row normalisers (COLSUM: L, KF_COLSUM: Lz)
  float* lse_out;       // [B*H][lse_stride]  KF_ROWLSE output
  float* partial;       // [B*H][n_chunks][kv_pad]
  float* partial_sq;    // same shape, RoCo only
  int batch, heads, q_len, kv_len, delta, causal, window;
  int lse_stride, kv_pad, n_chunks, chunk_blocks;
  int kv_group;         // query heads per K/V head (the key operand of head h is K head h / kv_group)
  // stationary operand as plain memory (configurations that keep it in TMEM load it with ordinary loads):
  const uint16_t* a_base;   // K (column-sum sweeps) or Q (row-LSE sweep), [batch, rows, a_heads, 128]
  int a_rows, a_heads;
  float scale_log2, cap_in, cap_out, inv_tau;
  uint32_t seed_lo, seed_hi;   // key of the in-kernel noise generator (KeyFormer sweeps without a noise tensor)
};

// CWG_ = compute warpgroups per CTA.  With two, warpgroup g reduces columns [g * BX/2, (g+1) * BX/2) of every
// product tile (both cover all 128 TMEM lanes, i.e. all stationary rows) and the two partial results of a row are
// added once at the end: twice the warps per scheduler hide the TMEM-load, shared-memory and special-function
// latencies of the element loop, which with one warp per scheduler and CTA bound the sweep (measured: special-
// function unit 55 % busy, issue slots 37 %, moving exponentials to the FMA pipe changed nothing).
// GEN_ (KeyFormer sweeps): the noise comes from the in-kernel generator instead of a tensor -- no noise stages.
template <int MODE_, int BX_, int STAGES_, int CWG_ = 1, bool GEN_ = false>
struct SweepCfg {
  static constexpr int MODE = MODE_, BX = BX_, STAGES = STAGES_, CWG = CWG_;
  static constexpr int D = 128, BM = 128;
  static constexpr bool GEN = GEN_;
  static_assert(!GEN || MODE != SWEEP_COLSUM, "only the KeyFormer sweeps use noise");
  static constexpr bool NOISE = MODE != SWEEP_COLSUM && !GEN;   // noise TENSOR streamed through the auxiliary ring
  static constexpr bool LSE_IN = MODE != SWEEP_KF_ROWLSE;
  // BX = 64: the stationary tile lives in TMEM (64 columns beside the two 64-column product tiles) and is the
  // A operand of the MMAs, which then read only the streamed operand from shared memory -- with both operands
  // in shared memory the M128 x N64 MMAs ask for 192 B/clk of a 128 B/clk port, and every shared-memory access
  // of the compute warps (noise, normalisers, barrier probes) queues behind them.
  static constexpr bool A_TMEM = BX == 64;
  static constexpr int A_BYTES = A_TMEM ? 0 : BM * D * 2;
  static constexpr int A_COL = 2 * BX;                                  // first TMEM column of the stationary tile
  static constexpr int X_STAGE_BYTES = BX * D * 2;
  static constexpr int NOISE_BYTES = NOISE ? BM * BX * 4 : 0;
  static constexpr int LSE_BYTES = LSE_IN ? BX * 4 : 0;
  static constexpr int N_STAGE_BYTES = NOISE_BYTES + LSE_BYTES;       // auxiliary ring read by the compute warps
  static constexpr int N_STAGE_STRIDE = (N_STAGE_BYTES + 1023) / 1024 * 1024;
  static constexpr int TMEM_COLS = A_TMEM ? 256 : 2 * BX;               // two product tiles (+ the stationary tile)
  static constexpr int COMPUTE_WARPS = 4 * CWG;
  static constexpr int THREADS = (COMPUTE_WARPS + 2) * 32;   // + TMA producer warp + MMA issuer warp
  // launch bound (registers): two CTAs share an SM -- the 320-thread column-sum CTAs and the KeyFormer CTAs
  static constexpr int CTAS_PER_SM = (CWG == 2 || MODE != SWEEP_COLSUM) ? 2 : 1;
  static_assert(CWG == 1 || CWG == 2, "one or two compute warpgroups");
  static_assert(BX / 32 % CWG == 0, "every compute warpgroup takes whole 32-column chunks");
  static constexpr int BAR_A_FULL = 0;
  static constexpr int BAR_X_FULL = 1;
  static constexpr int BAR_X_EMPTY = BAR_X_FULL + STAGES;
  static constexpr int BAR_N_FULL = BAR_X_EMPTY + STAGES;
  static constexpr int BAR_N_EMPTY = BAR_N_FULL + STAGES;
  static constexpr int BAR_T_FULL = BAR_N_EMPTY + STAGES;   // [2]
  static constexpr int BAR_T_EMPTY = BAR_T_FULL + 2;        // [2]
  static constexpr int BAR_DRAIN = BAR_T_EMPTY + 2;
  static constexpr int BAR_COMBINE = BAR_DRAIN + 1;         // second compute warpgroup's sums are in shared memory
  static constexpr int NUM_BARS = BAR_COMBINE + 1;
  static constexpr int COMBINE_BYTES = CWG == 2 ? 2 * 128 * 4 : 0;   // second warpgroup's partial sums
  static constexpr int SMEM_BYTES = A_BYTES + STAGES * X_STAGE_BYTES + STAGES * N_STAGE_STRIDE + COMBINE_BYTES +
                                    NUM_BARS * 8 + 16 + 1024;
};

template <class Cfg>
struct SweepCtx {
  uint8_t* sA;
  uint8_t* sX;
  uint8_t* sN;
  float* sCombine;   // [2][128], two compute warpgroups only
  uint64_t* bars;
  volatile int* abort_flag;
  uint32_t tmem_base;
  int a0;      // first stationary row (key index for the column sums, query index for the row LSE)
  int bh, b, h;
  int blk_lo, blk_hi;   // streamed blocks [blk_lo, blk_hi)
};

// ------------------------------- TMA producer -------------------------------
// GROUPED (column sums of the group-mean probabilities): the CTA belongs to one K/V head and streams, for every
// query block, the blocks of the `kv_group` query heads that share it, one after the other (item n = block
// n / kv_group of query head c.h * kv_group + n % kv_group).
template <class Cfg, bool GROUPED>
__device__ __forceinline__ void sweep_producer(const SweepCtx<Cfg>& c, const SweepParams& p, const CUtensorMap* tm_a,
                                               const CUtensorMap* tm_x, const CUtensorMap* tm_n) {
  constexpr int ST = Cfg::STAGES, BX = Cfg::BX;
  static_assert(!GROUPED || (Cfg::A_TMEM && !Cfg::NOISE), "grouped sweep: stationary tile in TMEM, no noise");
  if constexpr (!Cfg::A_TMEM) {
    mbar_expect_tx(&c.bars[Cfg::BAR_A_FULL], Cfg::A_BYTES);
#pragma unroll
    for (int ks = 0; ks < 2; ++ks)
      tma_load_4d(c.sA + ks * (Cfg::BM * 128), tm_a, &c.bars[Cfg::BAR_A_FULL], ks * 64,
                  Cfg::MODE == SWEEP_KF_ROWLSE ? c.h : c.h / p.kv_group, c.a0, c.b);
  }
  bool ok = true;
  int n_issued = 0;
  const int group = GROUPED ? p.kv_group : 1;
  const int n_items = (c.blk_hi - c.blk_lo) * group;
  for (int n = 0; n < n_items; ++n) {
    const int blk = c.blk_lo + (GROUPED ? n / group : n);
    const int st = n % ST, use = n / ST;
    // head of the streamed operand, and the row of the normaliser table that goes with it
    const int x_head = GROUPED ? c.h * group + (n - (blk - c.blk_lo) * group)
                               : (Cfg::MODE == SWEEP_KF_ROWLSE ? c.h / p.kv_group : c.h);
    const int lse_row = GROUPED ? c.b * p.heads + x_head : c.bh;
    if (use > 0 && !mbar_wait(&c.bars[Cfg::BAR_X_EMPTY + st], (use - 1) & 1, c.abort_flag, WAIT_X_EMPTY)) {
      ok = false;
      break;
    }
    mbar_expect_tx(&c.bars[Cfg::BAR_X_FULL + st], Cfg::X_STAGE_BYTES);
#pragma unroll
    for (int ks = 0; ks < 2; ++ks)
      tma_load_4d(c.sX + st * Cfg::X_STAGE_BYTES + ks * (BX * 128), tm_x, &c.bars[Cfg::BAR_X_FULL + st], ks * 64,
                  x_head, blk * BX, c.b);
    if constexpr (Cfg::N_STAGE_BYTES > 0) {
      if (use > 0 && !mbar_wait(&c.bars[Cfg::BAR_N_EMPTY + st], (use - 1) & 1, c.abort_flag, WAIT_N_EMPTY)) {
        ok = false;
        n_issued = n;  // X(n) issued, N(n) not
        break;
      }
      uint8_t* dst = c.sN + st * Cfg::N_STAGE_STRIDE;
      mbar_expect_tx(&c.bars[Cfg::BAR_N_FULL + st], Cfg::N_STAGE_BYTES);
      if constexpr (Cfg::NOISE) {
        // exp_rand viewed as a [B*H*q_len, kv_len] fp32 matrix; panels of 32 columns
        if constexpr (Cfg::MODE == SWEEP_KF_COLSUM) {
          // rows = queries of the streamed block, columns = the 128 stationary keys
#pragma unroll
          for (int pn = 0; pn < 4; ++pn)
            tma_load_2d(dst + pn * (BX * 128), tm_n, &c.bars[Cfg::BAR_N_FULL + st], c.a0 + pn * 32,
                        c.bh * p.q_len + blk * BX);
        } else {
          // rows = the 128 stationary queries, columns = keys of the streamed block
#pragma unroll
          for (int pn = 0; pn < BX / 32; ++pn)
            tma_load_2d(dst + pn * (128 * 128), tm_n, &c.bars[Cfg::BAR_N_FULL + st], blk * BX + pn * 32,
                        c.bh * p.q_len + c.a0);
        }
      }
      if constexpr (Cfg::LSE_IN) {
        // 1-D bulk copy of the BX row normalisers of this query block (lse rows are padded to 128)
        const float* src = p.lse + (int64_t)lse_row * p.lse_stride + blk * BX;
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
            ::"r"(smem_u32(dst + Cfg::NOISE_BYTES)), "l"(src), "r"((uint32_t)Cfg::LSE_BYTES),
              "r"(smem_u32(&c.bars[Cfg::BAR_N_FULL + st]))
            : "memory");
      }
    }
    n_issued = n + 1;
  }
  if (!ok || *c.abort_flag != 0) {
    // abort path: let our own bulk copies land before the CTA exits (bounded, 20 ms)
    const uint64_t t0 = global_timer_ns();
    while (!mbar_try_wait(&c.bars[Cfg::BAR_A_FULL], 0) && global_timer_ns() - t0 < 20000000ull) {
    }
    for (int st = 0; st < ST; ++st) {
      const int u = (n_issued - 1 - st) >= 0 ? (n_issued - 1 - st) / ST : -1;
      while (u >= 0 && !mbar_try_wait(&c.bars[Cfg::BAR_X_FULL + st], u & 1) && global_timer_ns() - t0 < 20000000ull) {
      }
      if constexpr (Cfg::N_STAGE_BYTES > 0) {
        while (u >= 0 && !mbar_try_wait(&c.bars[Cfg::BAR_N_FULL + st], u & 1) &&
               global_timer_ns() - t0 < 20000000ull) {
        }
      }
    }
  }
}

// -------------------------------- MMA issuer --------------------------------
// All 32 lanes walk the loop (warp-uniform control flow keeps the descriptor arithmetic on the uniform
// datapath); one elected lane issues.
template <class Cfg, bool BF16>
__device__ __forceinline__ void sweep_mma(const SweepCtx<Cfg>& c, int n_items) {
  constexpr int ST = Cfg::STAGES, BX = Cfg::BX;
  constexpr uint32_t IDESC = make_idesc(BF16, 128, BX, false, false);
  const uint32_t desc_hi = smem_desc_hi(1024);
  const uint32_t a_lo = smem_desc_lo(smem_u32(c.sA), 16), x_lo = smem_desc_lo(smem_u32(c.sX), 16);
  bool ok = mbar_wait(&c.bars[Cfg::BAR_A_FULL], 0, c.abort_flag, WAIT_Q_FULL);
  for (int n = 0; n < n_items && ok; ++n) {
    const int st = n % ST, tb = n & 1, tuse = n >> 1;
    if (tuse > 0) ok = mbar_wait(&c.bars[Cfg::BAR_T_EMPTY + tb], (tuse - 1) & 1, c.abort_flag, WAIT_T_EMPTY);
    ok = ok && mbar_wait(&c.bars[Cfg::BAR_X_FULL + st], (n / ST) & 1, c.abort_flag, WAIT_X_FULL);
    if (!ok) break;
    tc_fence_after();
    if (elect_one()) {
      const uint32_t b0 = x_lo + (uint32_t)(st * (Cfg::X_STAGE_BYTES >> 4));
      const uint32_t d_tmem = c.tmem_base + tb * BX;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t a_off = (uint32_t)(((kk / 4) * (128 * 128) + (kk % 4) * 32) >> 4);
        const uint32_t b_off = (uint32_t)(((kk / 4) * (BX * 128) + (kk % 4) * 32) >> 4);
        if constexpr (Cfg::A_TMEM) {
          // stationary tile in TMEM: 16 dims (one K step) = 8 columns of packed 16-bit pairs
          const uint32_t a_tmem = c.tmem_base + Cfg::A_COL + kk * 8;
          if (kk == 0)
            umma_ts_c<IDESC, 0>(d_tmem, a_tmem, b0 + b_off, desc_hi);
          else
            umma_ts_c<IDESC, 1>(d_tmem, a_tmem, b0 + b_off, desc_hi);
        } else {
          if (kk == 0)
            umma_ss_c<IDESC, 0>(d_tmem, a_lo + a_off, b0 + b_off, desc_hi);
          else
            umma_ss_c<IDESC, 1>(d_tmem, a_lo + a_off, b0 + b_off, desc_hi);
        }
      }
      umma_commit(&c.bars[Cfg::BAR_T_FULL + tb]);
      umma_commit(&c.bars[Cfg::BAR_X_EMPTY + st]);
    }
    __syncwarp();
  }
  if (elect_one()) umma_commit(&c.bars[Cfg::BAR_DRAIN]);
  __syncwarp();
  mbar_wait(&c.bars[Cfg::BAR_DRAIN], 0, c.abort_flag, WAIT_DRAIN);
}

// ------------------------- compute: per-key column sums -----------------------
template <class Cfg, bool SOFTCAP, int AUX>
__device__ __forceinline__ void sweep_compute_colsum(const SweepCtx<Cfg>& c, const SweepParams& p, int chunk) {
  constexpr int ST = Cfg::STAGES, BX = Cfg::BX;
  constexpr bool KF = Cfg::MODE == SWEEP_KF_COLSUM;
  const int warp_q = (threadIdx.x >> 5) & 3, lane = threadIdx.x & 31;
  const int key = c.a0 + warp_q * 32 + lane;
  const uint32_t lane_addr = c.tmem_base + ((uint32_t)(warp_q * 32) << 16);
  const float cmul = SOFTCAP ? 1.0f : p.scale_log2;
  // queries visible to this key: [i_lo, i_hi]
  int i_lo = p.causal ? key - p.delta : 0;
  int i_hi = (p.causal && p.window > 0) ? min(p.q_len - 1, key + p.window - 1 - p.delta) : p.q_len - 1;
  if (key >= p.kv_len) {
    i_lo = 1 << 28;
    i_hi = -1;
  }

  float2 acc2 = make_float2(0.f, 0.f), sq2 = make_float2(0.f, 0.f);
  // One 32-column chunk of the tile: p = exp2(x - L_i) for the thread's key against 32 queries.
  // cap_tag (soft-cap only): no lane of the warp holds |raw / cap| > 1 in this chunk -> polynomial branch alone
  auto chunk_body = [&](auto mask_tag, auto cap_tag, const uint32_t (&sr)[32], int ch, const float* lse_s,
                        const float* noise_col, int lo_c, int hi_c, float qbase, int i0) {
    constexpr bool MASK = decltype(mask_tag)::value;
    [[maybe_unused]] constexpr bool cap_poly_only = decltype(cap_tag)::value;
    const float2 c2 = make_float2(cmul, cmul);
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      const float4 L = *reinterpret_cast<const float4*>(lse_s + ch * 32 + i);
      float sv[4] = {__uint_as_float(sr[i]), __uint_as_float(sr[i + 1]), __uint_as_float(sr[i + 2]),
                     __uint_as_float(sr[i + 3])};
      if constexpr (SOFTCAP) softcap4(sv, p.cap_in, p.cap_out, cap_poly_only);
      float2 e0, e1;
      if constexpr (KF) {
        const float2 it2 = make_float2(p.inv_tau, p.inv_tau);
        float g[4];
        if constexpr (Cfg::GEN) {
          // One generator call yields the noise of ONE query against four consecutive keys, while this thread needs
          // one key against four consecutive queries: the four lanes of a quad (keys 4k .. 4k+3) each generate one of
          // the four queries and exchange the words (lane c sends word c ^ s to lane c ^ s in round s).
          const uint32_t cpos = lane & 3;
          uint32_t o[4] = {(uint32_t)key >> 2, (uint32_t)(i0 + ch * 32 + i) + cpos, (uint32_t)c.bh, 0u};
          philox4x32_10(o, p.seed_lo, p.seed_hi);
          xor_permute4(o, cpos);
          uint32_t r[4];
#pragma unroll
          for (int sft = 0; sft < 4; ++sft) r[sft] = __shfl_sync(0xffffffffu, o[sft], (lane & ~3) | (int)(cpos ^ sft));
          xor_permute4(r, cpos);
#pragma unroll
          for (int u = 0; u < 4; ++u) g[u] = -kf_gen_log2_exp_rand(r[u]);
        } else {
#pragma unroll
          for (int u = 0; u < 4; ++u) g[u] = -lg2_approx(noise_col[(ch * 32 + i + u) * 32]);
        }
        e0 = ffma2(ffma2(make_float2(sv[0], sv[1]), c2, make_float2(g[0], g[1])), it2, make_float2(-L.x, -L.y));
        e1 = ffma2(ffma2(make_float2(sv[2], sv[3]), c2, make_float2(g[2], g[3])), it2, make_float2(-L.z, -L.w));
      } else {
        e0 = ffma2(make_float2(sv[0], sv[1]), c2, make_float2(-L.x, -L.y));
        e1 = ffma2(make_float2(sv[2], sv[3]), c2, make_float2(-L.z, -L.w));
      }
      float pr[4];
      // A fixed, interleaved subset of the column groups of unmasked blocks takes its exponentials from the cubic
      // polynomial on the FMA pipe (exp2_poly2, relative error 7.5e-5): the sweep issues one exponential per
      // element and nothing else of weight, so the special-function unit (16 results per clock per SM) is its
      // bound; the share is kSweepPolyOf8 / 8.
      if (!MASK && (((i / 4) * kSweepPolyOf8) % 8) < kSweepPolyOf8) {
        e0 = exp2_poly2(e0);
        e1 = exp2_poly2(e1);
        pr[0] = e0.x, pr[1] = e0.y, pr[2] = e1.x, pr[3] = e1.y;
      } else {
        pr[0] = ex2_approx(e0.x), pr[1] = ex2_approx(e0.y), pr[2] = ex2_approx(e1.x), pr[3] = ex2_approx(e1.y);
      }
      if constexpr (MASK) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int col = ch * 32 + i + u;
          if (col < lo_c || col > hi_c) pr[u] = 0.f;
        }
      }
      const float2 p0 = make_float2(pr[0], pr[1]), p1 = make_float2(pr[2], pr[3]);
      acc2 = fadd2(acc2, fadd2(p0, p1));
      if constexpr (AUX == AUX_SQUARES) sq2 = ffma2(p1, p1, ffma2(p0, p0, sq2));
      if constexpr (AUX == AUX_CORM) {
        // Corm: does any query see this key with probability >= 1 / (i + 1)?  (kernels/corm.py:35-37,47-49;
        // tested as p * (i + 1) >= 1, the flag kept as 0/1 in the second accumulator)
        const float q1 = qbase + (float)(ch * 32 + i);
        sq2.x = fmaxf(sq2.x, fmaxf(pr[0] * q1 >= 1.0f ? 1.0f : 0.0f, pr[2] * (q1 + 2.0f) >= 1.0f ? 1.0f : 0.0f));
        sq2.y = fmaxf(sq2.y, fmaxf(pr[1] * (q1 + 1.0f) >= 1.0f ? 1.0f : 0.0f, pr[3] * (q1 + 3.0f) >= 1.0f ? 1.0f : 0.0f));
      }
    }
  };

  for (int blk = c.blk_lo; blk < c.blk_hi; ++blk) {
    const int n = blk - c.blk_lo, st = n % ST, tb = n & 1;
    [[maybe_unused]] const bool tl_on = threadIdx.x == 0;
    [[maybe_unused]] const int tl_base = (n & 63) * 8;
    if (tl_on) B200_TL(tl_base + 0);
    if (!mbar_wait(&c.bars[Cfg::BAR_T_FULL + tb], (n >> 1) & 1, c.abort_flag, WAIT_T_FULL)) return;
    if (tl_on) B200_TL(tl_base + 1);
    if (!mbar_wait(&c.bars[Cfg::BAR_N_FULL + st], (n / ST) & 1, c.abort_flag, WAIT_N_FULL)) return;
    tc_fence_after();
    if (tl_on) B200_TL(tl_base + 2);
    const uint8_t* nst = c.sN + st * Cfg::N_STAGE_STRIDE;
    const float* lse_s = reinterpret_cast<const float*>(nst + Cfg::NOISE_BYTES);
    const float* noise_col = reinterpret_cast<const float*>(nst + warp_q * (BX * 128)) + lane;  // + i * 32
    const int i0 = blk * BX;
    const int lo_c = i_lo - i0, hi_c = i_hi - i0;
    // does any (key, query) pair of this block need masking?
    const bool need_mask = (p.causal && (c.a0 + 127 - p.delta > i0)) || (i0 + BX > p.q_len) ||
                           (c.a0 + 128 > p.kv_len) ||
                           (p.causal && p.window > 0 && (c.a0 + p.window - 1 - p.delta < i0 + BX - 1));
    // the TMEM load of chunk ch+1 is in flight while chunk ch is being reduced; with two compute warpgroups
    // each takes its own half of the tile's columns
    constexpr int NCH = BX / 32 / Cfg::CWG;
    const int ch0 = Cfg::CWG == 2 ? (int)(threadIdx.x >> 7) * NCH : 0;
    uint32_t sr[2][32];
    tmem_ld32(lane_addr + tb * BX + ch0 * 32, sr[0]);
#pragma unroll
    for (int cc = 0; cc < NCH; ++cc) {
      const int ch = ch0 + cc;
      tmem_ld_wait();
      if (cc + 1 < NCH) tmem_ld32(lane_addr + tb * BX + (ch + 1) * 32, sr[(cc + 1) & 1]);
      auto run_chunk = [&](auto cap_tag) {
        if (need_mask)
          chunk_body(std::true_type{}, cap_tag, sr[cc & 1], ch, lse_s, noise_col, lo_c, hi_c, (float)(i0 + 1), i0);
        else
          chunk_body(std::false_type{}, cap_tag, sr[cc & 1], ch, lse_s, noise_col, lo_c, hi_c, (float)(i0 + 1), i0);
      };
      if constexpr (SOFTCAP) {
        if (softcap_chunk_poly_only(sr[cc & 1], p.cap_in))
          run_chunk(std::true_type{});
        else
          run_chunk(std::false_type{});
      } else {
        run_chunk(std::false_type{});
      }
      if (tl_on && cc < 4) B200_TL(tl_base + 3 + cc);
    }
    // this TMEM buffer and this auxiliary stage may be refilled
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(&c.bars[Cfg::BAR_T_EMPTY + tb]);
      mbar_arrive(&c.bars[Cfg::BAR_N_EMPTY + st]);
    }
    if (tl_on) B200_TL(tl_base + 7);
  }
  float acc = acc2.x + acc2.y;
  float aux = AUX == AUX_CORM ? fmaxf(sq2.x, sq2.y) : sq2.x + sq2.y;
  if constexpr (Cfg::CWG == 2) {
    // the second warpgroup hands its sums over through shared memory; the first adds them in a fixed order
    const int r = threadIdx.x & 127;
    if (threadIdx.x >= 128) {
      c.sCombine[r] = acc;
      c.sCombine[128 + r] = aux;
      __syncwarp();
      if (lane == 0) mbar_arrive(&c.bars[Cfg::BAR_COMBINE]);   // count 4: one arrival per warp of the second group
      return;
    }
    if (!mbar_wait(&c.bars[Cfg::BAR_COMBINE], 0, c.abort_flag, WAIT_T_FULL)) return;
    acc += c.sCombine[r];
    aux = AUX == AUX_CORM ? fmaxf(aux, c.sCombine[128 + r]) : aux + c.sCombine[128 + r];
  }
  const int64_t off = ((int64_t)c.bh * p.n_chunks + chunk) * p.kv_pad + key;
  p.partial[off] = acc;
  if constexpr (AUX != AUX_NONE) p.partial_sq[off] = aux;
}


// ------------- compute: per-key sums of the GROUP-MEAN probabilities ----------
// Grouped-query attention: the statistics are taken from pm_ij = (1 / g) sum_h p^h_ij, the probabilities averaged
// over the g query heads that share the K/V head (kernels/roco.py:39-40: mean over the group, THEN the square;
// figure/membound/attn.py:84-88, 240-242).  The g product tiles of one query block arrive one after the other;
// the thread of key j keeps the running sums over the heads for the block's 64 queries in registers and folds
// them into its accumulators after the last head of the group.
template <class Cfg, bool SOFTCAP, int AUX>
__device__ __forceinline__ void sweep_compute_colsum_grouped(const SweepCtx<Cfg>& c, const SweepParams& p, int chunk) {
  constexpr int ST = Cfg::STAGES, BX = Cfg::BX;
  static_assert(BX == 64, "the grouped sweep keeps one 64-query block of running sums in registers");
  const int warp_q = (threadIdx.x >> 5) & 3, lane = threadIdx.x & 31;
  const int key = c.a0 + warp_q * 32 + lane;
  const uint32_t lane_addr = c.tmem_base + ((uint32_t)(warp_q * 32) << 16);
  const float cmul = SOFTCAP ? 1.0f : p.scale_log2;
  int i_lo = p.causal ? key - p.delta : 0;
  int i_hi = (p.causal && p.window > 0) ? min(p.q_len - 1, key + p.window - 1 - p.delta) : p.q_len - 1;
  if (key >= p.kv_len) {
    i_lo = 1 << 28;
    i_hi = -1;
  }
  const int group = p.kv_group;
  const float inv_g = 1.0f / (float)group;
  const int n_items = (c.blk_hi - c.blk_lo) * group;
  float acc = 0.f, aux = 0.f;
  float pbar[BX];
#pragma unroll
  for (int i = 0; i < BX; ++i) pbar[i] = 0.f;
  int blk = c.blk_lo, hh = 0;
  for (int n = 0; n < n_items; ++n) {
    const int st = n % ST, tb = n & 1;
    if (!mbar_wait(&c.bars[Cfg::BAR_T_FULL + tb], (n >> 1) & 1, c.abort_flag, WAIT_T_FULL)) return;
    if (!mbar_wait(&c.bars[Cfg::BAR_N_FULL + st], (n / ST) & 1, c.abort_flag, WAIT_N_FULL)) return;
    tc_fence_after();
    const float* lse_s = reinterpret_cast<const float*>(c.sN + st * Cfg::N_STAGE_STRIDE + Cfg::NOISE_BYTES);
    const int i0 = blk * BX;
    const int lo_c = i_lo - i0, hi_c = i_hi - i0;
    const float keep = hh == 0 ? 0.f : 1.f;   // the first head of a group starts the running sums afresh
#pragma unroll
    for (int ch = 0; ch < BX / 32; ++ch) {
      uint32_t sr[32];
      tmem_ld32(lane_addr + tb * BX + ch * 32, sr);
      tmem_ld_wait();
      [[maybe_unused]] const bool cap_poly_only = SOFTCAP && softcap_chunk_poly_only(sr, p.cap_in);
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        const float4 L = *reinterpret_cast<const float4*>(lse_s + ch * 32 + i);
        float sv[4] = {__uint_as_float(sr[i]), __uint_as_float(sr[i + 1]), __uint_as_float(sr[i + 2]),
                       __uint_as_float(sr[i + 3])};
        if constexpr (SOFTCAP) softcap4(sv, p.cap_in, p.cap_out, cap_poly_only);
        const float2 c2 = make_float2(cmul, cmul);
        const float2 e0 = ffma2(make_float2(sv[0], sv[1]), c2, make_float2(-L.x, -L.y));
        const float2 e1 = ffma2(make_float2(sv[2], sv[3]), c2, make_float2(-L.z, -L.w));
        float pr[4] = {ex2_approx(e0.x), ex2_approx(e0.y), ex2_approx(e1.x), ex2_approx(e1.y)};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int col = ch * 32 + i + u;
          if (col < lo_c || col > hi_c) pr[u] = 0.f;   // masked pair, or a row / column beyond the tensors
          pbar[col] = fmaf(pbar[col], keep, pr[u]);
        }
      }
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(&c.bars[Cfg::BAR_T_EMPTY + tb]);
      mbar_arrive(&c.bars[Cfg::BAR_N_EMPTY + st]);
    }
    if (hh == group - 1) {
      const float q1 = (float)(i0 + 1);
#pragma unroll
      for (int col = 0; col < BX; ++col) {
        const float pm = pbar[col] * inv_g;
        acc += pm;
        if constexpr (AUX == AUX_SQUARES) aux = fmaf(pm, pm, aux);
        if constexpr (AUX == AUX_CORM) aux = fmaxf(aux, pm * (q1 + (float)col) >= 1.0f ? 1.0f : 0.0f);
      }
      hh = 0;
      ++blk;
    } else {
      ++hh;
    }
  }
  const int64_t off = ((int64_t)c.bh * p.n_chunks + chunk) * p.kv_pad + key;
  p.partial[off] = acc;
  if constexpr (AUX != AUX_NONE) p.partial_sq[off] = aux;
}

// --------------------- compute: per-query log-sum-exp of z --------------------
template <class Cfg>
__device__ __forceinline__ void sweep_compute_rowlse(const SweepCtx<Cfg>& c, const SweepParams& p) {
  constexpr int ST = Cfg::STAGES, BX = Cfg::BX;
  const int warp_q = (threadIdx.x >> 5) & 3, lane = threadIdx.x & 31;
  const int r_local = warp_q * 32 + lane;
  const int row = c.a0 + r_local;
  const uint32_t lane_addr = c.tmem_base + ((uint32_t)(warp_q * 32) << 16);
  const float cz = p.scale_log2 * p.inv_tau;
  float m = -1.0e30f, l = 0.f;
  const int hi_key = p.causal ? min(row + p.delta, p.kv_len - 1) : p.kv_len - 1;
  // with two compute warpgroups each takes half of the block's key columns: a row's running (maximum, sum) is then
  // split over two threads and merged once at the end
  constexpr int NCH = BX / 32 / Cfg::CWG;
  const int ch0 = Cfg::CWG == 2 ? (int)(threadIdx.x >> 7) * NCH : 0;

  for (int blk = c.blk_lo; blk < c.blk_hi; ++blk) {
    const int n = blk - c.blk_lo, st = n % ST, tb = n & 1;
    if (!mbar_wait(&c.bars[Cfg::BAR_T_FULL + tb], (n >> 1) & 1, c.abort_flag, WAIT_T_FULL)) return;
    if constexpr (Cfg::N_STAGE_BYTES > 0)
      if (!mbar_wait(&c.bars[Cfg::BAR_N_FULL + st], (n / ST) & 1, c.abort_flag, WAIT_N_FULL)) return;
    tc_fence_after();
    [[maybe_unused]] const uint8_t* nst = c.sN + st * Cfg::N_STAGE_STRIDE;
    const int hi_c = hi_key - blk * BX;
    float z[NCH * 32];
    float mx = -INFINITY;
#pragma unroll
    for (int cc = 0; cc < NCH; ++cc) {
      const int ch = ch0 + cc;
      uint32_t sr[32];
      tmem_ld32(lane_addr + tb * BX + ch * 32, sr);
      tmem_ld_wait();
      [[maybe_unused]] const uint8_t* panel = nst + ch * (128 * 128) + r_local * 128;
#pragma unroll
      for (int q4 = 0; q4 < 8; ++q4) {
        float lg[4];   // log2(exp_rand) of this query against four consecutive keys
        if constexpr (Cfg::GEN) {
          uint32_t o[4] = {(uint32_t)(blk * BX + ch * 32 + q4 * 4) >> 2, (uint32_t)row, (uint32_t)c.bh, 0u};
          philox4x32_10(o, p.seed_lo, p.seed_hi);
#pragma unroll
          for (int u = 0; u < 4; ++u) lg[u] = kf_gen_log2_exp_rand(o[u]);
        } else {
          // 128-byte swizzle written by TMA: 16-byte chunk q4 of row r sits at chunk (q4 ^ (r & 7))
          const float4 er = *reinterpret_cast<const float4*>(panel + ((q4 ^ (r_local & 7)) << 4));
          lg[0] = lg2_approx(er.x), lg[1] = lg2_approx(er.y), lg[2] = lg2_approx(er.z), lg[3] = lg2_approx(er.w);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int col = ch * 32 + q4 * 4 + u;
          float v = fmaf(__uint_as_float(sr[q4 * 4 + u]), cz, -lg[u] * p.inv_tau);
          if (col > hi_c) v = -INFINITY;
          z[cc * 32 + q4 * 4 + u] = v;
          mx = fmaxf(mx, v);
        }
      }
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(&c.bars[Cfg::BAR_T_EMPTY + tb]);
      if constexpr (Cfg::N_STAGE_BYTES > 0) mbar_arrive(&c.bars[Cfg::BAR_N_EMPTY + st]);
    }
    const float m_new = fmaxf(m, mx);
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int i = 0; i < NCH * 32; i += 2) {
      s0 += ex2_approx(z[i] - m_new);
      s1 += ex2_approx(z[i + 1] - m_new);
    }
    l = l * ex2_approx(m - m_new) + (s0 + s1);
    m = m_new;
  }
  if constexpr (Cfg::CWG == 2) {
    // merge the two halves of every row: (m, l) of the second warpgroup goes through shared memory
    if (threadIdx.x >= 128) {
      c.sCombine[r_local] = m;
      c.sCombine[128 + r_local] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(&c.bars[Cfg::BAR_COMBINE]);
      return;
    }
    if (!mbar_wait(&c.bars[Cfg::BAR_COMBINE], 0, c.abort_flag, WAIT_T_FULL)) return;
    const float m1 = c.sCombine[r_local], l1 = c.sCombine[128 + r_local];
    const float mm = fmaxf(m, m1);
    l = l * ex2_approx(m - mm) + l1 * ex2_approx(m1 - mm);
    m = mm;
  }
  if (row < p.q_len) p.lse_out[(int64_t)c.bh * p.lse_stride + row] = m + log2f(l);
}

// ----------------------------------- kernel ----------------------------------
// Grid: x = (batch, head) unit -- (batch, K/V head) when GROUPED --, y = rank of the stationary 128-row tile with the
// tile that meets the most streamed blocks first, z = chunk of streamed blocks.  Blocks are dispatched x-fastest,
// so the launch walks ALL units' heaviest tiles first and ends on the lightest ones (longest-processing-time-first
// over the whole launch, not per head): under a causal mask a tile's work ranges from one block to all of them.
template <int MODE, int BX, int STAGES, bool BF16, bool SOFTCAP, int AUX, bool GROUPED = false, int CWG = 1,
          bool GEN = false>
__global__ void __launch_bounds__((SweepCfg<MODE, BX, STAGES, CWG, GEN>::THREADS),
                                  (SweepCfg<MODE, BX, STAGES, CWG, GEN>::CTAS_PER_SM))
attn_sweep_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_x,
                  const __grid_constant__ CUtensorMap tm_n, const SweepParams p) {
  using Cfg = SweepCfg<MODE, BX, STAGES, CWG, GEN>;
  constexpr int CW = Cfg::COMPUTE_WARPS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  // A launch that follows an expired wait on this device drains immediately (the status word stays
  // set until the host reads it), so that one stuck kernel cannot stall a whole queue of launches.  The word is
  // loaded here and looked at after the set-up below, whose barrier it shares.
  __shared__ int s_skip;
  int status_now = 0;
  if (threadIdx.x == 0) status_now = *reinterpret_cast<volatile int*>(&g_device_status);

  B200_TL_INIT();
  [[maybe_unused]] const uint64_t cta_start_ns = global_timer_ns();
  [[maybe_unused]] const long long cta_start_clk = clock64();
  SweepCtx<Cfg> c;
  c.sA = smem;
  c.sX = c.sA + Cfg::A_BYTES;
  c.sN = c.sX + STAGES * Cfg::X_STAGE_BYTES;
  c.sCombine = reinterpret_cast<float*>(c.sN + STAGES * Cfg::N_STAGE_STRIDE);
  c.bars = reinterpret_cast<uint64_t*>(c.sN + STAGES * Cfg::N_STAGE_STRIDE + Cfg::COMBINE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(c.bars + Cfg::NUM_BARS);
  c.abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.z;
  // column sums: key tile 0 meets every query block under a causal mask; row sweep: the last query tile sees every key
  c.a0 = (MODE == SWEEP_KF_ROWLSE ? (int)(gridDim.y - 1 - blockIdx.y) : (int)blockIdx.y) * 128;
  c.bh = blockIdx.x;
  {
    const int unit_heads = GROUPED ? p.heads / p.kv_group : p.heads;   // GROUPED: one CTA per (batch, K/V head)
    c.b = c.bh / unit_heads;
    c.h = c.bh - c.b * unit_heads;
  }
  if constexpr (MODE == SWEEP_KF_ROWLSE) {
    const int r_last = min(c.a0 + 127, p.q_len - 1);
    c.blk_lo = 0;
    c.blk_hi = (p.causal ? min(p.kv_len - 1, r_last + p.delta) : p.kv_len - 1) / BX + 1;
  } else {
    const int i_first = p.causal ? max(0, c.a0 - p.delta) : 0;
    const int i_last = (p.causal && p.window > 0) ? min(p.q_len - 1, c.a0 + 127 + p.window - 1 - p.delta) : p.q_len - 1;
    const int lo = i_first / BX, hi = i_last / BX + 1;
    c.blk_lo = max(lo, chunk * p.chunk_blocks);
    c.blk_hi = min(hi, (chunk + 1) * p.chunk_blocks);
    if (c.blk_hi < c.blk_lo) c.blk_hi = c.blk_lo;
  }
  if (c.blk_hi == c.blk_lo) {
    // nothing visible in this chunk: its partial vector is all zeros
    if constexpr (MODE != SWEEP_KF_ROWLSE) {
      if (threadIdx.x < 128) {
        const int64_t off = ((int64_t)c.bh * p.n_chunks + chunk) * p.kv_pad + c.a0 + threadIdx.x;
        p.partial[off] = 0.f;
        if constexpr (AUX != AUX_NONE) p.partial_sq[off] = 0.f;
      }
    }
    return;
  }

  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < Cfg::NUM_BARS; ++i) {
      // arrivals per phase: every compute warp releases a product buffer / an auxiliary stage
      const bool warp_count = (i >= Cfg::BAR_N_EMPTY && i < Cfg::BAR_N_EMPTY + STAGES) ||
                              (i >= Cfg::BAR_T_EMPTY && i < Cfg::BAR_T_EMPTY + 2);
      const bool four = (Cfg::A_TMEM && i == Cfg::BAR_A_FULL) || i == Cfg::BAR_COMBINE;
      mbar_init(&c.bars[i], warp_count ? (uint32_t)Cfg::COMPUTE_WARPS : four ? 4u : 1u);
    }
    *c.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == CW && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_x);
    if constexpr (Cfg::NOISE) tma_prefetch_desc(&tm_n);
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
  if (s_skip != 0) {
    if (warp == 0) tmem_dealloc(c.tmem_base, Cfg::TMEM_COLS);
    return;
  }

  if (warp < CW) {
    if constexpr (Cfg::A_TMEM) if (warp < 4) {
      // thread r copies row r of the stationary tile (256 contiguous bytes) from global memory into TMEM lane r;
      // a 32-bit TMEM column holds two consecutive 16-bit elements, which is the order they have in memory
      const int row = c.a0 + (int)threadIdx.x;
      const int a_head = (GROUPED || MODE == SWEEP_KF_ROWLSE) ? c.h : c.h / p.kv_group;
      const uint4* src = reinterpret_cast<const uint4*>(
          p.a_base + (((int64_t)c.b * p.a_rows + row) * p.a_heads + a_head) * 128);
      const uint32_t dst = c.tmem_base + ((uint32_t)(warp * 32) << 16) + Cfg::A_COL;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t w[32];
#pragma unroll
        for (int v8 = 0; v8 < 8; ++v8) {
          const uint4 x = row < p.a_rows ? __ldg(src + half * 8 + v8) : make_uint4(0u, 0u, 0u, 0u);
          w[4 * v8] = x.x;
          w[4 * v8 + 1] = x.y;
          w[4 * v8 + 2] = x.z;
          w[4 * v8 + 3] = x.w;
        }
        tmem_st32(dst + half * 32, w);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&c.bars[Cfg::BAR_A_FULL]);
    }
    if constexpr (MODE == SWEEP_KF_ROWLSE)
      sweep_compute_rowlse<Cfg>(c, p);
    else if constexpr (GROUPED)
      sweep_compute_colsum_grouped<Cfg, SOFTCAP, AUX>(c, p, chunk);
    else
      sweep_compute_colsum<Cfg, SOFTCAP, AUX>(c, p, chunk);
  } else if (warp == CW) {
    if (lane == 0) sweep_producer<Cfg, GROUPED>(c, p, &tm_a, &tm_x, &tm_n);
  } else {
    sweep_mma<Cfg, BF16>(c, (c.blk_hi - c.blk_lo) * (GROUPED ? p.kv_group : 1));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(c.tmem_base, Cfg::TMEM_COLS);
  B200_TL_FLUSH();
  B200_TL_CTA(cta_start_ns, cta_start_clk, c.blk_hi - c.blk_lo);
}

// Adds the per-chunk partial vectors in chunk order: out[bh][j] = mul * sum_c partial[bh][c][j].
// Grouped-query scores: the partial vectors of the g query heads of one K/V head are adjacent, so the same loop
// over g * n_chunks rows with mul = 1/g yields the group mean of the column sums
// (kernels/roco.py:39-40 averages the probabilities over the group before summing over the queries).
__global__ void __launch_bounds__(256)
score_reduce_kernel(float* __restrict__ out, float* __restrict__ out_sq, const float* __restrict__ partial,
                    const float* __restrict__ partial_sq, int kv_len, int kv_pad, int n_chunks, float mul) {
  const int bh = blockIdx.y;
  const int j = blockIdx.x * 256 + threadIdx.x;
  if (j >= kv_len) return;
  const float* src = partial + (int64_t)bh * n_chunks * kv_pad + j;
  float a = 0.f;
  for (int cidx = 0; cidx < n_chunks; ++cidx) a += src[(int64_t)cidx * kv_pad];
  out[(int64_t)bh * kv_len + j] = mul == 1.0f ? a : a * mul;
  if (out_sq != nullptr) {
    const float* src2 = partial_sq + (int64_t)bh * n_chunks * kv_pad + j;
    float a2 = 0.f;
    for (int cidx = 0; cidx < n_chunks; ++cidx) a2 += src2[(int64_t)cidx * kv_pad];
    out_sq[(int64_t)bh * kv_len + j] = a2;
  }
}

// exp_rand[b, h, i, j] of the in-kernel generator, written out as the tensor the reference's KeyFormer module takes
// (kernels/kf.py:19): one thread per four consecutive keys.  The logarithm is taken in double precision, so the
// tensor is the correctly rounded -ln(u); the sweeps' own evaluation differs from it by < 5e-5 relative.
__global__ void __launch_bounds__(256)
kf_noise_fill_kernel(float* __restrict__ out, int64_t rows, int q_len, int kv_len, uint32_t seed_lo, uint32_t seed_hi) {
  const int64_t quads_per_row = (kv_len + 3) / 4;
  const int64_t total = rows * quads_per_row;
  for (int64_t g = (int64_t)blockIdx.x * 256 + threadIdx.x; g < total; g += (int64_t)gridDim.x * 256) {
    const int64_t row = g / quads_per_row;            // (b * heads + h) * q_len + i
    const uint32_t jq = (uint32_t)(g - row * quads_per_row);
    const int64_t bh = row / q_len;
    uint32_t o[4] = {jq, (uint32_t)(row - bh * q_len), (uint32_t)bh, 0u};
    philox4x32_10(o, seed_lo, seed_hi);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t j = (int64_t)jq * 4 + u;
      if (j < kv_len) out[row * kv_len + j] = (float)(-log(((double)(o[u] >> 9) + 0.5) * (1.0 / 8388608.0)));
    }
  }
}

// --------------------------------- host side ---------------------------------
// size of the library's built-in scratch for b200_attn_score_static (32 MiB per GPU that loads the library)
constexpr int64_t kStaticScoreScratchBytes = 32ll << 20;
int static_score_scratch(void** out);

#ifndef B200_SWEEP_CHUNK
#define B200_SWEEP_CHUNK 32
#endif
constexpr int kSweepChunkBlocks = B200_SWEEP_CHUNK;
#ifndef B200_COLSUM_BX
#define B200_COLSUM_BX 128
#endif
#ifndef B200_COLSUM_STAGES
#define B200_COLSUM_STAGES 2
#endif
// KeyFormer sweeps: two ring stages of 8 KB (streamed operand) + 32 KB (noise) keep a CTA at 83 KB of shared memory, so
// that two CTAs share an SM (measured at config 4: 430 -> 322 us against three stages and one CTA per SM)
#ifndef B200_KF_STAGES
#define B200_KF_STAGES 2
#endif
// compute warpgroups of the KeyFormer sweeps and of the plain column-sum sweep (see SweepCfg)
#ifndef B200_KF_CWG
#define B200_KF_CWG 2
#endif
#ifndef B200_COLSUM_CWG
#define B200_COLSUM_CWG (B200_COLSUM_BX == 128 ? 2 : 1)
#endif

struct ScoreWorkspace {
  int lse_stride, kv_pad, n_chunks_colsum, n_chunks_kf;
  int64_t lse_off, lse2_off, partial_off, partial_sq_off, total;
};

inline ScoreWorkspace score_workspace_layout(int batch, int q_len, int kv_len, int heads) {
  ScoreWorkspace w;
  const int64_t bh = (int64_t)batch * heads;
  w.lse_stride = (q_len + 127) / 128 * 128;
  w.kv_pad = (kv_len + 127) / 128 * 128;
  const int qblocks128 = (q_len + 127) / 128, qblocks64 = (q_len + 63) / 64;
  w.n_chunks_colsum = (qblocks128 + kSweepChunkBlocks - 1) / kSweepChunkBlocks;
  w.n_chunks_kf = (qblocks64 + kSweepChunkBlocks - 1) / kSweepChunkBlocks;
  const int n_chunks = std::max(w.n_chunks_colsum, w.n_chunks_kf);
  auto up = [](int64_t x) { return (x + 255) / 256 * 256; };
  w.lse_off = 0;
  w.lse2_off = up(bh * w.lse_stride * 4);
  w.partial_off = w.lse2_off + up(bh * w.lse_stride * 4);
  w.partial_sq_off = w.partial_off + up(bh * n_chunks * w.kv_pad * 4);
  w.total = w.partial_sq_off + up(bh * n_chunks * w.kv_pad * 4);
  return w;
}

inline int64_t score_workspace_bytes(int batch, int q_len, int kv_len, int heads) {
  if (batch <= 0 || q_len <= 0 || kv_len <= 0 || heads <= 0) return 0;
  return score_workspace_layout(batch, q_len, kv_len, heads).total;
}

// n_chunks chunks of streamed blocks x n_tiles stationary tiles x (batch x heads) units -- (batch x K/V heads) when GROUPED
template <int MODE, int BX, int STAGES, bool BF16, bool SOFTCAP, int AUX, bool GROUPED = false, int CWG = 1,
          bool GEN = false>
int launch_sweep(const CUtensorMap& ta, const CUtensorMap& tx, const CUtensorMap& tn, const SweepParams& p,
                 int n_chunks, int n_tiles, cudaStream_t stream) {
  using Cfg = SweepCfg<MODE, BX, STAGES, CWG, GEN>;
  auto kern = attn_sweep_kernel<MODE, BX, STAGES, BF16, SOFTCAP, AUX, GROUPED, CWG, GEN>;
  static thread_local int configured_dev = -1;
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    B200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    configured_dev = dev;
  }
  dim3 grid(p.batch * (GROUPED ? p.heads / p.kv_group : p.heads), n_tiles, n_chunks);
  kern<<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(ta, tx, tn, p);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

inline int score_common_checks(const void* q, const void* k, const void* v, void* out, void* workspace,
                               int64_t workspace_bytes, int batch, int q_len, int kv_len, int heads, int head_dim,
                               int dtype) {
  if (!q || !k || !v || !out) return B200_ERR_BAD_ARGUMENT;
  if (batch <= 0 || q_len <= 0 || kv_len <= 0 || heads <= 0) return B200_ERR_BAD_ARGUMENT;
  if (dtype != B200_F16 && dtype != B200_BF16) return B200_ERR_BAD_DTYPE;
  if (head_dim != 128) return B200_ERR_UNSUPPORTED;
  if (kv_len < q_len) return B200_ERR_UNSUPPORTED;
  if ((int64_t)batch * heads > 65535) return B200_ERR_UNSUPPORTED;
  if (!workspace || workspace_bytes < score_workspace_bytes(batch, q_len, kv_len, heads)) return B200_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return B200_ERR_MISALIGNED;
  return B200_OK;
}

// Flags of the Corm variant: out[bh][j] = (max over chunks of the 0/1 partial flags) != 0.
__global__ void __launch_bounds__(256)
corm_reduce_kernel(uint8_t* __restrict__ out, const float* __restrict__ partial_flag, int kv_len, int kv_pad,
                   int n_chunks) {
  const int bh = blockIdx.y;
  const int j = blockIdx.x * 256 + threadIdx.x;
  if (j >= kv_len) return;
  const float* src = partial_flag + (int64_t)bh * n_chunks * kv_pad + j;
  float a = 0.f;
  for (int cidx = 0; cidx < n_chunks; ++cidx) a = fmaxf(a, src[(int64_t)cidx * kv_pad]);
  out[(int64_t)bh * kv_len + j] = a != 0.f ? 1 : 0;
}

// out[r][j] = (1 / kernel) * sum_{d = -kernel/2 .. kernel/2} in[r][j + d], zero padded (SnapKV's pooling of
// the column sums: F.avg_pool1d(kernel_size, padding = kernel_size // 2, stride = 1), kernels/snapkv.py:36-38)
__global__ void __launch_bounds__(256)
avg_pool1d_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t rows, int len, int kernel) {
  const int64_t r = blockIdx.y;
  const int j = blockIdx.x * 256 + threadIdx.x;
  if (j >= len) return;
  const float* row = in + r * len;
  const int half = kernel / 2;
  float a = 0.f;
  for (int d = -half; d <= half; ++d) {
    const int jj = j + d;
    if (jj >= 0 && jj < len) a += row[jj];
  }
  out[r * len + j] = a / (float)kernel;
}

// corm_flags (optional): uint8 [B, H, Skv]; when given, the second statistic is the Corm flag and score_sq must be null.
inline int attn_score_impl(const void* q, const void* k, const void* v, void* out, float* score, float* score_sq,
                           void* workspace, int64_t workspace_bytes, int batch, int q_len, int kv_len, int heads,
                           int head_dim, int dtype, int causal, int window, float softcap, float scale,
                           cudaStream_t stream, uint8_t* corm_flags = nullptr, int kv_heads = 0) {
  if (kv_heads <= 0) kv_heads = heads;
  if (heads % kv_heads != 0) return B200_ERR_BAD_ARGUMENT;
  const int group = heads / kv_heads;
  int rc = score_common_checks(q, k, v, out, workspace, workspace_bytes, batch, q_len, kv_len, heads, head_dim, dtype);
  if (rc != B200_OK) return rc;
  if (!score) return B200_ERR_BAD_ARGUMENT;
  if (window > 0 && !causal) return B200_ERR_UNSUPPORTED;
  if (corm_flags != nullptr && (score_sq != nullptr || softcap > 0.f)) return B200_ERR_BAD_ARGUMENT;
  // The group mean commutes with the column sum (the ordered reduce adds the g heads' partial vectors), but not
  // with the square or with Corm's threshold test: those take the grouped sweep, which averages per (key, query).
  const bool grouped = group > 1 && (score_sq != nullptr || corm_flags != nullptr);
  const ScoreWorkspace w = score_workspace_layout(batch, q_len, kv_len, heads);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  float* lse = reinterpret_cast<float*>(ws + w.lse_off);

  rc = attn_fwd_impl_lse_stride(q, k, v, out, lse, w.lse_stride, batch, q_len, kv_len, heads, kv_heads, head_dim,
                                dtype, causal, window, softcap, scale, stream);
  if (rc != B200_OK) return rc;

  const bool bf16 = dtype == B200_BF16;
  CUtensorMap ta, tx, tn;
  if ((rc = make_bshd_tensor_map(&ta, k, batch, kv_len, kv_heads, head_dim, 128, bf16)) != B200_OK) return rc;
  if ((rc = make_bshd_tensor_map(&tx, q, batch, q_len, heads, head_dim, grouped ? 64 : B200_COLSUM_BX, bf16)) != B200_OK)
    return rc;
  tn = ta;  // unused

  SweepParams p;
  std::memset(&p, 0, sizeof(p));
  p.lse = lse;
  p.partial = reinterpret_cast<float*>(ws + w.partial_off);
  p.partial_sq = reinterpret_cast<float*>(ws + w.partial_sq_off);
  p.batch = batch;
  p.heads = heads;
  p.q_len = q_len;
  p.kv_len = kv_len;
  p.delta = kv_len - q_len;
  p.causal = causal ? 1 : 0;
  p.window = window > 0 ? window : 0;
  p.lse_stride = w.lse_stride;
  p.kv_pad = w.kv_pad;
  p.n_chunks = w.n_chunks_colsum;
  p.chunk_blocks = kSweepChunkBlocks * (128 / (grouped ? 64 : B200_COLSUM_BX));
  p.a_base = static_cast<const uint16_t*>(k);
  p.a_rows = kv_len;
  p.a_heads = kv_heads;
  p.kv_group = group;
  const float kLog2e = 1.4426950408889634f;
  p.scale_log2 = scale * kLog2e;
  p.cap_in = softcap > 0.f ? scale / softcap : 0.f;
  p.cap_out = softcap * kLog2e;
  p.inv_tau = 1.0f;
  const bool cap = softcap > 0.f, sq = score_sq != nullptr;
  const int gy = w.kv_pad / 128;
  if (gy > 65535 || p.n_chunks > 65535) return B200_ERR_UNSUPPORTED;

  if (grouped) {
    // one CTA per (batch, K/V head, key tile, chunk); 64-query blocks, stationary K tile in TMEM
#define B200_SWEEPG(BF, CAP, AUXV) \
  launch_sweep<SWEEP_COLSUM, 64, B200_KF_STAGES, BF, CAP, AUXV, true>(ta, tx, tn, p, p.n_chunks, gy, stream)
    if (corm_flags != nullptr)
      rc = bf16 ? B200_SWEEPG(true, false, AUX_CORM) : B200_SWEEPG(false, false, AUX_CORM);
    else if (bf16)
      rc = cap ? B200_SWEEPG(true, true, AUX_SQUARES) : B200_SWEEPG(true, false, AUX_SQUARES);
    else
      rc = cap ? B200_SWEEPG(false, true, AUX_SQUARES) : B200_SWEEPG(false, false, AUX_SQUARES);
#undef B200_SWEEPG
    if (rc != B200_OK) return rc;
    dim3 ggrid((kv_len + 255) / 256, batch * kv_heads);
    score_reduce_kernel<<<ggrid, 256, 0, stream>>>(score, score_sq, p.partial, p.partial_sq, kv_len, w.kv_pad,
                                                   p.n_chunks, 1.0f);
    B200_CUDA_TRY(cudaGetLastError());
    if (corm_flags != nullptr) {
      corm_reduce_kernel<<<ggrid, 256, 0, stream>>>(corm_flags, p.partial_sq, kv_len, w.kv_pad, p.n_chunks);
      B200_CUDA_TRY(cudaGetLastError());
    }
    return B200_OK;
  }

#define B200_SWEEP0(BF, CAP, AUXV)                                                                      \
  launch_sweep<SWEEP_COLSUM, B200_COLSUM_BX, B200_COLSUM_STAGES, BF, CAP, AUXV, false, B200_COLSUM_CWG>( \
      ta, tx, tn, p, p.n_chunks, gy, stream)
  if (corm_flags != nullptr)
    rc = bf16 ? B200_SWEEP0(true, false, AUX_CORM) : B200_SWEEP0(false, false, AUX_CORM);
  else if (bf16)
    rc = cap ? (sq ? B200_SWEEP0(true, true, AUX_SQUARES) : B200_SWEEP0(true, true, AUX_NONE))
             : (sq ? B200_SWEEP0(true, false, AUX_SQUARES) : B200_SWEEP0(true, false, AUX_NONE));
  else
    rc = cap ? (sq ? B200_SWEEP0(false, true, AUX_SQUARES) : B200_SWEEP0(false, true, AUX_NONE))
             : (sq ? B200_SWEEP0(false, false, AUX_SQUARES) : B200_SWEEP0(false, false, AUX_NONE));
#undef B200_SWEEP0
  if (rc != B200_OK) return rc;

  dim3 rgrid((kv_len + 255) / 256, batch * kv_heads);
  score_reduce_kernel<<<rgrid, 256, 0, stream>>>(score, score_sq, p.partial, p.partial_sq, kv_len, w.kv_pad,
                                                 p.n_chunks * group, 1.0f / (float)group);
  B200_CUDA_TRY(cudaGetLastError());
  if (corm_flags != nullptr) {
    corm_reduce_kernel<<<rgrid, 256, 0, stream>>>(corm_flags, p.partial_sq, kv_len, w.kv_pad, p.n_chunks);
    B200_CUDA_TRY(cudaGetLastError());
  }
  return B200_OK;
}

// kv_heads < heads (grouped-query attention): the second softmax is taken per query head against the K/V head it
// shares, and the score of a K/V head is the mean over its query heads (figure/membound/attn.py:162-165) -- the mean
// commutes with the sum over the queries, so the ordered reduce adds the g heads' partial vectors and scales by 1/g.
inline int attn_kf_impl(const void* q, const void* k, const void* v, const float* exp_rand, void* out,
                        float* kf_score, void* workspace, int64_t workspace_bytes, int batch, int q_len, int kv_len,
                        int heads, int head_dim, int dtype, int causal, float tau, float scale, cudaStream_t stream,
                        int kv_heads = 0, uint64_t seed = 0) {
  // exp_rand == nullptr: the noise is generated in the kernels from `seed` (see philox4x32_10 above)
  const bool gen = exp_rand == nullptr;
  if (kv_heads <= 0) kv_heads = heads;
  if (heads % kv_heads != 0) return B200_ERR_BAD_ARGUMENT;
  const int group = heads / kv_heads;
  int rc = score_common_checks(q, k, v, out, workspace, workspace_bytes, batch, q_len, kv_len, heads, head_dim, dtype);
  if (rc != B200_OK) return rc;
  if (!kf_score || !(tau > 0.f)) return B200_ERR_BAD_ARGUMENT;
  if (!gen && (kv_len % 4 != 0 || !aligned16(exp_rand))) return B200_ERR_MISALIGNED;
  if ((int64_t)batch * heads * q_len >= (1ll << 31)) return B200_ERR_UNSUPPORTED;
  const ScoreWorkspace w = score_workspace_layout(batch, q_len, kv_len, heads);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  float* lse2 = reinterpret_cast<float*>(ws + w.lse2_off);

  // attention output (its own LSE is not needed by the KeyFormer score)
  rc = attn_fwd_impl_lse_stride(q, k, v, out, nullptr, 0, batch, q_len, kv_len, heads, kv_heads, head_dim, dtype,
                                causal, 0, 0.f, scale, stream);
  if (rc != B200_OK) return rc;

  const bool bf16 = dtype == B200_BF16;
  CUtensorMap tq128, tk64, tk128, tq64, tn_rows128, tn_rows64;
  if ((rc = make_bshd_tensor_map(&tq128, q, batch, q_len, heads, head_dim, 128, bf16)) != B200_OK) return rc;
  if ((rc = make_bshd_tensor_map(&tq64, q, batch, q_len, heads, head_dim, 64, bf16)) != B200_OK) return rc;
  if ((rc = make_bshd_tensor_map(&tk128, k, batch, kv_len, kv_heads, head_dim, 128, bf16)) != B200_OK) return rc;
  if ((rc = make_bshd_tensor_map(&tk64, k, batch, kv_len, kv_heads, head_dim, 64, bf16)) != B200_OK) return rc;
  const int64_t rows = (int64_t)batch * heads * q_len;
  if (gen) {
    tn_rows128 = tq128;   // unused
    tn_rows64 = tq128;
  } else {
    if ((rc = make_f32_matrix_tensor_map(&tn_rows128, exp_rand, rows, kv_len, 128, 32, true)) != B200_OK) return rc;
    if ((rc = make_f32_matrix_tensor_map(&tn_rows64, exp_rand, rows, kv_len, 64, 32, false)) != B200_OK) return rc;
  }

  SweepParams p;
  std::memset(&p, 0, sizeof(p));
  p.lse = lse2;
  p.lse_out = lse2;
  p.partial = reinterpret_cast<float*>(ws + w.partial_off);
  p.partial_sq = nullptr;
  p.batch = batch;
  p.heads = heads;
  p.q_len = q_len;
  p.kv_len = kv_len;
  p.delta = kv_len - q_len;
  p.causal = causal ? 1 : 0;
  p.window = 0;
  p.lse_stride = w.lse_stride;
  p.kv_pad = w.kv_pad;
  p.n_chunks = w.n_chunks_kf;
  p.chunk_blocks = kSweepChunkBlocks;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.inv_tau = 1.0f / tau;
  p.kv_group = group;
  p.seed_lo = (uint32_t)seed;
  p.seed_hi = (uint32_t)(seed >> 32);

  // sweep 1: Lz_i = log2 sum_j exp2(z_ij), one CTA per 128 queries
  const int q_tiles = (q_len + 127) / 128;
  if (q_tiles > 65535 || w.kv_pad / 128 > 65535 || p.n_chunks > 65535) return B200_ERR_UNSUPPORTED;
  p.a_base = static_cast<const uint16_t*>(q);
  p.a_rows = q_len;
  p.a_heads = heads;
#define B200_KF_SWEEP(MODE_, BF, GEN_, TA, TX, TN, NC, NT) \
  launch_sweep<MODE_, 64, B200_KF_STAGES, BF, false, AUX_NONE, false, B200_KF_CWG, GEN_>(TA, TX, TN, p, NC, NT, stream)
  if (gen)
    rc = bf16 ? B200_KF_SWEEP(SWEEP_KF_ROWLSE, true, true, tq128, tk64, tn_rows128, 1, q_tiles)
              : B200_KF_SWEEP(SWEEP_KF_ROWLSE, false, true, tq128, tk64, tn_rows128, 1, q_tiles);
  else
    rc = bf16 ? B200_KF_SWEEP(SWEEP_KF_ROWLSE, true, false, tq128, tk64, tn_rows128, 1, q_tiles)
              : B200_KF_SWEEP(SWEEP_KF_ROWLSE, false, false, tq128, tk64, tn_rows128, 1, q_tiles);
  if (rc != B200_OK) return rc;
  // sweep 2: per-key sums of exp2(z_ij - Lz_i)
  const int gy = w.kv_pad / 128;
  p.a_base = static_cast<const uint16_t*>(k);
  p.a_rows = kv_len;
  p.a_heads = kv_heads;
  if (gen)
    rc = bf16 ? B200_KF_SWEEP(SWEEP_KF_COLSUM, true, true, tk128, tq64, tn_rows64, p.n_chunks, gy)
              : B200_KF_SWEEP(SWEEP_KF_COLSUM, false, true, tk128, tq64, tn_rows64, p.n_chunks, gy);
  else
    rc = bf16 ? B200_KF_SWEEP(SWEEP_KF_COLSUM, true, false, tk128, tq64, tn_rows64, p.n_chunks, gy)
              : B200_KF_SWEEP(SWEEP_KF_COLSUM, false, false, tk128, tq64, tn_rows64, p.n_chunks, gy);
#undef B200_KF_SWEEP
  if (rc != B200_OK) return rc;

  dim3 rgrid((kv_len + 255) / 256, batch * kv_heads);
  score_reduce_kernel<<<rgrid, 256, 0, stream>>>(kf_score, nullptr, p.partial, nullptr, kv_len, w.kv_pad,
                                                 p.n_chunks * group, 1.0f / (float)group);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

}  // namespace b200
