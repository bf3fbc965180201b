// KV-cache eviction step that follows the score-producing attention variants: per (batch, head) keep the
// `budget` keys with the largest score, in position order, and gather their K and V rows into a compact cache.
//
// Reference: deepgengraph_exp/cases/models/h2o.py:51-57 (identical in models/kf.py:54-60):
//     _, idx = torch.topk(score, k=budget, dim=-1, sorted=True); idx = idx.sort(dim=-1)[0]
//     k_cache = gather(k, idx); v_cache = gather(v, idx); kv_cache = cat([k_cache, v_cache], dim=1)
// i.e. the result only depends on the SET of the top-`budget` keys; it is emitted in ascending key order.
//
// One CTA per (batch, head): a 4-pass radix select (8 bits per pass, shared-memory histogram) finds the value of
// the budget-th largest score, one ordered compaction pass emits the selected key indices already sorted, and the
// CTA then copies the selected rows with 16-byte accesses.  Ties at the threshold value are resolved towards the
// lower key index (torch.topk leaves that choice unspecified).  HBM-bound: reads the scores five times from L2
// (16 KB per head) and moves 2 * budget * D elements.
#pragma once

#include "common.cuh"

namespace b200 {

__device__ __forceinline__ uint32_t score_key(float f) {
  // monotone map float -> uint32 (larger float <=> larger key); -0.0 and +0.0 differ, NaNs sort above +inf
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int kEvictThreads = 256;

// exclusive block-wide prefix sum of one int per thread; returns the thread's offset, *total = block sum
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_sums, int* total) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  __syncthreads();   // protects warp_sums against its previous use
  if (lane == 31) warp_sums[wid] = incl;
  __syncthreads();
  int base = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < kEvictThreads / 32; ++w) {
    const int s = warp_sums[w];
    if (w < wid) base += s;
    tot += s;
  }
  *total = tot;
  return base + incl - v;
}

template <int ELEM_BYTES>
__global__ void __launch_bounds__(kEvictThreads)
kv_evict_topk_kernel(const float* __restrict__ score, const uint8_t* __restrict__ k, const uint8_t* __restrict__ v,
                     uint8_t* __restrict__ kv_cache, int32_t* __restrict__ indices_out, int seq, int heads,
                     int head_dim, int budget) {
  __shared__ int hist[256];
  __shared__ int warp_sums[kEvictThreads / 32];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;
  extern __shared__ int32_t s_idx[];   // [budget] selected key indices, ascending

  const int bh = blockIdx.x, b = bh / heads, h = bh - b * heads;
  const float* sc = score + (int64_t)bh * seq;

  // ---- radix select: key value of the budget-th largest score ----
  if (threadIdx.x == 0) {
    s_prefix = 0;
    s_remaining = budget;
  }
  uint32_t mask = 0;
  for (int pass = 3; pass >= 0; --pass) {
    for (int i = threadIdx.x; i < 256; i += kEvictThreads) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const int shift = pass * 8;
    for (int i = threadIdx.x; i < seq; i += kEvictThreads) {
      const uint32_t u = score_key(sc[i]);
      if ((u & mask) == prefix) atomicAdd(&hist[(u >> shift) & 0xff], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int remaining = s_remaining, bin = 255;
      for (; bin > 0; --bin) {
        if (hist[bin] >= remaining) break;
        remaining -= hist[bin];
      }
      s_prefix = prefix | ((uint32_t)bin << shift);
      s_remaining = remaining;   // how many keys equal to the final prefix are still needed
    }
    mask |= 0xffu << shift;
    __syncthreads();
  }
  const uint32_t thr = s_prefix;
  const int need_equal = s_remaining;

  // ---- ordered compaction: selected indices in ascending order ----
  int sel_base = 0, eq_base = 0;
  for (int i0 = 0; i0 < seq; i0 += kEvictThreads) {
    const int i = i0 + threadIdx.x;
    const uint32_t u = i < seq ? score_key(sc[i]) : 0u;
    const int is_eq = (i < seq && u == thr) ? 1 : 0;
    int eq_total, sel_total;
    const int eq_before = eq_base + block_exclusive_scan(is_eq, warp_sums, &eq_total);
    const int is_sel = (i < seq && (u > thr || (is_eq && eq_before < need_equal))) ? 1 : 0;
    const int pos = sel_base + block_exclusive_scan(is_sel, warp_sums, &sel_total);
    if (is_sel && pos < budget) s_idx[pos] = i;
    sel_base += sel_total;
    eq_base += eq_total;
  }
  __syncthreads();

  if (indices_out != nullptr)
    for (int i = threadIdx.x; i < budget; i += kEvictThreads) indices_out[(int64_t)bh * budget + i] = s_idx[i];

  // ---- gather: kv_cache[b, 0, i, h, :] = k[b, idx_i, h, :], kv_cache[b, 1, i, h, :] = v[b, idx_i, h, :] ----
  const int row_bytes = head_dim * ELEM_BYTES;            // multiple of 16, checked on the host
  const int vec_per_row = row_bytes / 16;
  const int64_t src_row_stride = (int64_t)heads * row_bytes;                 // [B, S, H, D]
  const int64_t src_batch = (int64_t)b * seq * src_row_stride + (int64_t)h * row_bytes;
  const int64_t dst_plane = (int64_t)budget * heads * row_bytes;             // [B, 2, budget, H, D]
  const int64_t dst_batch = (int64_t)b * 2 * dst_plane + (int64_t)h * row_bytes;
  const int total = budget * vec_per_row;
  for (int g = threadIdx.x; g < total; g += kEvictThreads) {
    const int r = g / vec_per_row, c = g - r * vec_per_row;
    const int64_t src = src_batch + (int64_t)s_idx[r] * src_row_stride + c * 16;
    const int64_t dst = dst_batch + (int64_t)r * src_row_stride + c * 16;
    *reinterpret_cast<uint4*>(kv_cache + dst) = *reinterpret_cast<const uint4*>(k + src);
    *reinterpret_cast<uint4*>(kv_cache + dst + dst_plane) = *reinterpret_cast<const uint4*>(v + src);
  }
}

inline int kv_evict_topk_impl(const float* score, const void* k, const void* v, void* kv_cache, int32_t* indices,
                              int batch, int seq, int heads, int head_dim, int budget, int elem_bytes,
                              cudaStream_t stream) {
  if (!score || !k || !v || !kv_cache) return B200_ERR_BAD_ARGUMENT;
  if (batch <= 0 || seq <= 0 || heads <= 0 || head_dim <= 0) return B200_ERR_BAD_ARGUMENT;
  if (budget <= 0 || budget > seq) return B200_ERR_BAD_ARGUMENT;
  if (elem_bytes != 2 && elem_bytes != 4) return B200_ERR_BAD_DTYPE;
  if ((head_dim * elem_bytes) % 16 != 0 || !aligned16(k) || !aligned16(v) || !aligned16(kv_cache))
    return B200_ERR_MISALIGNED;
  if (budget > 12288) return B200_ERR_UNSUPPORTED;   // index list lives in shared memory (48 KB)
  const size_t smem = (size_t)budget * sizeof(int32_t);
  const int grid = batch * heads;
  if (elem_bytes == 2)
    kv_evict_topk_kernel<2><<<grid, kEvictThreads, smem, stream>>>(score, (const uint8_t*)k, (const uint8_t*)v,
                                                                   (uint8_t*)kv_cache, indices, seq, heads, head_dim,
                                                                   budget);
  else
    kv_evict_topk_kernel<4><<<grid, kEvictThreads, smem, stream>>>(score, (const uint8_t*)k, (const uint8_t*)v,
                                                                   (uint8_t*)kv_cache, indices, seq, heads, head_dim,
                                                                   budget);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

}  // namespace b200
