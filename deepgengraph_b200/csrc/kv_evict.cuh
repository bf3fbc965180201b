// KV-cache eviction step that follows the score-producing attention variants: per (batch, head) keep the
// `budget` keys with the largest score, in position order, and gather their K and V rows into a compact cache.
//
// Reference: deepgengraph_exp/cases/models/h2o.py:51-57 (identical in models/kf.py:54-60):
//     _, idx = torch.topk(score, k=budget, dim=-1, sorted=True); idx = idx.sort(dim=-1)[0]
//     k_cache = gather(k, idx); v_cache = gather(v, idx); kv_cache = cat([k_cache, v_cache], dim=1)
// i.e. the result only depends on the SET of the top-`budget` keys; it is emitted in ascending key order.
//
// One to eight CTAs per (batch, head), each of which repeats the (cheap) selection and gathers its share of the
// rows: the order keys are staged in shared memory once, a 4-pass radix select (8 bits per pass, shared-memory
// histogram) finds the value of the budget-th largest score, one ordered compaction (per-thread key segments, two
// block scans in all) emits the selected key indices already sorted, and the rows are copied with 16-byte accesses.  Ties at the threshold value are
// resolved towards the lower key index (torch.topk leaves that choice unspecified).  The selection is a chain of
// block-wide steps on 16 KB of keys (latency-bound); the gather moves 2 * budget * D elements per head.
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


// Block-wide radix select (4 passes of 8 bits, most significant first): key value of the `want`-th largest key
// among the keys with use(i) true.  Returns the threshold; *need_equal = how many keys EQUAL to it belong to
// the top `want`.  The histogram is built with plain shared-memory atomics (aggregating equal bins per warp with
// match.any first measured slower: 28.5 vs 23.0 us for the top-k kernel at 2 x 32 heads of 4096 scores), and the
// bin that holds the want-th key is found with one block-wide suffix scan instead of a serial walk over the bins.
template <class KeyFn, class UseFn>
__device__ __forceinline__ uint32_t block_radix_select(KeyFn key, UseFn use, int seq, int want, int* hist,
                                                       int* warp_sums, uint32_t* s_prefix, int* s_remaining,
                                                       int* need_equal) {
  static_assert(kEvictThreads == 256, "one thread per histogram bin");
  __syncthreads();
  if (threadIdx.x == 0) {
    *s_prefix = 0;
    *s_remaining = want;
  }
  uint32_t mask = 0;
  for (int pass = 3; pass >= 0; --pass) {
    hist[threadIdx.x] = 0;
    __syncthreads();
    const uint32_t prefix = *s_prefix;
    const int remaining = *s_remaining;
    const int shift = pass * 8;
    for (int i0 = 0; i0 < seq; i0 += kEvictThreads) {
      const int i = i0 + threadIdx.x;
      if (i < seq && use(i)) {
        const uint32_t u = key(i);
        if ((u & mask) == prefix) atomicAdd(&hist[(u >> shift) & 0xff], 1);
      }
    }
    __syncthreads();
    // thread t owns bin 255 - t: `above` = keys in higher bins; the wanted bin has above < remaining <= above + own
    const int own = hist[255 - threadIdx.x];
    int total;
    const int above = block_exclusive_scan(own, warp_sums, &total);
    if (above < remaining && remaining <= above + own) {
      *s_prefix = prefix | ((uint32_t)(255 - threadIdx.x) << shift);
      *s_remaining = remaining - above;
    } else if (threadIdx.x == 255 && remaining > total) {   // fewer candidates than wanted: take them all
      *s_prefix = prefix;
      *s_remaining = remaining - (total - own);
    }
    mask |= 0xffu << shift;
    __syncthreads();
  }
  *need_equal = *s_remaining;
  return *s_prefix;
}


// Position of key i inside a shared-memory key array: one padding word per 32 keys, so that both access patterns of
// the kernels are free of bank conflicts -- consecutive threads on consecutive keys (histogram passes) and thread t on
// its own contiguous segment of keys (ordered compaction; a segment of 16 keys would otherwise put 16 lanes on one bank).
__device__ __forceinline__ int skew(int i) { return i + (i >> 5); }
inline size_t skewed_words(int n) { return (size_t)n + (size_t)(n >> 5) + 1; }

// Ordered compaction.  Thread t owns the contiguous keys [t * K, (t + 1) * K), K = ceil(seq / threads): it counts the
// keys of its segment that are selected for sure (`sure`) and those that tie at the threshold (`tie`), ONE block-wide
// scan per count turns them into the number of such keys before the segment, and a second walk over the segment
// emits every selected key with its final position: (#sure before it) + min(#ties before it, need_tie) -- the first
// `need_tie` ties in key order are the ones taken.  (The previous form scanned the block once per 256 keys: sixteen
// scans of two barriers each at 4096 keys, where this one has two.)
template <class SureFn, class TieFn, class EmitFn>
__device__ __forceinline__ void ordered_compact(SureFn sure, TieFn tie, EmitFn emit, int seq, int need_tie,
                                                int* warp_sums) {
  const int per_thread = (seq + kEvictThreads - 1) / kEvictThreads;
  const int lo = min(seq, (int)threadIdx.x * per_thread), hi = min(seq, lo + per_thread);
  int n_sure = 0, n_tie = 0;
  for (int i = lo; i < hi; ++i) {
    n_sure += sure(i) ? 1 : 0;
    n_tie += tie(i) ? 1 : 0;
  }
  int total;
  int sure_before = block_exclusive_scan(n_sure, warp_sums, &total);
  int tie_before = block_exclusive_scan(n_tie, warp_sums, &total);
  for (int i = lo; i < hi; ++i) {
    const bool is_sure = sure(i), is_tie = tie(i);
    if (is_sure || (is_tie && tie_before < need_tie)) emit(i, sure_before + min(tie_before, need_tie));
    sure_before += is_sure ? 1 : 0;
    tie_before += is_tie ? 1 : 0;
  }
}

// Gather of the selected rows: kv_cache[b, 0, i, h, :] = k[b, idx_i, h, :], kv_cache[b, 1, i, h, :] = v[b, idx_i, h, :].
// The CTAs of one (batch, head) -- gridDim.y of them, each of which has made the same selection -- take
// interleaved slices of the rows; four 16-byte K and V loads are in flight per thread before the first store.
__device__ __forceinline__ void gather_selected_rows(const int32_t* s_idx, const uint8_t* __restrict__ k,
                                                     const uint8_t* __restrict__ v, uint8_t* __restrict__ kv_cache,
                                                     int b, int h, int seq, int heads, int row_bytes, int keep) {
  const int vec_per_row = row_bytes / 16;                 // row_bytes is a multiple of 16, checked on the host
  const int64_t src_row_stride = (int64_t)heads * row_bytes;                 // [B, S, H, D]
  const int64_t src_batch = (int64_t)b * seq * src_row_stride + (int64_t)h * row_bytes;
  const int64_t dst_plane = (int64_t)keep * heads * row_bytes;               // [B, 2, keep, H, D]
  const int64_t dst_batch = (int64_t)b * 2 * dst_plane + (int64_t)h * row_bytes;
  const int total = keep * vec_per_row;
  const int stride = kEvictThreads * gridDim.y;
  constexpr int U = 4;
  for (int g0 = blockIdx.y * kEvictThreads + threadIdx.x; g0 < total; g0 += U * stride) {
    uint4 kk[U], vv[U];
    int64_t dst[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int g = g0 + u * stride;
      if (g < total) {
        const int r = g / vec_per_row, c = g - r * vec_per_row;
        const int64_t src = src_batch + (int64_t)s_idx[r] * src_row_stride + c * 16;
        dst[u] = dst_batch + (int64_t)r * src_row_stride + c * 16;
        kk[u] = *reinterpret_cast<const uint4*>(k + src);
        vv[u] = *reinterpret_cast<const uint4*>(v + src);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (g0 + u * stride < total) {
        *reinterpret_cast<uint4*>(kv_cache + dst[u]) = kk[u];
        *reinterpret_cast<uint4*>(kv_cache + dst[u] + dst_plane) = vv[u];
      }
    }
  }
}

// CTAs per (batch, head): enough to fill the GPU when there are few heads (every CTA repeats the selection,
// which reads 16 KB of scores from L2, and gathers its share of the rows)
inline int evict_ctas_per_head(int batch_heads) {
  const int want = (2 * sm_count() + batch_heads - 1) / batch_heads;
  return std::max(1, std::min(8, want));
}

template <int ELEM_BYTES>
__global__ void __launch_bounds__(kEvictThreads)
kv_evict_topk_kernel(const float* __restrict__ score, const uint8_t* __restrict__ k, const uint8_t* __restrict__ v,
                     uint8_t* __restrict__ kv_cache, int32_t* __restrict__ indices_out, int seq, int heads,
                     int head_dim, int budget, int staged) {
  __shared__ int hist[256];
  __shared__ int warp_sums[kEvictThreads / 32];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;
  extern __shared__ int32_t s_idx[];   // [budget] selected key indices, ascending
  uint32_t* s_keys = reinterpret_cast<uint32_t*>(s_idx + budget);   // [seq] order keys, when they fit (`staged`)

  const int bh = blockIdx.x, b = bh / heads, h = bh - b * heads;
  const float* sc = score + (int64_t)bh * seq;

  // The five passes below each touch every score; staged in shared memory once (all loads in flight together)
  // they cost a shared-memory read instead of a dependent L2 round trip per pass.
  if (staged) {
#pragma unroll 8
    for (int i = threadIdx.x; i < seq; i += kEvictThreads) s_keys[skew(i)] = score_key(sc[i]);
  }
  auto key_of = [&](int i) { return staged ? s_keys[skew(i)] : score_key(sc[i]); };

  // ---- radix select: key value of the budget-th largest score ----
  int need_equal;
  const uint32_t thr = block_radix_select(key_of, [](int) { return true; }, seq, budget, hist, warp_sums, &s_prefix,
                                          &s_remaining, &need_equal);

  // ---- ordered compaction: selected indices in ascending order ----
  // Selected = every key above the threshold plus the first `need_equal` keys equal to it.
  ordered_compact([&](int i) { return key_of(i) > thr; }, [&](int i) { return key_of(i) == thr; },
                  [&](int i, int pos) {
                    if (pos < budget) s_idx[pos] = i;
                  },
                  seq, need_equal, warp_sums);
  __syncthreads();

  if (indices_out != nullptr && blockIdx.y == 0)
    for (int i = threadIdx.x; i < budget; i += kEvictThreads) indices_out[(int64_t)bh * budget + i] = s_idx[i];

  gather_selected_rows(s_idx, k, v, kv_cache, b, h, seq, heads, head_dim * ELEM_BYTES, budget);
}

// ---------------------------------------------------------------------------------------------------------
// RoCo's selection (deepgengraph_exp/cases/models/roco.py:52-66):
//   std   = sqrt(sq / q_len - (score / q_len) ** 2)
//   A     = the `recent` keys with the LARGEST std            (topk(std, largest=True, k=recent))
//   B     = among the other keys, the `budget` keys with the largest score / q_len
//   cache = K, V rows of A u B in position order              -> [B, 2, budget + recent, H, D]
// One CTA per (batch, head): radix select on std, an ordered pass that marks A in a shared-memory byte map,
// radix select on the mean score over the unmarked keys, one ordered compaction, gather.  The statistics are
// recomputed from the two score vectors in every pass (L2 hits) with the reference's fp32 operation order
// (round-to-nearest division, multiply, subtract, square root -- no contraction, no approximations), so the
// ordering of the keys is the reference's.  NaN (variance rounded below zero) ranks above +inf, as in torch.topk.
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t score_key_nan_high(float f) {
  return (f != f) ? 0xffffffffu : score_key(f);
}
__device__ __forceinline__ float roco_mean(float score, float q_len) { return __fdiv_rn(score, q_len); }
__device__ __forceinline__ float roco_std(float score, float sq, float q_len) {
  const float m = __fdiv_rn(score, q_len);
  return __fsqrt_rn(__fsub_rn(__fdiv_rn(sq, q_len), __fmul_rn(m, m)));
}

template <int ELEM_BYTES>
__global__ void __launch_bounds__(kEvictThreads)
kv_evict_roco_kernel(const float* __restrict__ score, const float* __restrict__ score_sq,
                     const uint8_t* __restrict__ k, const uint8_t* __restrict__ v, uint8_t* __restrict__ kv_cache,
                     int32_t* __restrict__ indices_out, int seq, int heads, int head_dim, float q_len, int budget,
                     int recent, int staged) {
  __shared__ int hist[256];
  __shared__ int warp_sums[kEvictThreads / 32];
  __shared__ uint32_t s_prefix;
  __shared__ int s_remaining;
  extern __shared__ int32_t s_dyn[];
  const int keep = budget + recent;
  int32_t* s_idx = s_dyn;                                        // [keep] selected key indices, ascending
  const int key_words = staged ? seq + (seq >> 5) + 1 : 0;      // padded key arrays (see skew)
  uint32_t* s_std = reinterpret_cast<uint32_t*>(s_dyn + keep);   // order keys of std   (when `staged`)
  uint32_t* s_mean = s_std + key_words;                          // order keys of score / q_len
  uint8_t* in_a = reinterpret_cast<uint8_t*>(s_mean + key_words);   // [seq] 1 = key belongs to A

  const int bh = blockIdx.x, b = bh / heads, h = bh - b * heads;
  const float* sc = score + (int64_t)bh * seq;
  const float* sq = score_sq + (int64_t)bh * seq;
  if (staged) {
#pragma unroll 4
    for (int i = threadIdx.x; i < seq; i += kEvictThreads) {
      const float a = sc[i], a2 = sq[i];
      s_std[skew(i)] = score_key_nan_high(roco_std(a, a2, q_len));
      s_mean[skew(i)] = score_key_nan_high(roco_mean(a, q_len));
    }
  }
  auto std_key = [&](int i) { return staged ? s_std[skew(i)] : score_key_nan_high(roco_std(sc[i], sq[i], q_len)); };
  auto mean_key = [&](int i) { return staged ? s_mean[skew(i)] : score_key_nan_high(roco_mean(sc[i], q_len)); };

  // ---- A: the `recent` keys with the largest std (ties towards the lower index) ----
  for (int i = threadIdx.x; i < seq; i += kEvictThreads) in_a[i] = 0;
  if (recent > 0) {
    int need_eq;
    const uint32_t thr = block_radix_select(std_key, [](int) { return true; }, seq, recent, hist, warp_sums,
                                            &s_prefix, &s_remaining, &need_eq);
    __syncthreads();   // in_a cleared by all threads before any thread marks its segment
    ordered_compact([&](int i) { return std_key(i) > thr; }, [&](int i) { return std_key(i) == thr; },
                    [&](int i, int) { in_a[i] = 1; }, seq, need_eq, warp_sums);
  }
  __syncthreads();

  // ---- B: among the other keys, the `budget` keys with the largest mean score ----
  int need_eq_b = 0;
  uint32_t thr_b = 0xffffffffu;
  if (budget > 0)
    thr_b = block_radix_select(mean_key, [&](int i) { return in_a[i] == 0; }, seq, budget, hist, warp_sums,
                               &s_prefix, &s_remaining, &need_eq_b);

  // ---- ordered compaction of A u B ----
  // "sure" keys (in A, or above the B threshold) and the first need_eq_b keys that tie at the B threshold
  ordered_compact([&](int i) { return in_a[i] != 0 || (budget > 0 && mean_key(i) > thr_b); },
                  [&](int i) { return in_a[i] == 0 && budget > 0 && mean_key(i) == thr_b; },
                  [&](int i, int pos) {
                    if (pos < keep) s_idx[pos] = i;
                  },
                  seq, need_eq_b, warp_sums);
  __syncthreads();

  if (indices_out != nullptr && blockIdx.y == 0)
    for (int i = threadIdx.x; i < keep; i += kEvictThreads) indices_out[(int64_t)bh * keep + i] = s_idx[i];

  gather_selected_rows(s_idx, k, v, kv_cache, b, h, seq, heads, head_dim * ELEM_BYTES, keep);
}

// Dynamic shared memory beyond which a kernel must opt in (cudaFuncAttributeMaxDynamicSharedMemorySize).  The
// 48 KB default covers static AND dynamic shared memory together, and both eviction kernels carry about 1 KB of
// static arrays (histogram, scan scratch), so the opt-in starts well below 48 KB of dynamic memory.
constexpr size_t kEvictSmemOptIn = 40 * 1024;

template <int ELEM_BYTES>
int launch_kv_evict_roco(dim3 grid, size_t smem, cudaStream_t stream, const float* score, const float* score_sq,
                         const void* k, const void* v, void* kv_cache, int32_t* indices, int seq, int heads,
                         int head_dim, int q_len, int budget, int recent, int staged) {
  auto kern = kv_evict_roco_kernel<ELEM_BYTES>;
  static thread_local int configured_dev = -1;   // one per instantiation: every kernel needs its own attribute call
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (smem > kEvictSmemOptIn && configured_dev != dev) {
    B200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    configured_dev = dev;
  }
  kern<<<grid, kEvictThreads, smem, stream>>>(score, score_sq, (const uint8_t*)k, (const uint8_t*)v,
                                              (uint8_t*)kv_cache, indices, seq, heads, head_dim, (float)q_len, budget,
                                              recent, staged);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

template <int ELEM_BYTES>
int launch_kv_evict_topk(dim3 grid, size_t smem, cudaStream_t stream, const float* score, const void* k,
                         const void* v, void* kv_cache, int32_t* indices, int seq, int heads, int head_dim,
                         int budget, int staged) {
  auto kern = kv_evict_topk_kernel<ELEM_BYTES>;
  static thread_local int configured_dev = -1;
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (smem > kEvictSmemOptIn && configured_dev != dev) {
    B200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    configured_dev = dev;
  }
  kern<<<grid, kEvictThreads, smem, stream>>>(score, (const uint8_t*)k, (const uint8_t*)v, (uint8_t*)kv_cache, indices,
                                              seq, heads, head_dim, budget, staged);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

inline int kv_evict_roco_impl(const float* score, const float* score_sq, const void* k, const void* v,
                              void* kv_cache, int32_t* indices, int batch, int seq, int heads, int head_dim,
                              int q_len, int budget, int recent, int elem_bytes, cudaStream_t stream) {
  if (!score || !score_sq || !k || !v || !kv_cache) return B200_ERR_BAD_ARGUMENT;
  if (batch <= 0 || seq <= 0 || heads <= 0 || head_dim <= 0 || q_len <= 0) return B200_ERR_BAD_ARGUMENT;
  if (budget < 0 || recent < 0 || budget + recent <= 0 || budget + recent > seq) return B200_ERR_BAD_ARGUMENT;
  if (elem_bytes != 2 && elem_bytes != 4) return B200_ERR_BAD_DTYPE;
  if ((head_dim * elem_bytes) % 16 != 0 || !aligned16(k) || !aligned16(v) || !aligned16(kv_cache))
    return B200_ERR_MISALIGNED;
  const size_t smem_min = (size_t)(budget + recent) * sizeof(int32_t) + (size_t)((seq + 15) / 16) * 16;
  if (smem_min > 200 * 1024) return B200_ERR_UNSUPPORTED;
  const size_t key_bytes = 2 * skewed_words(seq) * sizeof(uint32_t);   // std and mean keys, padded
  const int staged = smem_min + key_bytes <= 200 * 1024 ? 1 : 0;
  const size_t smem = smem_min + (staged ? key_bytes : 0);
  const dim3 grid(batch * heads, evict_ctas_per_head(batch * heads));
  return elem_bytes == 2
             ? launch_kv_evict_roco<2>(grid, smem, stream, score, score_sq, k, v, kv_cache, indices, seq, heads,
                                       head_dim, q_len, budget, recent, staged)
             : launch_kv_evict_roco<4>(grid, smem, stream, score, score_sq, k, v, kv_cache, indices, seq, heads,
                                       head_dim, q_len, budget, recent, staged);
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
  const size_t smem_idx = (size_t)budget * sizeof(int32_t);
  const size_t key_bytes = skewed_words(seq) * sizeof(uint32_t);   // padded key array
  const int staged = smem_idx + key_bytes <= 200 * 1024 ? 1 : 0;
  const size_t smem = smem_idx + (staged ? key_bytes : 0);
  const dim3 grid(batch * heads, evict_ctas_per_head(batch * heads));
  return elem_bytes == 2 ? launch_kv_evict_topk<2>(grid, smem, stream, score, k, v, kv_cache, indices, seq, heads,
                                                   head_dim, budget, staged)
                         : launch_kv_evict_topk<4>(grid, smem, stream, score, k, v, kv_cache, indices, seq, heads,
                                                   head_dim, budget, staged);
}

}  // namespace b200
