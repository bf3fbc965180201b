// Bandwidth kernels: RMSNorm, fused-add RMSNorm, SiLU/GELU-gate, online rotary embedding.
// All of them are HBM-bound; they move 16 bytes per thread per access, keep a row in
// registers between the reduction and the scaling (one read of the input instead of
// the two passes of the reference kernels), and run as persistent grids sized to the
// SM count.
#pragma once

#include <type_traits>

#include "common.cuh"

namespace b200 {

// ---------------------------------------------------------------------------
// 16-byte vector of elements of type T
// ---------------------------------------------------------------------------
template <typename T>
struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  uint4 raw;
};

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

template <typename T>
__device__ __forceinline__ void unpack16(const uint4& raw, float (&f)[16 / sizeof(T)]) {
  const T* p = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < (int)(16 / sizeof(T)); ++i) f[i] = to_f32<T>(p[i]);
}
template <typename T>
__device__ __forceinline__ uint4 pack16(const float (&f)[16 / sizeof(T)]) {
  uint4 raw;
  T* p = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < (int)(16 / sizeof(T)); ++i) p[i] = from_f32<T>(f[i]);
  return raw;
}

// y = T(x * inv) * w with the last product taken in T (csrc/norm.cu:54), for one 16-byte vector.  For the 16-bit
// types the product of the two T values is one packed multiply (a single rounding, the same result as the fp32
// product rounded once): a third of the instructions of the convert-multiply-convert form.
template <typename T>
__device__ __forceinline__ uint4 scale_round_mul(const float (&x)[16 / sizeof(T)], float inv, const uint4& w_raw) {
  uint4 out;
  if constexpr (sizeof(T) == 4) {
    const float* w = reinterpret_cast<const float*>(&w_raw);
    float* o = reinterpret_cast<float*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = (x[i] * inv) * w[i];
  } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&w_raw);
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) o2[i] = __hmul2(__floats2bfloat162_rn(x[2 * i] * inv, x[2 * i + 1] * inv), w2[i]);
  } else {
    const __half2* w2 = reinterpret_cast<const __half2*>(&w_raw);
    __half2* o2 = reinterpret_cast<__half2*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) o2[i] = __hmul2(__floats2half2_rn(x[2 * i] * inv, x[2 * i + 1] * inv), w2[i]);
  }
  return out;
}

__device__ __forceinline__ uint4 ld_nc_16(const void* p) {  // streaming read, no L1 allocation
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void st_16(void* p, const uint4& v) { *reinterpret_cast<uint4*>(p) = v; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum over the whole block; every thread receives the result.  `red` holds 33 floats.
template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  constexpr int WARPS = THREADS / 32;
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  __syncthreads();  // protects `red` against the previous use
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float t = (lane < WARPS) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// ---------------------------------------------------------------------------
// RMSNorm.  out = T(x * rsqrt(mean(x^2) + eps)) * w, the last product taken in T
// exactly as the reference does (csrc/norm.cu:54).
// One warp per row, the row kept in registers: MAXV 16-byte vectors per lane.  FUSED_ADD: x = input + residual, residual <- T(x), and the second
// phase re-reads the ROUNDED residual like csrc/norm.cu:80 (variance from the
// unrounded sum, csrc/norm.cu:68-70).
// ---------------------------------------------------------------------------
template <typename T, int MAXV, bool FUSED_ADD, int THREADS>
__global__ void __launch_bounds__(THREADS)
rms_norm_rows_kernel(T* __restrict__ out, T* __restrict__ input, T* __restrict__ residual,
                     const T* __restrict__ weight, float epsilon, int64_t num_tokens, int hidden) {
  // One WARP per row: the row lives in the warp's registers as raw 16-byte vectors (lane l holds vectors
  // l, l + 32, ...), the reduction is five shuffles, and no block-wide barrier sits between a row's load and
  // its store -- every warp of the grid streams rows independently.
  constexpr int VN = 16 / sizeof(T);
  const int nvec = hidden / VN;  // hidden % VN == 0 checked on the host
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = (int64_t)blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5);
  const int64_t warp_count = (int64_t)gridDim.x * (THREADS / 32);
  for (int64_t row = warp_global; row < num_tokens; row += warp_count) {
    T* in_row = input + row * hidden;
    uint4 raw[MAXV];
    float ss = 0.f;
    if constexpr (FUSED_ADD) {
      T* res_row = residual + row * hidden;
      // the input row is loaded whole, the residual row in two halves (each half's loads are issued together, before
      // that half's stores): the second operand never needs more than half a row of registers, which lets more
      // rows be resident per SM
      constexpr int HV = MAXV >= 8 ? (MAXV + 1) / 2 : MAXV;
#pragma unroll
      for (int v = 0; v < MAXV; ++v) {
        const int idx = lane + v * 32;
        if (idx < nvec) raw[v] = ld_16(in_row + (int64_t)idx * VN);
      }
#pragma unroll
      for (int h0 = 0; h0 < MAXV; h0 += HV) {
        uint4 rres[HV];
#pragma unroll
        for (int v = 0; v < HV; ++v) {
          const int idx = lane + (h0 + v) * 32;
          if (idx < nvec) rres[v] = ld_16(res_row + (int64_t)idx * VN);
        }
#pragma unroll
        for (int v = 0; v < HV; ++v) {
          const int idx = lane + (h0 + v) * 32;
          if (idx < nvec) {
            float x[VN], r[VN];
            unpack16<T>(raw[h0 + v], x);
            unpack16<T>(rres[v], r);
#pragma unroll
            for (int i = 0; i < VN; ++i) {
              x[i] += r[i];
              ss += x[i] * x[i];      // variance from the unrounded sum (csrc/norm.cu:68-70)
            }
            raw[h0 + v] = pack16<T>(x);    // phase two sees the rounded residual (csrc/norm.cu:80)
            st_16(res_row + (int64_t)idx * VN, raw[h0 + v]);
          }
        }
      }
    } else {
#pragma unroll
      for (int v = 0; v < MAXV; ++v) {
        const int idx = lane + v * 32;
        if (idx < nvec) raw[v] = ld_nc_16(in_row + (int64_t)idx * VN);
      }
#pragma unroll
      for (int v = 0; v < MAXV; ++v) {
        const int idx = lane + v * 32;
        if (idx < nvec) {
          float x[VN];
          unpack16<T>(raw[v], x);
#pragma unroll
          for (int i = 0; i < VN; ++i) ss += x[i] * x[i];
        }
      }
    }
    const float inv = rsqrtf(warp_sum(ss) / (float)hidden + epsilon);
    T* out_row = (FUSED_ADD ? input : out) + row * hidden;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int idx = lane + v * 32;
      if (idx < nvec) {
        float x[VN];
        unpack16<T>(raw[v], x);
        st_16(out_row + (int64_t)idx * VN, scale_round_mul<T>(x, inv, ld_16(weight + (int64_t)idx * VN)));
      }
    }
  }
}

// Generic fallback (any hidden size, any alignment): two passes over the row like the
// reference, scalar accesses.  Only used for shapes the vector kernel cannot take.
template <typename T, bool FUSED_ADD>
__global__ void __launch_bounds__(256)
rms_norm_generic_kernel(T* __restrict__ out, T* __restrict__ input, T* __restrict__ residual,
                        const T* __restrict__ weight, float epsilon, int64_t num_tokens, int hidden) {
  __shared__ float red[33];
  for (int64_t row = blockIdx.x; row < num_tokens; row += gridDim.x) {
    T* in_row = input + row * hidden;
    T* res_row = FUSED_ADD ? residual + row * hidden : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += 256) {
      float x = to_f32<T>(in_row[i]);
      if constexpr (FUSED_ADD) {
        x += to_f32<T>(res_row[i]);
        res_row[i] = from_f32<T>(x);
      }
      ss += x * x;
    }
    const float total = block_sum<256>(ss, red);
    const float inv = rsqrtf(total / (float)hidden + epsilon);
    T* out_row = (FUSED_ADD ? input : out) + row * hidden;
    for (int i = threadIdx.x; i < hidden; i += 256) {
      const float x = to_f32<T>(FUSED_ADD ? res_row[i] : in_row[i]);
      out_row[i] = from_f32<T>(to_f32<T>(from_f32<T>(x * inv)) * to_f32<T>(weight[i]));
    }
  }
}

template <typename T, bool FUSED_ADD>
int launch_rms_norm(void* out, void* input, void* residual, const void* weight, float eps, int64_t num_tokens,
                    int hidden, cudaStream_t stream) {
  constexpr int VN = 16 / sizeof(T);
  const int sms = sm_count();
  const bool vec_ok = (hidden % VN == 0) && aligned16(input) && aligned16(weight) &&
                      (FUSED_ADD ? aligned16(residual) : aligned16(out));
  const int nvec = hidden / VN;
  T* o = (T*)out;
  T* in = (T*)input;
  T* res = (T*)residual;
  const T* w = (const T*)weight;
  if (vec_ok && nvec <= 32 * 32) {
    // One row per warp, small blocks (4 warps): the register footprint of a row (MAXV 16-byte vectors per lane) limits
    // an SM to a few hundred resident threads, and with small blocks those threads belong to several blocks that
    // start and finish at different times, so the load phase of one block overlaps the store phase of another.
    constexpr int TH = 128;
    static const int env_grid = std::getenv("B200_RMS_GRID_PER_SM") ? std::atoi(std::getenv("B200_RMS_GRID_PER_SM")) : 0;
    const int per_sm = env_grid > 0 ? env_grid : 16;
    const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((num_tokens + TH / 32 - 1) / (TH / 32), (int64_t)sms * per_sm));
#define B200_RMS_LAUNCH(MAXV_) \
  rms_norm_rows_kernel<T, MAXV_, FUSED_ADD, TH><<<grid, TH, 0, stream>>>(o, in, res, w, eps, num_tokens, hidden)
    if (nvec <= 64) B200_RMS_LAUNCH(2);
    else if (nvec <= 128) B200_RMS_LAUNCH(4);
    else if (nvec <= 256) B200_RMS_LAUNCH(8);
    else if (nvec <= 448) B200_RMS_LAUNCH(14);
    else if (nvec <= 512) B200_RMS_LAUNCH(16);
    else B200_RMS_LAUNCH(32);
#undef B200_RMS_LAUNCH
  } else {
    const int grid = (int)std::min<int64_t>(num_tokens, (int64_t)sms * 8);
    rms_norm_generic_kernel<T, FUSED_ADD><<<grid, 256, 0, stream>>>(o, in, res, w, eps, num_tokens, hidden);
  }
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

// ---------------------------------------------------------------------------
// Gated activations.  out[t, i] = T(act(x)) * y with x = in[t, i], y = in[t, d + i]
// (csrc/activation.cu:6-22: the activation is rounded to T, the product taken in T).
// ---------------------------------------------------------------------------
struct SiluOp {
  __device__ __forceinline__ float operator()(float x) const { return x / (1.0f + __expf(-x)); }
};
// ACCURATE = true (fp32 tensors): tanh(u) = 1 - 2 / (1 + e^{2u}), spelled out because fast-math maps tanhf to the
// hardware approximation.  ACCURATE = false (16-bit tensors): tanh.approx.f32 itself -- its error (~5e-4 absolute)
// is a quarter of a bf16 ulp of the result and halves the special-function work of the kernel.
template <bool ACCURATE>
struct GeluTanhOpT {
  __device__ __forceinline__ float operator()(float x) const {
    const float kAlpha = 0.7978845608028654f;  // sqrt(2/pi)
    const float inner = kAlpha * (x + 0.044715f * x * x * x);
    const float t = ACCURATE ? 1.0f - 2.0f / (1.0f + __expf(2.0f * inner)) : tanh_approx(inner);
    return 0.5f * x * (1.0f + t);
  }
};
using GeluTanhOp = GeluTanhOpT<true>;

// out = T(act(x)) * y for one 16-byte vector (csrc/activation.cu:6-22: the activation is rounded to T, the product is
// taken in T).  16-bit types: the product is one packed multiply on the raw y pairs (a single rounding, like the fp32
// product rounded once).
template <typename T, typename Op>
__device__ __forceinline__ uint4 act_round_mul(const uint4& x_raw, const uint4& y_raw) {
  constexpr int VN = 16 / sizeof(T);
  Op op;
  float x[VN];
  unpack16<T>(x_raw, x);
  uint4 out;
  if constexpr (sizeof(T) == 4) {
    const float* y = reinterpret_cast<const float*>(&y_raw);
    float* o = reinterpret_cast<float*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = op(x[i]) * y[i];
  } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    const __nv_bfloat162* y2 = reinterpret_cast<const __nv_bfloat162*>(&y_raw);
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) o2[i] = __hmul2(__floats2bfloat162_rn(op(x[2 * i]), op(x[2 * i + 1])), y2[i]);
  } else {
    const __half2* y2 = reinterpret_cast<const __half2*>(&y_raw);
    __half2* o2 = reinterpret_cast<__half2*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) o2[i] = __hmul2(__floats2half2_rn(op(x[2 * i]), op(x[2 * i + 1])), y2[i]);
  }
  return out;
}

// Index = int when the vector count fits 31 bits (a 64-bit division per vector costs more than the activation)
template <typename T, typename Op, typename Index>
__global__ void __launch_bounds__(256)
act_and_mul_vec_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t num_tokens, int d) {
  constexpr int VN = 16 / sizeof(T);
  const Index vec_per_row = (Index)(d / VN);
  const Index total = (Index)num_tokens * vec_per_row;
  const Index step = (Index)gridDim.x * 256;
  // two vectors per thread and step: four 16-byte loads in flight before the first store
  for (Index g = (Index)blockIdx.x * 256 + threadIdx.x; g < total; g += 2 * step) {
    const Index g1 = g + step;
    const Index t0 = g / vec_per_row, t1 = g1 / vec_per_row;
    const Index c0 = g - t0 * vec_per_row, c1 = g1 - t1 * vec_per_row;
    const T* x0 = in + (int64_t)t0 * 2 * d + (int64_t)c0 * VN;
    const T* x1 = in + (int64_t)t1 * 2 * d + (int64_t)c1 * VN;
    const bool two = g1 < total;
    const uint4 a0 = ld_nc_16(x0), b0 = ld_nc_16(x0 + d);
    uint4 a1 = a0, b1 = b0;
    if (two) {
      a1 = ld_nc_16(x1);
      b1 = ld_nc_16(x1 + d);
    }
    st_16(out + (int64_t)t0 * d + (int64_t)c0 * VN, act_round_mul<T, Op>(a0, b0));
    if (two) st_16(out + (int64_t)t1 * d + (int64_t)c1 * VN, act_round_mul<T, Op>(a1, b1));
  }
}

template <typename T, typename Op>
__global__ void __launch_bounds__(256)
act_and_mul_generic_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t num_tokens, int d) {
  const int64_t total = num_tokens * d;
  Op op;
  for (int64_t g = (int64_t)blockIdx.x * 256 + threadIdx.x; g < total; g += (int64_t)gridDim.x * 256) {
    const int64_t t = g / d;
    const int i = (int)(g - t * d);
    const float x = to_f32<T>(in[t * 2 * (int64_t)d + i]);
    const float y = to_f32<T>(in[t * 2 * (int64_t)d + d + i]);
    out[g] = from_f32<T>(to_f32<T>(from_f32<T>(op(x))) * y);
  }
}

template <typename T, typename Op>
int launch_act_and_mul(void* out, const void* in, int64_t num_tokens, int d, cudaStream_t stream) {
  constexpr int VN = 16 / sizeof(T);
  const int sms = sm_count();
  const bool vec_ok = (d % VN == 0) && aligned16(out) && aligned16(in);
  if (vec_ok) {
    const int64_t total = num_tokens * (d / VN);
    const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((total + 511) / 512, (int64_t)sms * 16));
    if (total + 2 * (int64_t)grid * 256 < (int64_t)1 << 31)
      act_and_mul_vec_kernel<T, Op, int><<<grid, 256, 0, stream>>>((T*)out, (const T*)in, num_tokens, d);
    else
      act_and_mul_vec_kernel<T, Op, int64_t><<<grid, 256, 0, stream>>>((T*)out, (const T*)in, num_tokens, d);
  } else {
    const int64_t total = num_tokens * d;
    const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((total + 255) / 256, (int64_t)sms * 16));
    act_and_mul_generic_kernel<T, Op><<<grid, 256, 0, stream>>>((T*)out, (const T*)in, num_tokens, d);
  }
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

// ---------------------------------------------------------------------------
// Online rotary embedding (NeoX pairing: element i rotates with element i + D/2),
// csrc/pos_encoding.cu:83-111.  One warp per token (grid-stride); the D/2 angles
// are evaluated once per token, then every head is rotated with 16-byte accesses.
// Angles: the reference computes pos / __powf(theta, 2i/D) and __sincosf of it in
// fp32 (it is built with --use_fast_math, as this library is); at positions of
// several thousand radians an fp32 angle alone is off by 5e-4.  Here the inverse
// frequencies are evaluated once per thread in fp64 (fast-math does not touch
// double precision), the angle pos * inv_freq and its reduction to [-pi, pi] are
// fp64 too, and only the reduced angle goes through the fp32 sine / cosine
// intrinsics, which are accurate to ~5e-7 on that range.
// ---------------------------------------------------------------------------
template <typename T, int HEAD_DIM>
__global__ void __launch_bounds__(256)
rotary_online_kernel(const int32_t* __restrict__ positions, T* __restrict__ query, T* __restrict__ key,
                     int64_t num_tokens, int heads, int kv_heads, int64_t q_stride, int64_t k_stride,
                     float theta, int vec_ok) {
  // One WARP per token: its D/2 angles go to a warp-private slice of shared memory (no block-wide barrier),
  // then the warp rotates every query and key head of the token.
  constexpr int HALF = HEAD_DIM / 2;
  constexpr int VN = 16 / sizeof(T);
  constexpr int WARPS = 256 / 32;
  __shared__ float s_cos_all[WARPS][HALF];
  __shared__ float s_sin_all[WARPS][HALF];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  float* s_cos = s_cos_all[wib];
  float* s_sin = s_sin_all[wib];
  const int64_t warp_global = (int64_t)blockIdx.x * WARPS + wib;
  const int64_t warp_count = (int64_t)gridDim.x * WARPS;
  // inverse frequencies theta^(-2i/D) of the elements this lane evaluates (i = lane, lane + 32, ...), in fp64
  constexpr int PER_LANE = HALF / 32;
  double inv_freq[PER_LANE];
  {
    const double l2t = log2((double)theta);
#pragma unroll
    for (int t = 0; t < PER_LANE; ++t) inv_freq[t] = exp2(-(double)(2 * (lane + 32 * t)) / (double)HEAD_DIM * l2t);
  }
  constexpr double kTwoPi = 6.283185307179586476925286766559, kInvTwoPi = 0.15915494309189533576888376337251;
  for (int64_t tok = warp_global; tok < num_tokens; tok += warp_count) {
    const double pos = (double)positions[tok];
    __syncwarp();
#pragma unroll
    for (int t = 0; t < PER_LANE; ++t) {
      const double ang = pos * inv_freq[t];
      const float r = (float)fma(-kTwoPi, rint(ang * kInvTwoPi), ang);   // in [-pi, pi]
      s_sin[lane + 32 * t] = __sinf(r);
      s_cos[lane + 32 * t] = __cosf(r);
    }
    __syncwarp();
    if (vec_ok) {
      constexpr int VPH = HALF / VN;  // vectors per half head
      const int total = (heads + kv_heads) * VPH;
      // U element pairs per lane and step: all 2 * U 16-byte loads are issued before the first store, so that a
      // warp keeps 4 KB in flight (with one pair per step the kernel was bound by load latency at ~70 % of the
      // copy rate)
      constexpr int U = 4;
      for (int g0 = lane; g0 < total; g0 += 32 * U) {
        T* base[U];
        int col[U];
        uint4 rx[U], ry[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int g = g0 + 32 * u;
          if (g < total) {
            const int head = g / VPH;
            col[u] = (g - head * VPH) * VN;
            base[u] = (head < heads) ? query + tok * q_stride + (int64_t)head * HEAD_DIM
                                     : key + tok * k_stride + (int64_t)(head - heads) * HEAD_DIM;
            rx[u] = ld_16(base[u] + col[u]);
            ry[u] = ld_16(base[u] + HALF + col[u]);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (g0 + 32 * u < total) {
            const int c = col[u];
            float x[VN], y[VN], ox[VN], oy[VN];
            unpack16<T>(rx[u], x);
            unpack16<T>(ry[u], y);
#pragma unroll
            for (int i = 0; i < VN; ++i) {
              const float cs = s_cos[c + i], sn = s_sin[c + i];
              ox[i] = x[i] * cs - y[i] * sn;
              oy[i] = y[i] * cs + x[i] * sn;
            }
            st_16(base[u] + c, pack16<T>(ox));
            st_16(base[u] + HALF + c, pack16<T>(oy));
          }
        }
      }
    } else {
      const int total = (heads + kv_heads) * HALF;
      for (int g = lane; g < total; g += 32) {
        const int head = g / HALF;
        const int c = g - head * HALF;
        T* base = (head < heads) ? query + tok * q_stride + (int64_t)head * HEAD_DIM
                                 : key + tok * k_stride + (int64_t)(head - heads) * HEAD_DIM;
        const float x = to_f32<T>(base[c]), y = to_f32<T>(base[HALF + c]);
        const float cs = s_cos[c], sn = s_sin[c];
        base[c] = from_f32<T>(x * cs - y * sn);
        base[HALF + c] = from_f32<T>(y * cs + x * sn);
      }
    }
  }
}

template <typename T>
int launch_rotary(const int32_t* positions, void* query, void* key, int64_t num_tokens, int heads, int kv_heads,
                  int head_dim, int64_t q_stride, int64_t k_stride, float theta, cudaStream_t stream) {
  constexpr int VN = 16 / sizeof(T);
  const int vec_ok = aligned16(query) && aligned16(key) && (q_stride % VN == 0) && (k_stride % VN == 0) &&
                     ((head_dim / 2) % VN == 0);
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((num_tokens + 7) / 8, (int64_t)sm_count() * 8));
  T* q = (T*)query;
  T* k = (T*)key;
  switch (head_dim) {
    case 64:
      rotary_online_kernel<T, 64><<<grid, 256, 0, stream>>>(positions, q, k, num_tokens, heads, kv_heads, q_stride,
                                                            k_stride, theta, vec_ok);
      break;
    case 128:
      rotary_online_kernel<T, 128><<<grid, 256, 0, stream>>>(positions, q, k, num_tokens, heads, kv_heads, q_stride,
                                                             k_stride, theta, vec_ok);
      break;
    case 256:
      rotary_online_kernel<T, 256><<<grid, 256, 0, stream>>>(positions, q, k, num_tokens, heads, kv_heads, q_stride,
                                                             k_stride, theta, vec_ok);
      break;
    default:
      return B200_ERR_UNSUPPORTED;
  }
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

}  // namespace b200
