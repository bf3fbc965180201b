// C ABI of the library (declared in include/b200attn.h).  The whole library is this one
// translation unit: the kernels live in the .cuh files included below.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "elementwise.cuh"
#include "attn_fwd.cuh"
#include "attn_fwd_persist.cuh"
#include "attn_sweep.cuh"
#include "kv_evict.cuh"

namespace b200 {

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// token_stride / batch_stride in elements; 0 = contiguous [batch, seq, heads, dim]
int make_bshd_tensor_map(CUtensorMap* map, const void* base, int batch, int seq, int heads, int dim, int box_rows,
                         bool bf16, int64_t token_stride, int64_t batch_stride) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return B200_ERR_CUDA;
  if (token_stride == 0) token_stride = (int64_t)heads * dim;
  if (batch_stride == 0) batch_stride = (int64_t)seq * token_stride;
  const cuuint64_t dims[4] = {(cuuint64_t)dim, (cuuint64_t)heads, (cuuint64_t)seq, (cuuint64_t)batch};
  const cuuint64_t strides[3] = {(cuuint64_t)dim * 2, (cuuint64_t)token_stride * 2, (cuuint64_t)batch_stride * 2};
  const cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                         const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = (int)r;
    return B200_ERR_CUDA;
  }
  return B200_OK;
}

int make_f32_matrix_tensor_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int box_rows,
                               int box_cols, bool swizzle128) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return B200_ERR_CUDA;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 4};
  const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE,
                         swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = (int)r;
    return B200_ERR_CUDA;
  }
  return B200_OK;
}

// Self-test of the bounded-wait machinery: one warp waits on an mbarrier that nobody ever arrives on.  The wait
// gives up after `limit_ns`, records WAIT_SELFTEST in the device status word and the kernel ends normally.
__global__ void bounded_wait_selftest_kernel(uint64_t limit_ns, int* gave_up) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const bool ok = mbar_try_wait(&bar, 0) || mbar_wait_slow(&bar, 0, &abort_flag, WAIT_SELFTEST, limit_ns);
  if (threadIdx.x == 0 && gave_up != nullptr) *gave_up = ok ? 0 : 1;
}

// ---------------------------------------------------------------------------------------------
// Built-in scratch of b200_attn_score_static: a fixed array in the library's device image, so that callers
// which must not allocate device memory still have somewhere to put the row normalisers and partial sums.
// In host code the array's NAME is only a stand-in for the symbol, not a device address; the address is looked
// up once per device (with that device current) through cudaGetSymbolAddress and cached.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_score_scratch[kStaticScoreScratchBytes];

int static_score_scratch(void** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static void* cached[kMaxDevices] = {};
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return B200_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    B200_CUDA_TRY(cudaGetSymbolAddress(&p, g_score_scratch));
    if (p == nullptr) return B200_ERR_CUDA;
    cached[dev] = p;
  }
  *out = cached[dev];
  return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" {

const char* b200_status_string(int status) {
  switch (status) {
    case B200_OK: return "ok";
    case B200_ERR_BAD_ARGUMENT: return "bad argument";
    case B200_ERR_BAD_DTYPE: return "unsupported dtype";
    case B200_ERR_MISALIGNED: return "misaligned pointer or stride";
    case B200_ERR_UNSUPPORTED: return "unsupported shape";
    case B200_ERR_WORKSPACE: return "workspace missing or too small";
    case B200_ERR_CUDA: return "CUDA call failed";
    case B200_ERR_DEVICE_TIMEOUT: return "device-side wait expired";
    default: return "unknown status";
  }
}

int b200_last_cuda_error(void) { return g_last_cuda_error; }

int b200_abi_version(void) { return 2; }

int b200_device_status(int* status_out) {
  if (!status_out) return B200_ERR_BAD_ARGUMENT;
  int word = 0;
  B200_CUDA_TRY(cudaDeviceSynchronize());
  B200_CUDA_TRY(cudaMemcpyFromSymbol(&word, g_device_status, sizeof(int)));
  if (word != 0) {
    const int zero = 0;
    B200_CUDA_TRY(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)));
    // a launch that gave up may have left its tile counters mid-count
    void* counters = nullptr;
    B200_CUDA_TRY(cudaGetSymbolAddress(&counters, g_sched_counters));
    B200_CUDA_TRY(cudaMemset(counters, 0, sizeof(unsigned int) * kSchedPool * 2));
  }
  *status_out = word;
  return word == 0 ? B200_OK : B200_ERR_DEVICE_TIMEOUT;
}

int b200_selftest_bounded_wait(int limit_ms, int* gave_up_device, void* stream) {
  if (limit_ms <= 0 || limit_ms > 1000) return B200_ERR_BAD_ARGUMENT;
  bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((uint64_t)limit_ms * 1000000ull, gave_up_device);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

int b200_rms_norm(void* out, const void* input, const void* weight, float epsilon, int64_t num_tokens,
                  int hidden_size, int dtype, void* stream) {
  if (!out || !input || !weight || num_tokens < 0 || hidden_size <= 0) return B200_ERR_BAD_ARGUMENT;
  if (num_tokens == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  void* in = const_cast<void*>(input);
  switch (dtype) {
    case B200_F32: return launch_rms_norm<float, false>(out, in, nullptr, weight, epsilon, num_tokens, hidden_size, s);
    case B200_F16: return launch_rms_norm<__half, false>(out, in, nullptr, weight, epsilon, num_tokens, hidden_size, s);
    case B200_BF16:
      return launch_rms_norm<__nv_bfloat16, false>(out, in, nullptr, weight, epsilon, num_tokens, hidden_size, s);
    default: return B200_ERR_BAD_DTYPE;
  }
}

int b200_fused_add_rms_norm(void* input, void* residual, const void* weight, float epsilon, int64_t num_tokens,
                            int hidden_size, int dtype, void* stream) {
  if (!input || !residual || !weight || num_tokens < 0 || hidden_size <= 0) return B200_ERR_BAD_ARGUMENT;
  if (num_tokens == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case B200_F32:
      return launch_rms_norm<float, true>(nullptr, input, residual, weight, epsilon, num_tokens, hidden_size, s);
    case B200_F16:
      return launch_rms_norm<__half, true>(nullptr, input, residual, weight, epsilon, num_tokens, hidden_size, s);
    case B200_BF16:
      return launch_rms_norm<__nv_bfloat16, true>(nullptr, input, residual, weight, epsilon, num_tokens, hidden_size,
                                                  s);
    default: return B200_ERR_BAD_DTYPE;
  }
}

int b200_silu_and_mul(void* out, const void* input, int64_t num_tokens, int d, int dtype, void* stream) {
  if (!out || !input || num_tokens < 0 || d <= 0) return B200_ERR_BAD_ARGUMENT;
  if (num_tokens == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case B200_F32: return launch_act_and_mul<float, SiluOp>(out, input, num_tokens, d, s);
    case B200_F16: return launch_act_and_mul<__half, SiluOp>(out, input, num_tokens, d, s);
    case B200_BF16: return launch_act_and_mul<__nv_bfloat16, SiluOp>(out, input, num_tokens, d, s);
    default: return B200_ERR_BAD_DTYPE;
  }
}

int b200_gelu_tanh_and_mul(void* out, const void* input, int64_t num_tokens, int d, int dtype, void* stream) {
  if (!out || !input || num_tokens < 0 || d <= 0) return B200_ERR_BAD_ARGUMENT;
  if (num_tokens == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case B200_F32: return launch_act_and_mul<float, GeluTanhOp>(out, input, num_tokens, d, s);
    case B200_F16: return launch_act_and_mul<__half, GeluTanhOpT<false>>(out, input, num_tokens, d, s);
    case B200_BF16: return launch_act_and_mul<__nv_bfloat16, GeluTanhOpT<false>>(out, input, num_tokens, d, s);
    default: return B200_ERR_BAD_DTYPE;
  }
}

int b200_rotary_embedding_online(const int32_t* positions, void* query, void* key, int64_t num_tokens, int heads,
                                 int kv_heads, int head_dim, int64_t query_stride, int64_t key_stride,
                                 float rope_theta, int dtype, void* stream) {
  if (!positions || !query || !key || num_tokens < 0 || heads <= 0 || kv_heads <= 0) return B200_ERR_BAD_ARGUMENT;
  if (query_stride < (int64_t)heads * head_dim || key_stride < (int64_t)kv_heads * head_dim)
    return B200_ERR_BAD_ARGUMENT;
  if (num_tokens == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case B200_F32:
      return launch_rotary<float>(positions, query, key, num_tokens, heads, kv_heads, head_dim, query_stride,
                                  key_stride, rope_theta, s);
    case B200_F16:
      return launch_rotary<__half>(positions, query, key, num_tokens, heads, kv_heads, head_dim, query_stride,
                                   key_stride, rope_theta, s);
    case B200_BF16:
      return launch_rotary<__nv_bfloat16>(positions, query, key, num_tokens, heads, kv_heads, head_dim, query_stride,
                                          key_stride, rope_theta, s);
    default: return B200_ERR_BAD_DTYPE;
  }
}

int b200_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int batch, int q_len,
                  int kv_len, int heads, int kv_heads, int head_dim, int dtype, int causal, int window,
                  float softcap, float scale, void* stream) {
  return attn_fwd_impl(q, k, v, out, lse, batch, q_len, kv_len, heads, kv_heads, head_dim, dtype, causal, window,
                       softcap, scale, (cudaStream_t)stream);
}

int b200_attn_fwd_strided(const void* q, const void* k, const void* v, void* out, float* lse, int batch, int q_len,
                          int kv_len, int heads, int kv_heads, int head_dim, int dtype, int64_t q_token_stride,
                          int64_t q_batch_stride, int64_t k_token_stride, int64_t k_batch_stride,
                          int64_t v_token_stride, int64_t v_batch_stride, int causal, int window, float softcap,
                          float scale, void* stream) {
  const int64_t st[6] = {q_token_stride, q_batch_stride, k_token_stride, k_batch_stride, v_token_stride, v_batch_stride};
  const int64_t row[6] = {(int64_t)heads * head_dim, 0, (int64_t)kv_heads * head_dim, 0, (int64_t)kv_heads * head_dim, 0};
  const int64_t len[6] = {0, q_len, 0, kv_len, 0, kv_len};
  for (int i = 0; i < 6; i += 2) {
    if (st[i] < row[i] || st[i + 1] < st[i] * len[i + 1]) return B200_ERR_BAD_ARGUMENT;   // overlapping rows / batches
    if (st[i] % 8 != 0 || st[i + 1] % 8 != 0) return B200_ERR_MISALIGNED;                 // TMA: 16-byte strides
  }
  AttnStrides strides{q_token_stride, q_batch_stride, k_token_stride, k_batch_stride, v_token_stride, v_batch_stride};
  return attn_fwd_impl_lse_stride(q, k, v, out, lse, q_len, batch, q_len, kv_len, heads, kv_heads, head_dim, dtype,
                                  causal, window, softcap, scale, (cudaStream_t)stream, &strides);
}

int64_t b200_attn_score_workspace_bytes(int batch, int q_len, int kv_len, int heads) {
  return score_workspace_bytes(batch, q_len, kv_len, heads);
}

int b200_attn_score(const void* q, const void* k, const void* v, void* out, float* score, float* score_sq,
                    void* workspace, int64_t workspace_bytes, int batch, int q_len, int kv_len, int heads,
                    int head_dim, int dtype, int causal, int window, float softcap, float scale, void* stream) {
  return attn_score_impl(q, k, v, out, score, score_sq, workspace, workspace_bytes, batch, q_len, kv_len, heads,
                         head_dim, dtype, causal, window, softcap, scale, (cudaStream_t)stream);
}

int b200_attn_corm(const void* q, const void* k, const void* v, void* out, float* score, uint8_t* corm_flags,
                   void* workspace, int64_t workspace_bytes, int batch, int q_len, int kv_len, int heads,
                   int head_dim, int dtype, int causal, float scale, void* stream) {
  if (!corm_flags) return B200_ERR_BAD_ARGUMENT;
  return attn_score_impl(q, k, v, out, score, nullptr, workspace, workspace_bytes, batch, q_len, kv_len, heads,
                         head_dim, dtype, causal, 0, 0.f, scale, (cudaStream_t)stream, corm_flags);
}

int b200_avg_pool1d_f32(const float* input, float* output, int64_t rows, int length, int kernel_size, void* stream) {
  if (!input || !output || rows < 0 || length <= 0 || kernel_size <= 0 || (kernel_size & 1) == 0)
    return B200_ERR_BAD_ARGUMENT;
  if (rows == 0) return B200_OK;
  if (rows > 65535) return B200_ERR_UNSUPPORTED;
  dim3 grid((length + 255) / 256, (unsigned)rows);
  avg_pool1d_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(input, output, rows, length, kernel_size);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

int b200_kv_evict_topk(const float* score, const void* k, const void* v, void* kv_cache, int32_t* indices,
                       int batch, int seq_len, int heads, int head_dim, int budget, int dtype, void* stream) {
  const int elem = dtype == B200_F32 ? 4 : (dtype == B200_F16 || dtype == B200_BF16) ? 2 : 0;
  if (elem == 0) return B200_ERR_BAD_DTYPE;
  return kv_evict_topk_impl(score, k, v, kv_cache, indices, batch, seq_len, heads, head_dim, budget, elem,
                            (cudaStream_t)stream);
}

int b200_attn_score_gqa(const void* q, const void* k, const void* v, void* out, float* score, float* score_sq,
                        uint8_t* corm_flags, void* workspace, int64_t workspace_bytes, int batch, int q_len,
                        int kv_len, int heads, int kv_heads, int head_dim, int dtype, int causal, int window,
                        float softcap, float scale, void* stream) {
  if (kv_heads <= 0) return B200_ERR_BAD_ARGUMENT;
  return attn_score_impl(q, k, v, out, score, score_sq, workspace, workspace_bytes, batch, q_len, kv_len, heads,
                         head_dim, dtype, causal, window, softcap, scale, (cudaStream_t)stream, corm_flags, kv_heads);
}

int b200_attn_kf_score_gqa(const void* q, const void* k, const void* v, const float* exp_rand, void* out,
                           float* kf_score, void* workspace, int64_t workspace_bytes, int batch, int q_len,
                           int kv_len, int heads, int kv_heads, int head_dim, int dtype, int causal, float tau,
                           float scale, void* stream) {
  if (kv_heads <= 0) return B200_ERR_BAD_ARGUMENT;
  return attn_kf_impl(q, k, v, exp_rand, out, kf_score, workspace, workspace_bytes, batch, q_len, kv_len, heads,
                      head_dim, dtype, causal, tau, scale, (cudaStream_t)stream, kv_heads);
}

int b200_kv_evict_roco(const float* score, const float* score_sq, const void* k, const void* v, void* kv_cache,
                       int32_t* indices, int batch, int seq_len, int heads, int head_dim, int q_len, int budget,
                       int recent, int dtype, void* stream) {
  const int elem = dtype == B200_F32 ? 4 : (dtype == B200_F16 || dtype == B200_BF16) ? 2 : 0;
  if (elem == 0) return B200_ERR_BAD_DTYPE;
  return kv_evict_roco_impl(score, score_sq, k, v, kv_cache, indices, batch, seq_len, heads, head_dim, q_len, budget,
                            recent, elem, (cudaStream_t)stream);
}

int b200_attn_kf_score(const void* q, const void* k, const void* v, const float* exp_rand, void* out,
                       float* kf_score, void* workspace, int64_t workspace_bytes, int batch, int q_len, int kv_len,
                       int heads, int head_dim, int dtype, int causal, float tau, float scale, void* stream) {
  return attn_kf_impl(q, k, v, exp_rand, out, kf_score, workspace, workspace_bytes, batch, q_len, kv_len, heads,
                      head_dim, dtype, causal, tau, scale, (cudaStream_t)stream);
}

int b200_attn_kf_score_seeded(const void* q, const void* k, const void* v, uint64_t seed, void* out, float* kf_score,
                              void* workspace, int64_t workspace_bytes, int batch, int q_len, int kv_len, int heads,
                              int kv_heads, int head_dim, int dtype, int causal, float tau, float scale, void* stream) {
  if (kv_heads <= 0) return B200_ERR_BAD_ARGUMENT;
  return attn_kf_impl(q, k, v, nullptr, out, kf_score, workspace, workspace_bytes, batch, q_len, kv_len, heads,
                      head_dim, dtype, causal, tau, scale, (cudaStream_t)stream, kv_heads, seed);
}

int b200_kf_noise_fill(float* exp_rand, uint64_t seed, int batch, int heads, int q_len, int kv_len, void* stream) {
  if (!exp_rand || batch < 0 || heads <= 0 || q_len < 0 || kv_len < 0) return B200_ERR_BAD_ARGUMENT;
  const int64_t rows = (int64_t)batch * heads * q_len;
  if (rows == 0 || kv_len == 0) return B200_OK;
  if ((int64_t)batch * heads > 0xffffffffll) return B200_ERR_UNSUPPORTED;
  const int64_t quads = rows * ((kv_len + 3) / 4);
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((quads + 255) / 256, (int64_t)sm_count() * 16));
  kf_noise_fill_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(exp_rand, rows, q_len, kv_len, (uint32_t)seed,
                                                               (uint32_t)(seed >> 32));
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

int b200_attn_score_static(const void* q, const void* k, const void* v, void* out, float* score, float* score_sq,
                           int batch, int q_len, int kv_len, int heads, int head_dim, int dtype, int causal,
                           int window, float softcap, float scale, void* stream) {
  const int64_t need = score_workspace_bytes(batch, q_len, kv_len, heads);
  if (need <= 0) return B200_ERR_BAD_ARGUMENT;
  if (need > kStaticScoreScratchBytes) return B200_ERR_WORKSPACE;   // problem too large for the built-in scratch
  void* scratch = nullptr;
  const int rc = static_score_scratch(&scratch);
  if (rc != B200_OK) return rc;
  return attn_score_impl(q, k, v, out, score, score_sq, scratch, kStaticScoreScratchBytes, batch, q_len, kv_len,
                         heads, head_dim, dtype, causal, window, softcap, scale, (cudaStream_t)stream);
}

#ifdef B200_TIMELINE
// tuning builds only: where selected threads of CTA `block` stamp their phase clocks
int b200_debug_set_timeline(void* buffer, int block) {
  long long* p = (long long*)buffer;
  B200_CUDA_TRY(cudaMemcpyToSymbol(g_timeline, &p, sizeof(p)));
  B200_CUDA_TRY(cudaMemcpyToSymbol(g_timeline_block, &block, sizeof(int)));
  return B200_OK;
}
int b200_debug_set_cta_times(void* buffer) {
  long long* p = (long long*)buffer;
  B200_CUDA_TRY(cudaMemcpyToSymbol(g_cta_times, &p, sizeof(p)));
  return B200_OK;
}
#endif

}  // extern "C"
