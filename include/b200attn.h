/*
 * b200attn.h -- C ABI of the B200 (sm_100a) fused attention core modules and
 * their companion bandwidth ops.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void*, may be NULL for the legacy default stream), enqueues its
 * kernels on that stream and returns without synchronising.  The return value
 * is a b200_status code (0 = success); nothing throws and no call allocates
 * device memory: scratch buffers are sized by the *_workspace_bytes queries and
 * supplied by the caller.  (The library image itself carries two fixed device
 * arrays per GPU that loads it: the 32 MiB scratch of b200_attn_score_static and
 * a small pool of scheduler counters.)
 *
 * Tensor layouts follow the reference project (DeepGenGroup/DeepGenGraph):
 *   q            [batch, q_len,  heads,    head_dim]   ("BSHD", contiguous)
 *   k, v         [batch, kv_len, kv_heads, head_dim]
 *   out          [batch, q_len,  heads,    head_dim]
 *   score vectors[batch, heads, kv_len]  float32
 *   exp_rand     [batch, heads, q_len, kv_len] float32
 */
#ifndef B200ATTN_H_
#define B200ATTN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of the 16/32-bit tensors */
enum b200_dtype { B200_F32 = 0, B200_F16 = 1, B200_BF16 = 2 };

enum b200_status {
  B200_OK = 0,
  B200_ERR_BAD_ARGUMENT = 1,   /* null pointer, non-positive size, unsupported head_dim ... */
  B200_ERR_BAD_DTYPE = 2,      /* dtype not supported by this entry point            */
  B200_ERR_MISALIGNED = 3,     /* pointer or stride not aligned as the kernel needs   */
  B200_ERR_UNSUPPORTED = 4,    /* shape outside what the kernels implement            */
  B200_ERR_WORKSPACE = 5,      /* workspace missing or too small                      */
  B200_ERR_CUDA = 6,           /* a CUDA runtime/driver call failed (see b200_last_cuda_error) */
  B200_ERR_DEVICE_TIMEOUT = 7  /* a bounded device-side wait expired (see b200_device_status)  */
};

/* Human-readable name of a status code. */
const char* b200_status_string(int status);
/* cudaError_t of the most recent failing CUDA call made by this library on the calling thread. */
int b200_last_cuda_error(void);
/* Library ABI version (bumped when a signature changes). */
int b200_abi_version(void);

/*
 * Reads (and clears) the device-side status word of the current device.
 * Kernels with bounded waits (mbarrier spins) record a non-zero code there and
 * exit cleanly instead of hanging; 0 means no wait ever expired.  This call
 * synchronises the device.  *status_out receives the raw word:
 * bits 0..7 = which wait expired, bits 8..31 = (blockIdx.x & 0xffffff).
 */
int b200_device_status(int* status_out);

/*
 * Self-test of the bounded device-side waits (no counterpart in the reference, which has no failure handling:
 * compile.py:207-212 swallows errors).  Launches one warp that waits on a barrier nobody signals; after
 * `limit_ms` (1..1000) the wait gives up, the kernel ends normally, *gave_up_device (device int, may be NULL)
 * becomes 1 and the device status word holds code 17, which the next b200_device_status call reports as
 * B200_ERR_DEVICE_TIMEOUT and clears.  The GPU stays fully usable: nothing traps and nothing hangs.
 */
int b200_selftest_bounded_wait(int limit_ms, int* gave_up_device, void* stream);

/* ------------------------------------------------------------------------- *
 * Bandwidth ops.  Replace the reference's csrc/ natives
 * (csrc/ffi.cpp:4-8, csrc/op.h:2-6).
 * ------------------------------------------------------------------------- */

/* out = T(x * rsqrt(mean(x^2) + eps)) * weight   -- replaces rms_norm, csrc/norm.cu:34-56,85-98 */
int b200_rms_norm(void* out, const void* input, const void* weight, float epsilon,
                  int64_t num_tokens, int hidden_size, int dtype, void* stream);

/* residual = T(input + residual); input = rms_norm(residual) * weight, both in place
 * -- replaces fused_add_rms_norm, csrc/norm.cu:59-83,100-113 */
int b200_fused_add_rms_norm(void* input, void* residual, const void* weight, float epsilon,
                            int64_t num_tokens, int hidden_size, int dtype, void* stream);

/* out[t, i] = T(silu(in[t, i])) * in[t, d + i]   -- replaces silu_and_mul, csrc/activation.cu:6-34 */
int b200_silu_and_mul(void* out, const void* input, int64_t num_tokens, int d, int dtype,
                      void* stream);

/* out[t, i] = T(gelu_tanh(in[t, i])) * in[t, d + i] -- GeGLU sibling of silu_and_mul (same
 * contract as csrc/activation.cu:6-34 with the tanh-approximated GELU as the gate). */
int b200_gelu_tanh_and_mul(void* out, const void* input, int64_t num_tokens, int d, int dtype,
                           void* stream);

/* In-place NeoX-style rotary embedding with on-the-fly frequencies
 * -- replaces rotary_embedding_online, csrc/pos_encoding.cu:64-113,180-199.
 * query [num_tokens, heads * head_dim] with row stride query_stride (elements),
 * key   [num_tokens, kv_heads * head_dim] with row stride key_stride,
 * positions int32 [num_tokens].  head_dim in {64, 128, 256}. */
int b200_rotary_embedding_online(const int32_t* positions, void* query, void* key,
                                 int64_t num_tokens, int heads, int kv_heads, int head_dim,
                                 int64_t query_stride, int64_t key_stride, float rope_theta,
                                 int dtype, void* stream);

/* ------------------------------------------------------------------------- *
 * Fused attention core modules.  Replace the kernels that the reference's
 * compiler generates for deepgengraph_exp/cases/kernels/{attn,gemma2,h2o,roco,kf}.py
 * (emitter: 3rd/deepgengraph/lib/Translate/to_triton.cpp:480-638).
 * ------------------------------------------------------------------------- */

/*
 * out = softmax(mask(softcap(q k^T * scale))) v
 *   -- Attn.forward   deepgengraph_exp/cases/kernels/attn.py:18-34
 *   -- Gemma2.forward deepgengraph_exp/cases/kernels/gemma2.py:19-38 (softcap > 0)
 * causal != 0 : key j visible to query i iff j <= i + (kv_len - q_len)
 * window  > 0 : additionally i + (kv_len - q_len) - j < window
 * softcap > 0 : logits <- softcap * tanh(logits / softcap) after scaling, before masking
 * heads % kv_heads == 0 (grouped-query attention); head_dim in {128, 256}; dtype f16 or bf16.
 * lse (optional, may be NULL): float32 [batch, heads, q_len], receives
 *   log2(sum_j exp(logit_ij)) (base-2 log-sum-exp of the scaled, capped, masked logits);
 *   the score passes below consume it.
 * The kernel is a persistent grid whose CTAs draw query tiles from a counter; every launch takes a counter pair
 * from a pool of 256 per GPU inside the library (returned to zero by the launch itself).  Launches in flight at
 * the same time therefore use different pairs unless more than 256 are outstanding; a launch captured into a
 * CUDA graph keeps the pair it drew at capture time.  The first call on a device looks up the pool's address
 * (cudaGetSymbolAddress) and sets the kernel's shared-memory attribute: make it before any stream capture.
 */
int b200_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse,
                  int batch, int q_len, int kv_len, int heads, int kv_heads, int head_dim,
                  int dtype, int causal, int window, float softcap, float scale, void* stream);

/*
 * b200_attn_fwd for q / k / v that are VIEWS into a larger buffer -- typically the [tokens, (heads + 2 kv_heads) *
 * head_dim] output of the fused QKV projection, rotated in place by b200_rotary_embedding_online.  Replaces the
 * split -> contiguous x 3 -> view sequence of the reference's model glue
 * (deepgengraph_exp/cases/models/attn.py:36-42, models/h2o.py / roco.py / kf.py likewise): no copy is made, the TMA
 * descriptors carry the strides.
 * *_token_stride: elements between consecutive tokens (>= heads * head_dim, resp. kv_heads * head_dim);
 * *_batch_stride: elements between batches (>= len * token stride).  Head h of a token starts h * head_dim
 * elements into the token's row.  All strides must be multiples of 8 elements (16 bytes); `out` is contiguous
 * [batch, q_len, heads, head_dim].
 */
int b200_attn_fwd_strided(const void* q, const void* k, const void* v, void* out, float* lse,
                          int batch, int q_len, int kv_len, int heads, int kv_heads, int head_dim, int dtype,
                          int64_t q_token_stride, int64_t q_batch_stride,
                          int64_t k_token_stride, int64_t k_batch_stride,
                          int64_t v_token_stride, int64_t v_batch_stride,
                          int causal, int window, float softcap, float scale, void* stream);

/* Bytes of scratch that b200_attn_score / b200_attn_kf_score need for these sizes. */
int64_t b200_attn_score_workspace_bytes(int batch, int q_len, int kv_len, int heads);

/*
 * Attention output plus per-key column sums of the fp32 softmax probabilities:
 *   score[b, h, j]    = sum_i p_ij          -- H2O.forward  kernels/h2o.py:35-38
 *   score_sq[b, h, j] = sum_i p_ij^2        -- RoCo.forward kernels/roco.py:42-48 (optional, may be NULL)
 * heads must equal kv_heads (the reference asserts group_size == 1, kernels/h2o.py:16).
 * workspace: at least b200_attn_score_workspace_bytes(...) bytes, 256-byte aligned.
 */
int b200_attn_score(const void* q, const void* k, const void* v, void* out, float* score,
                    float* score_sq, void* workspace, int64_t workspace_bytes, int batch,
                    int q_len, int kv_len, int heads, int head_dim, int dtype, int causal,
                    int window, float softcap, float scale, void* stream);

/*
 * b200_attn_score / b200_attn_corm for grouped-query attention (heads > kv_heads): every statistic is taken from
 * the probabilities AVERAGED over the heads / kv_heads query heads that share a K/V head
 *   pm_ij = mean_h p^h_ij;  score_j = sum_i pm_ij;  score_sq_j = sum_i pm_ij^2;  corm_j = any_i(pm_ij >= 1/(i+1))
 *   -- the group_size > 1 branches of kernels/roco.py:25-27,39-46 and figure/membound/attn.py:84-88,123-131,240-244
 *      (the modules under kernels/ assert group_size == 1; the ones under figure/membound run it).
 * k, v   [batch, kv_len, kv_heads, head_dim];  score, score_sq float32 and corm_flags uint8 [batch, kv_heads, kv_len].
 * score_sq and corm_flags are optional (NULL) and exclusive; corm_flags needs softcap == 0.
 * The workspace is sized for `heads` (b200_attn_score_workspace_bytes(batch, q_len, kv_len, heads)).
 */
int b200_attn_score_gqa(const void* q, const void* k, const void* v, void* out, float* score, float* score_sq,
                        uint8_t* corm_flags, void* workspace, int64_t workspace_bytes, int batch, int q_len,
                        int kv_len, int heads, int kv_heads, int head_dim, int dtype, int causal, int window,
                        float softcap, float scale, void* stream);

/*
 * b200_attn_score without a caller-provided workspace and without any device allocation.
 * (No counterpart in the reference project: its generated launchers allocate freely through PyTorch.)
 *
 * For callers that are not allowed to call cudaMalloc -- a plugin whose host forbids allocation after
 * start-up, code that runs where the allocator may not be entered, a process whose device memory is already
 * fully committed -- the library carries its own scratch: a fixed 32 MiB array in its
 * device image (every GPU that loads the library holds those 32 MiB until the process exits).  Inputs and
 * outputs are still the caller's.  Semantics and results are those of b200_attn_score.
 *
 *  - Limit: b200_attn_score_workspace_bytes(batch, q_len, kv_len, heads) must not exceed 33554432 bytes
 *    (batch 2 x 32 heads x seq 4096 needs 6 MiB, batch 8 needs 24 MiB); larger problems return
 *    B200_ERR_WORKSPACE and launch nothing.
 *  - The first call on each device looks up the scratch address (cudaGetSymbolAddress, with that device
 *    current) and caches it; make that first call outside of any stream capture.
 *  - All calls on a device share the one array, which keeps the previous call's contents.  Nothing in it has
 *    to start at zero (every element that is read is written earlier in the same call), but two calls that
 *    overlap on the GPU (for example on different streams) race on it: serialise them.
 *  - batch, q_len, kv_len and heads must be positive: an empty problem returns B200_ERR_BAD_ARGUMENT here
 *    (as it does at b200_attn_score) and launches nothing.
 */
int b200_attn_score_static(const void* q, const void* k, const void* v, void* out, float* score,
                           float* score_sq, int batch, int q_len, int kv_len, int heads, int head_dim,
                           int dtype, int causal, int window, float softcap, float scale, void* stream);

/*
 * Corm: attention output, the column sums `score` (workspace by-product, required) and
 *   corm_flags[b, h, j] = any_i( p_ij >= 1 / (i + 1) )     -- Corm.forward kernels/corm.py:35-37
 * uint8 [batch, heads, kv_len] (1 = true).  The reference passes the thresholds as a [q_len, kv_len] tensor
 * built by Corm.prepare (kernels/corm.py:47-49: row i holds 1 / (i + 1)); this entry point evaluates the same
 * thresholds in the kernel (tested as p * (i + 1) >= 1).
 */
int b200_attn_corm(const void* q, const void* k, const void* v, void* out, float* score,
                   uint8_t* corm_flags, void* workspace, int64_t workspace_bytes, int batch, int q_len,
                   int kv_len, int heads, int head_dim, int dtype, int causal, float scale, void* stream);

/*
 * out[r, j] = mean over the window of `kernel_size` (odd) centred on j of in[r, :], zero padded, divisor
 * kernel_size -- the pooling SnapKV applies to the column sums (kernels/snapkv.py:36-38:
 * F.avg_pool1d(kernel_size=5, padding=2, stride=1)).  float32 [rows, length].
 */
int b200_avg_pool1d_f32(const float* input, float* output, int64_t rows, int length, int kernel_size,
                        void* stream);

/*
 * KV-cache eviction after a score-producing variant: per (batch, head) keep the `budget` keys with the largest
 * score, in ascending key order, and gather their rows
 *   -- deepgengraph_exp/cases/models/h2o.py:51-57, models/kf.py:54-60 (topk -> sort -> gather -> cat).
 * score    float32 [batch, heads, seq_len]
 * k, v     [batch, seq_len, heads, head_dim]   (dtype gives the element size only)
 * kv_cache [batch, 2, budget, heads, head_dim] (plane 0 = keys, plane 1 = values)
 * indices  int32 [batch, heads, budget], optional (may be NULL): the selected key positions, ascending
 * Ties at the budget-th score keep the lower key index.  budget <= min(seq_len, 12288).
 */
int b200_kv_evict_topk(const float* score, const void* k, const void* v, void* kv_cache, int32_t* indices,
                       int batch, int seq_len, int heads, int head_dim, int budget, int dtype, void* stream);

/*
 * RoCo's KV-cache eviction -- deepgengraph_exp/cases/models/roco.py:52-66:
 *   std = sqrt(score_sq / q_len - (score / q_len)^2)                (fp32, the reference's operation order)
 *   A   = the `recent` keys with the largest std                    (roco.py:55, topk(std, largest=True))
 *   B   = among the other keys, the `budget` keys with the largest score / q_len   (roco.py:54,56-57)
 *   kv_cache = rows of A u B in ascending key order                 (roco.py:58-65)
 * score, score_sq  float32 [batch, heads, seq_len]  (column sums of p and p^2 from b200_attn_score)
 * k, v             [batch, seq_len, heads, head_dim]
 * kv_cache         [batch, 2, budget + recent, heads, head_dim]
 * indices          int32 [batch, heads, budget + recent], optional (may be NULL)
 * Ties keep the lower key index; a NaN std (variance rounded below zero) ranks highest, as in torch.topk.
 */
int b200_kv_evict_roco(const float* score, const float* score_sq, const void* k, const void* v, void* kv_cache,
                       int32_t* indices, int batch, int seq_len, int heads, int head_dim, int q_len, int budget,
                       int recent, int dtype, void* stream);

/*
 * KeyFormer: attention output plus
 *   kf_score[b, h, j] = sum_i softmax_j((logit_ij - log(exp_rand_ij)) / tau)
 *   -- KeyFormer.forward kernels/kf.py:19-42
 * exp_rand: float32 [batch, heads, q_len, kv_len], strictly positive.
 * kv_len must be a multiple of 4 (16-byte rows of exp_rand).
 */
int b200_attn_kf_score(const void* q, const void* k, const void* v, const float* exp_rand,
                       void* out, float* kf_score, void* workspace, int64_t workspace_bytes,
                       int batch, int q_len, int kv_len, int heads, int head_dim, int dtype,
                       int causal, float tau, float scale, void* stream);

/*
 * b200_attn_kf_score for grouped-query attention: exp_rand stays [batch, heads, q_len, kv_len] (one noise plane per
 * QUERY head), k, v are [batch, kv_len, kv_heads, head_dim], and kf_score float32 [batch, kv_heads, kv_len] is the
 * mean over the query heads of a K/V head of their column sums -- figure/membound/attn.py:162-165.
 */
int b200_attn_kf_score_gqa(const void* q, const void* k, const void* v, const float* exp_rand, void* out,
                           float* kf_score, void* workspace, int64_t workspace_bytes, int batch, int q_len,
                           int kv_len, int heads, int kv_heads, int head_dim, int dtype, int causal, float tau,
                           float scale, void* stream);

/*
 * KeyFormer with the noise generated inside the kernels instead of read from a [batch, heads, q_len, kv_len] tensor
 * (1.07 GB at batch 2 x 32 heads x seq 2048, 17 GB at seq 8192).  No counterpart in the reference, whose module takes
 * the tensor (kernels/kf.py:19,36-37) from the caller (kf.py:48, models/kf.py:44).
 * Element (b, h, i, j) comes from Philox4x32-10: counter (j >> 2, i, b * heads + h, 0), key (seed & 0xffffffff,
 * seed >> 32), output word j & 3; word r maps to u = ((r >> 9) + 1/2) * 2^-23 and exp_rand = -ln(u), so that
 * -ln(exp_rand) is a Gumbel(0, 1) variate.  b200_kf_noise_fill writes exactly that tensor (correctly rounded), so
 * b200_attn_kf_score[_gqa] on the filled tensor and this entry point agree to the accuracy of the kernels' log2.
 * kv_heads == heads or a divisor of it (scores are then the group mean, as in b200_attn_kf_score_gqa).
 */
int b200_attn_kf_score_seeded(const void* q, const void* k, const void* v, uint64_t seed, void* out, float* kf_score,
                              void* workspace, int64_t workspace_bytes, int batch, int q_len, int kv_len, int heads,
                              int kv_heads, int head_dim, int dtype, int causal, float tau, float scale, void* stream);

/* exp_rand float32 [batch, heads, q_len, kv_len] of the generator above (see b200_attn_kf_score_seeded). */
int b200_kf_noise_fill(float* exp_rand, uint64_t seed, int batch, int heads, int q_len, int kv_len, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200ATTN_H_ */
