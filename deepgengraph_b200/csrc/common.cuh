// Shared device helpers for the sm_100a kernels: mbarrier with bounded waits,
// TMA tile loads, tcgen05 (TMEM alloc / MMA / ld / st) wrappers and the UMMA
// descriptor encoders.  Everything here is inline PTX for sm_100a.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "../../include/b200attn.h"

namespace b200 {

// ---------------------------------------------------------------------------
// host-side error plumbing
// ---------------------------------------------------------------------------
// The library is built as ONE translation unit (b200attn.cu includes every .cuh), so the
// globals below are plain definitions.
inline thread_local int g_last_cuda_error = 0;

#define B200_CUDA_TRY(expr)                          \
  do {                                               \
    cudaError_t _e = (expr);                         \
    if (_e != cudaSuccess) {                         \
      ::b200::g_last_cuda_error = (int)_e;           \
      (void)cudaGetLastError();                      \
      return B200_ERR_CUDA;                          \
    }                                                \
  } while (0)

// Device status word (one per device, lives in the library image).  Kernels
// record the first expired wait here instead of spinning forever.
__device__ int g_device_status = 0;

// Optional phase timeline for kernel tuning (compiled in with -DB200_TIMELINE only): selected threads of one
// CTA stamp clock64() into a caller-provided buffer.
#ifdef B200_TIMELINE
__device__ long long* g_timeline = nullptr;
__device__ int g_timeline_block = 0;
__device__ long long* g_cta_times = nullptr;   // [num CTAs][8]: start ns, end ns, SM id, key blocks, SM clocks
constexpr int kTimelineSlots = 2048;
__shared__ unsigned int s_timeline[kTimelineSlots];   // stamps stay in shared memory until the CTA ends
__device__ __forceinline__ unsigned int clock32() {
  unsigned int c;
  asm volatile("mov.u32 %0, %%clock;" : "=r"(c));
  return c;
}
#define B200_TL_INIT()                                                               \
  do {                                                                               \
    for (int _i = threadIdx.x; _i < kTimelineSlots; _i += blockDim.x) s_timeline[_i] = 0; \
    __syncthreads();                                                                 \
  } while (0)
#define B200_TL(slot) do { s_timeline[(slot)] = clock32(); } while (0)
#define B200_TL_FLUSH()                                                                                  \
  do {                                                                                                   \
    if (g_timeline != nullptr &&                                                                         \
        (int)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z)) == g_timeline_block)        \
      for (int _i = threadIdx.x; _i < kTimelineSlots; _i += blockDim.x) g_timeline[_i] = s_timeline[_i];  \
  } while (0)
#define B200_TL_CTA(start_ns, start_clk, nblocks)                                                              \
  do {                                                                                              \
    if (g_cta_times != nullptr && threadIdx.x == 0) {                                               \
      const long long _id = blockIdx.x + gridDim.x * (blockIdx.y + (long long)gridDim.y * blockIdx.z); \
      unsigned _sm;                                                                                 \
      asm volatile("mov.u32 %0, %%smid;" : "=r"(_sm));                                              \
      g_cta_times[_id * 8 + 0] = (long long)(start_ns);                                             \
      g_cta_times[_id * 8 + 1] = (long long)global_timer_ns();                                      \
      g_cta_times[_id * 8 + 2] = _sm;                                                               \
      g_cta_times[_id * 8 + 3] = (nblocks);                                                         \
      g_cta_times[_id * 8 + 4] = clock64() - (long long)(start_clk);                                \
    }                                                                                               \
  } while (0)
#else
#define B200_TL_CTA(start_ns, start_clk, nblocks) do { } while (0)
#define B200_TL_INIT() do { } while (0)
#define B200_TL(slot) do { } while (0)
#define B200_TL_FLUSH() do { } while (0)
#endif

// codes stored in the low byte of the status word
enum WaitCode : int {
  WAIT_Q_FULL = 1,
  WAIT_K_FULL = 2,
  WAIT_V_FULL = 3,
  WAIT_K_EMPTY = 4,
  WAIT_V_EMPTY = 5,
  WAIT_S_FULL = 6,
  WAIT_P_FULL = 7,
  WAIT_O_FULL = 8,
  WAIT_X_FULL = 9,    // streamed operand of the score sweeps
  WAIT_X_EMPTY = 10,
  WAIT_T_FULL = 11,   // TMEM tile of the score sweeps
  WAIT_T_EMPTY = 12,
  WAIT_N_FULL = 13,   // noise tile
  WAIT_N_EMPTY = 14,
  WAIT_DRAIN = 15,
  WAIT_TURN = 16,     // exp-phase turn-taking between the two query tiles
  WAIT_SELFTEST = 17, // b200_selftest_bounded_wait
  WAIT_SCHED = 18,    // persistent attention: next tile descriptor
  WAIT_Q_FREE = 19    // persistent attention: Q buffer released by the previous tile
};

// ---------------------------------------------------------------------------
// small PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// One lane of a converged warp.  Role loops run on ALL lanes (warp-uniform control flow keeps their address and
// descriptor arithmetic on the uniform datapath) and only the instruction that must be issued once is guarded.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  // make the initialised barriers visible to the async proxy (TMA, tcgen05.commit)
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// 32-byte global store (one full sector per lane; the address must be 32-byte aligned)
__device__ __forceinline__ void st_global_v8(void* ptr, const uint32_t (&w)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(w[0]), "r"(w[1]), "r"(w[2]),
               "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}

// Non-blocking probe (try_wait may suspend the thread for a while when the phase is still open).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  `abort_flag` is a CTA-shared word: once any thread of the CTA
// has given up, every other wait of that CTA returns false quickly, so that all
// roles fall through to the common tear-down (TMEM is always released).
// Limit: 2 s of wall time -- three orders of magnitude above any legitimate wait.
constexpr uint64_t kWaitLimitNs = 2000000000ull;

__device__ __forceinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                            int code, uint64_t limit_ns = kWaitLimitNs) {
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0xff) == 0) {
      if (*abort_flag != 0) return false;
      if (global_timer_ns() - t0 > limit_ns) {
        *abort_flag = code;
        atomicCAS(&g_device_status, 0, code | (int)((blockIdx.x & 0xffffff) << 8));
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, code);
}

// ---------------------------------------------------------------------------
// TMA (tiled bulk tensor copies, global -> shared, completion on an mbarrier)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05: tensor memory management
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {  // whole warp
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// arrive on `bar` once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ---------------------------------------------------------------------------
// UMMA descriptors
// ---------------------------------------------------------------------------
// Shared-memory matrix descriptor (64 bit) for a 128-byte-swizzled tile:
//   [0,14)  start address >> 4      [16,30) leading byte offset >> 4
//   [32,46) stride byte offset >> 4 [46,48) version = 1 (sm_100)
//   [61,64) layout type, 2 = SWIZZLE_128B
// K-major operand (rows of 64 16-bit elements = 128 B, 8-row groups 1024 B apart):
//   SBO = 1024, LBO unused (1).  Advancing K by 16 elements = +32 B on the start address.
// MN-major operand (rows along K, 64 contiguous MN elements per 128 B row):
//   SBO = 1024 (next 8 K rows), LBO = bytes between 64-wide MN column blocks.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fff);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// The same descriptor split into its two 32-bit halves, so that an MMA issuer can keep the constant upper
// half in a register and step the start address with a single 32-bit add (shared memory is < 256 KB, so
// (address >> 4) + offset never carries out of the 14-bit field).
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
  return ((saddr >> 4) & 0x3fff) | (((lbo_bytes >> 4) & 0x3fff) << 16);
}
__host__ __device__ constexpr uint32_t smem_desc_hi(uint32_t sbo_bytes) {
  return ((sbo_bytes >> 4) & 0x3fff) | (1u << 14) | (2u << 29);
}
__device__ __forceinline__ uint64_t desc_from_halves(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// Instruction descriptor for kind::f16 (fp16/bf16 inputs, fp32 accumulate):
//   [4,6) D format (1 = f32)  [7,10) A format  [10,13) B format (0 = f16, 1 = bf16)
//   [15] A major  [16] B major (0 = K, 1 = MN)  [17,23) N >> 3  [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc(bool bf16, int m, int n, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((a_mn_major ? 1u : 0u) << 15) |
         ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same with the accumulate flag and the instruction descriptor as compile-time constants (the predicate folds
// away: an MMA issuer is a single thread, every instruction it does not execute is latency off the chain).
template <uint32_t IDESC, int ACC>
__device__ __forceinline__ void umma_ss_c(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "n"(IDESC), "n"(ACC)
      : "memory");
}
template <uint32_t IDESC, int ACC>
__device__ __forceinline__ void umma_ts_c(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t desc_hi) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(desc_hi), "n"(IDESC), "n"(ACC)
      : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05.ld / st, shape 32x32b: thread t of warp w touches TMEM lane 32*(w%4)+t,
// register r <-> column (base + r).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
        "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
        "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------
// math helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// three-input maximum and packed two-wide fp32 arithmetic (sm_100): halve the issue slots of the softmax
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)), "l"(reinterpret_cast<uint64_t&>(c)));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)));
  return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  float2 d;
  asm("mul.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)));
  return d;
}
// Soft-cap tanh (kernels/gemma2.py:30-34 caps the logits with cap * tanh(s / cap)), y = s / cap:
//   |y| <= 1 -- every logit up to the cap itself -- : y * r(y^2), r an own degree-4 minimax fit of tanh(y) / y
//              (max relative error 7e-6, seventy times tighter than tanh.approx), on the FMA pipe;
//   |y| >  1 : tanh.approx.
// The choice depends on the element's own value only, so the forward kernel and the score sweeps, which visit the
// elements in different groupings, evaluate the same function on the same element; callers vote per block whether
// any lane holds an element of the second kind and otherwise never issue the special-function instruction (the
// exponentials already load that unit: a tanh.approx per element doubled its work).
constexpr float kCapPolyMax = 1.0f;
constexpr float kCapR0 = 0.999993085861206f, kCapR1 = -0.332980751991272f, kCapR2 = 0.1303686499595642f,
                kCapR3 = -0.04481850564479828f, kCapR4 = 0.009036950767040253f;
// r(y^2) * mul for two elements (mul folds the factor that follows the tanh into the polynomial)
__device__ __forceinline__ float2 softcap_r2(float2 y, float mul) {
  const float2 q = fmul2(y, y);
  float2 r = ffma2(q, make_float2(kCapR4 * mul, kCapR4 * mul), make_float2(kCapR3 * mul, kCapR3 * mul));
  r = ffma2(r, q, make_float2(kCapR2 * mul, kCapR2 * mul));
  r = ffma2(r, q, make_float2(kCapR1 * mul, kCapR1 * mul));
  r = ffma2(r, q, make_float2(kCapR0 * mul, kCapR0 * mul));
  return r;
}
// the full function for one element (both branches evaluated, selected by |y|)
__device__ __forceinline__ float softcap_tanh(float y) {
  const float q = y * y;
  float r = fmaf(q, kCapR4, kCapR3);
  r = fmaf(r, q, kCapR2);
  r = fmaf(r, q, kCapR1);
  r = fmaf(r, q, kCapR0);
  return fabsf(y) <= kCapPolyMax ? y * r : tanh_approx(y);
}

// warp vote over a 32-column chunk of raw logits: true when every lane's |raw * cap_in| stays <= 1
__device__ __forceinline__ bool softcap_chunk_poly_only(const uint32_t (&sr)[32], float cap_in) {
  float a0 = 0.f, a1 = 0.f;
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    a0 = fmax3(a0, fabsf(__uint_as_float(sr[i])), fabsf(__uint_as_float(sr[i + 1])));
    a1 = fmax3(a1, fabsf(__uint_as_float(sr[i + 2])), fabsf(__uint_as_float(sr[i + 3])));
  }
  return !__any_sync(0xffffffffu, fmaxf(a0, a1) * cap_in > kCapPolyMax);
}
// sv <- cap_out * softcap_tanh(sv * cap_in) for four raw logits (poly_only is warp-uniform)
__device__ __forceinline__ void softcap4(float (&sv)[4], float cap_in, float cap_out, bool poly_only) {
  if (poly_only) {
    const float2 a2 = make_float2(cap_in, cap_in);
    const float2 y0 = fmul2(make_float2(sv[0], sv[1]), a2), y1 = fmul2(make_float2(sv[2], sv[3]), a2);
    const float2 t0 = fmul2(y0, softcap_r2(y0, cap_out)), t1 = fmul2(y1, softcap_r2(y1, cap_out));
    sv[0] = t0.x, sv[1] = t0.y, sv[2] = t1.x, sv[3] = t1.y;
  } else {
#pragma unroll
    for (int u = 0; u < 4; ++u) sv[u] = softcap_tanh(sv[u] * cap_in) * cap_out;
  }
}

// warp-group register re-allocation (all 128 threads of an aligned group of four warps execute it)
template <int N>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// ---------------------------------------------------------------------------
// host helpers
// ---------------------------------------------------------------------------
inline int sm_count() {
  static thread_local int cached_dev = -1, cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached = n;
    cached_dev = dev;
  }
  return cached;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---------------------------------------------------------------------------
// host: TMA descriptor encoding through the driver entry point (no -lcuda needed)
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_tiled();

// BSHD tensor [batch, seq, heads, dim] of 16-bit elements, box = (64 dims, 1 head, box_rows rows, 1 batch),
// 128-byte swizzle.  Returns a b200_status.
int make_bshd_tensor_map(CUtensorMap* map, const void* base, int batch, int seq, int heads, int dim, int box_rows,
                         bool bf16, int64_t token_stride = 0, int64_t batch_stride = 0);
// Row-major float32 matrix [rows, cols], box = (box_cols, box_rows); swizzle128 selects the 128-byte swizzle
// (box_cols must then be 32).
int make_f32_matrix_tensor_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int box_rows,
                               int box_cols, bool swizzle128);

}  // namespace b200
