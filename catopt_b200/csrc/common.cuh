// Shared device helpers for the sm_100a executors: bf16 widening, the
// mbarrier / bulk-copy (TMA engine) PTX wrappers with bounded waits, and the
// launch-check macro used by every C-ABI entry point.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/catopt_b200.h"

namespace cb2 {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

// Upper bound on polls of one mbarrier phase before a kernel gives up.  Each
// failed try_wait already blocks for a hardware-chosen interval, so this is
// far beyond any legitimate copy latency while still ending in well under a
// second.
constexpr uint32_t kMaxBarrierPolls = 1u << 22;

#define CB2_LAUNCH_CHECK()                         \
  do {                                             \
    if (cudaGetLastError() != cudaSuccess) {       \
      return CB2_LAUNCH_FAIL;                      \
    }                                              \
  } while (0)

__host__ __device__ inline bool aligned16(const void* p) {
  return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

// ---- bf16 <-> fp32 --------------------------------------------------------
// A bf16 is the upper half of an fp32: widening is exact and is a shift/mask.
// 16-byte asynchronous copy global -> shared (bypasses L1 and the register file), commit / wait groups.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(uint32_t(__cvta_generic_to_shared(smem_dst))),
               "l"(gmem_src)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ float bf16lo_to_f32(uint32_t packed) {
  return __uint_as_float(packed << 16);
}
__device__ __forceinline__ float bf16hi_to_f32(uint32_t packed) {
  return __uint_as_float(packed & 0xffff0000u);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ float round_to_bf16(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

// ---- shared-memory addresses ---------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier -------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(count)
               : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar,
                                                      uint32_t bytes) {
  asm volatile(
      "mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
          smem_u32(bar)),
      "r"(bytes)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar))
               : "memory");
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
// Bounded wait: true when the phase completed, false when the poll budget ran
// out (the caller then records CB2_WAIT_TIMEOUT and leaves).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar,
                                                  uint32_t parity) {
  for (uint32_t i = 0; i < kMaxBarrierPolls; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

// Default budget of a wait inside a kernel: far beyond any legitimate latency, short enough that a
// protocol error shows up as a status word within seconds instead of a hung GPU.
constexpr unsigned long long kDefaultWaitNs = 4000000000ull;

// A wait's budget is counted on the SM's own cycle counter AND in polls: the wait gives up only
// when more than `budget_ns` x 2 cycles have passed (4 s at 2 GHz, 6 s at a power-capped 1.3 GHz
// for the default) and it has really polled that long (at least budget / 128 ns polls, capped at
// 2^20).  A wall-clock timer that the driver steps, or a stretch during which the context was not
// running, therefore cannot end a wait that would have been satisfied.
__device__ __forceinline__ long long sm_cycles() {
  long long c;
  asm volatile("mov.u64 %0, %%clock64;" : "=l"(c));
  return c;
}
struct WaitBudget {
  long long c0, cycles;
  uint32_t min_polls;
  __device__ __forceinline__ explicit WaitBudget(unsigned long long budget_ns)
      : c0(sm_cycles()), cycles((long long)(budget_ns * 2ull)),
        min_polls(budget_ns / 128ull > (1ull << 20) ? (1u << 20) : uint32_t(budget_ns / 128ull)) {}
  __device__ __forceinline__ bool spent(uint32_t polls) const {
    return polls >= min_polls && sm_cycles() - c0 > cycles;
  }
};

// Wait for kernels whose roles wait on one another: gives up when its budget is spent (see
// WaitBudget), or as soon as another role has raised `*abort` (so one expired wait ends the
// whole CTA quickly instead of cascading).  The wait that gives up leaves `site` (non-zero: a
// kernel may pass the source line, so that the host can say which wait it was) in `*abort`.
__device__ __forceinline__ bool mbar_wait_abortable(uint64_t* bar, uint32_t parity,
                                                    volatile int* abort,
                                                    uint64_t budget_ns = kDefaultWaitNs, int site = 1) {
  if (mbar_try_wait(bar, parity)) return true;
  const WaitBudget budget(budget_ns);
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 31u) == 0) {
      if (*abort) return false;
      if (budget.spent(i)) {
        *abort = site;
        return false;
      }
    }
  }
}

// Bounded wait for a flag in global memory that another CTA (or an earlier kernel) sets
// (acquire).  Gives up when its budget is spent, or as soon as a sibling thread has
// raised the shared `*abort` word; on expiry it raises `*abort` itself.  Never traps.
__device__ __forceinline__ bool wait_flag_abortable(const int* flag, volatile int* abort,
                                                    unsigned long long budget_ns = kDefaultWaitNs, int site = 1) {
  const WaitBudget budget(budget_ns);
  for (uint32_t it = 0;; ++it) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v != 0) return true;
    if (*abort) return false;
    if ((it & 63u) == 63u) {
      if (budget.spent(it)) { *abort = site; return false; }
      __nanosleep(200);
    }
  }
}

// ---- additive attention bias -------------------------------------------------
// fp32 bias added to the scaled scores of softmax attention (torch's attn_mask in its additive
// form, -inf = key hidden): element (b, h, t, j) at p[b sb + h sh + t sq + j], strides in
// elements, 0 for a broadcast axis; p == nullptr: no bias.
struct OmBias {
  const float* p;
  long long sb, sh, sq;
  int H;
};

// ---- bulk asynchronous copies (TMA engine, untiled form) -------------------
// global -> shared, completion counted in bytes on `bar`.  Both addresses must
// be 16-byte aligned and `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src,
                                         uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Wait until at most N of this thread's bulk groups still READ shared memory.
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Make generic-proxy writes to shared memory visible to the async proxy
// (required before a bulk store or an MMA reads what threads just wrote).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

}  // namespace cb2
