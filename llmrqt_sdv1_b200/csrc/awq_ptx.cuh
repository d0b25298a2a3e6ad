// mbarrier and bulk-copy (TMA) PTX wrappers shared by the GEMV and GEMM kernels.
#pragma once
#include <stdint.h>

namespace awq {

constexpr unsigned long long kWaitLimitCycles = 4000000000ull;  // ~2 s at 2 GHz
#ifndef AWQ_WAIT_HINT_NS
#define AWQ_WAIT_HINT_NS 2000u   // suspend-time hint of a blocked mbarrier wait
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same with a suspend-time hint (nanoseconds): the warp may sleep in hardware until the phase
// completes or the hint runs out, instead of coming back to spin and take issue slots from the warps
// that have work.
__device__ __forceinline__ bool mbar_try_wait_sleep(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and raises *abort_flag) if the phase did not
// complete in time or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = clock64();
  unsigned spins = 0;
  while (true) {
    if (mbar_try_wait_sleep(bar, parity, AWQ_WAIT_HINT_NS)) return true;
#ifdef AWQ_WAIT_NANOSLEEP
    __nanosleep(AWQ_WAIT_NANOSLEEP);
#endif
    if ((++spins & 63u) == 0u) {
      if (*abort_flag != 0) return false;
      if (clock64() - t0 > kWaitLimitCycles) {
        atomicCAS(const_cast<int*>(abort_flag), 0, code);
        return false;
      }
    }
  }
}
// Wait bounded by time only (used to let outstanding copies land after a failure).
__device__ __forceinline__ bool mbar_wait_timed(uint32_t bar, uint32_t parity) {
  const unsigned long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > kWaitLimitCycles) return false;
  }
  return true;
}
// Untiled bulk copy global -> shared; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

}  // namespace awq
