// mbarrier helpers shared by the kernels that wait on TMA copies and tensor-core commits.
//
// No wait in this package spins for ever: mbar_wait polls a bounded number of times and returns false when it
// gave up.  The kernel then raises JLX_STATUS_WAIT_TIMEOUT in the status word, lets its copies in flight land
// (bounded again), frees any tensor memory it holds and returns; the host reads the status word after the step.
#pragma once
#include <stdint.h>

#ifndef JLX_WAIT_LIMIT
#define JLX_WAIT_LIMIT (1u << 22)  // polls; each poll itself waits a bounded time in hardware
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: false after `limit` polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit = JLX_WAIT_LIMIT) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// The same for a wait that is expected to be long: the warp sleeps between polls, so that waiting warps do not
// compete for issue slots, or for power, with the warps that work.
__device__ __forceinline__ bool mbar_wait_long(uint32_t bar, uint32_t parity, uint32_t limit = JLX_WAIT_LIMIT) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    __nanosleep(128);
  }
  return false;
}
