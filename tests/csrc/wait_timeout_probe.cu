// Test-only kernel: makes one of the package's bounded waits run out, the allowed way.  It initialises an
// mbarrier that nothing ever arrives at, waits on it with the package's own mbar_wait (mbarrier.cuh) under a
// limit of a few thousand polls, raises JLX_STATUS_WAIT_TIMEOUT in the status word it was given, and returns.
// No copy is in flight, nothing is left waiting, and the context stays usable.
#include "common.cuh"
#include "mbarrier.cuh"

__global__ void wait_that_runs_out_kernel(int* status, unsigned limit, int* gave_up) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = mbar_wait(smem_u32(&bar), 0, limit);
    if (!ok) atomicOr(status, JLX_STATUS_WAIT_TIMEOUT);
    *gave_up = ok ? 0 : 1;
  }
}

JLX_API int jlx_test_wait_that_runs_out(int* status, unsigned limit, int* gave_up, cudaStream_t stream) {
  JLX_REQUIRE(status && gave_up, "wait probe: null pointer");
  JLX_REQUIRE(limit > 0 && limit <= 100000, "wait probe: the limit must stay small (got %u)", limit);
  wait_that_runs_out_kernel<<<1, 32, 0, stream>>>(status, limit, gave_up);
  JLX_LAUNCH_CHECK("wait_that_runs_out");
  return 0;
}
