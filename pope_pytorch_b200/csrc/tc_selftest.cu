// Self-test of the bounded-wait discipline of the tensor-core kernels (sm_100a).
//
// Every mbarrier wait in the attention / similarity kernels is bounded: after a fixed number of parked tries the
// waiter gives up, sets bit 0 of the sticky device status word, and the CTA unwinds through its normal exit (frees its
// tensor memory, returns).  That path never runs in a healthy kernel, so this file provides the one launch that takes
// it on purpose: a single CTA with the role skeleton of the real kernels (a TMEM allocation owned by one warp, an
// mbarrier initialised for one arrival) in which nobody ever arrives.  The wait uses the same mbar_wait as the real
// kernels with a limit of 8 tries and a 1 microsecond park hint, so the launch ends after a few microseconds with
// the status bit set and the device fully usable.  Nothing here faults, traps or spins without bound.
#include "kernels.h"
#include "tc_common.cuh"

namespace pope {

__global__ void __launch_bounds__(128, 1) bounded_wait_selftest_kernel(unsigned int* status) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5;
  if (warp == 0) {
    tmem_alloc(&tmem_slot, 32);
    tmem_relinquish();
  }
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_init_fence();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem = tmem_slot;
  bool failed = false;
  if (warp == 1) {
    // the barrier's first phase never completes: 8 parked tries of at most 1 us each, then give up
    bool ok = false;
    for (uint32_t i = 0; i < 8 && !ok; ++i) ok = mbar_try_wait(&bar, 0, 1000u);
    failed = !ok;
  }
  if (failed && (threadIdx.x & 31) == 0) atomicOr(status, 1u);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 32);
}

cudaError_t tc_selftest_bounded_wait(cudaStream_t st) {
  unsigned int* status = tc_status_ptr();
  if (!status) return cudaErrorInvalidSymbol;
  bounded_wait_selftest_kernel<<<1, 128, 0, st>>>(status);
  return cudaGetLastError();
}

}  // namespace pope
