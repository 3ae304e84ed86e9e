// Test hook for the bounded-wait policy of dsa_common.cuh: one thread waits on an mbarrier that
// nobody arrives at, with a small poll limit passed by the caller, and must come back with the
// time-out status instead of spinning.  No TMA, no MMA, no tensor memory: only the wait helper
// that every pipeline role of the real kernels uses.
#include "dsa_common.cuh"
#include "dsa_host.h"

namespace dsa {

__global__ void __launch_bounds__(32) bounded_wait_probe_kernel(uint32_t poll_limit, int* status, int* result) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
    abort_flag = 0;
    const bool ok = mbar_wait_limit(&bar, 0, &abort_flag, status, poll_limit);
    if (result) *result = ok ? 0 : (abort_flag ? 1 : 2);
  }
}

int bounded_wait_probe_launch(uint32_t poll_limit, int32_t* status, cudaStream_t stream) {
  bounded_wait_probe_kernel<<<1, 32, 0, stream>>>(poll_limit, status, nullptr);
  return check_launch("bounded_wait_probe");
}

}  // namespace dsa
