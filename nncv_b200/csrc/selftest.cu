// A kernel that does nothing but run a bounded wait to its limit: it initialises an mbarrier
// nobody ever arrives on, waits on it with a short clock budget, reports the time-out into the
// device status word exactly as the convolution kernels do, and returns.  It exists so that the
// host side of the failure path (status word -> NNCV_B200_ETIMEOUT -> the next call works again)
// can be exercised without a fault, a trap or an unbounded loop.  nncv has no device code and no
// counterpart.
#include <cuda_runtime.h>

#include "kernels.h"
#include "ptx.cuh"

namespace nncv_b200 {

namespace {

__global__ void __launch_bounds__(32) wait_selftest_kernel(int* error_flag, long long limit_clocks) {
  __shared__ __align__(8) unsigned long long bar;
  const uint32_t b = ptx::smem_u32(&bar);
  if (threadIdx.x == 0) {
    ptx::mbar_init(b, 1);
    ptx::mbar_fence_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    // phase 0 never completes: no thread and no copy arrives on this barrier
    if (!ptx::mbar_wait_limit(b, 0, limit_clocks) && error_flag) atomicCAS(error_flag, 0, (int)kErrWaitEpilogue);
  }
}

}  // namespace

cudaError_t launch_wait_selftest(int* error_flag, long long limit_clocks, cudaStream_t stream) {
  if (limit_clocks < 1) limit_clocks = 1;
  if (limit_clocks > (1LL << 24)) limit_clocks = 1LL << 24;   // a few milliseconds at most
  wait_selftest_kernel<<<1, 32, 0, stream>>>(error_flag, limit_clocks);
  return cudaGetLastError();
}

}  // namespace nncv_b200
