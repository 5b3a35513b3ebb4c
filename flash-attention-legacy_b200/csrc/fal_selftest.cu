// Self-test of the bounded wait every tcgen05 / TMA kernel of this library relies on: a thread block
// waits on an mbarrier that nothing will ever complete.  The wait (the library's own mbar_wait, with
// its production limit of about one second) must give up, record kDevWaitTimeout + barrier_id in the
// status word and let the kernel end normally -- the device stays usable, nothing traps.
// The reference has no counterpart: its kernels synchronise with __syncthreads only.
#include "fal_launch.h"
#include "sm100_ptx.cuh"

namespace fal {

namespace {

__global__ void __launch_bounds__(64) fal_selftest_wait_kernel(int barrier_id, int* status, int* waits_given_up) {
  __shared__ __align__(8) uint64_t bar_mem;
  __shared__ int abort_flag;
  const uint32_t bar = smem_u32(&bar_mem);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(bar, 1);  // one arrival expected; nobody arrives
    fence_mbar_init();
  }
  __syncthreads();
  const WaitCtx wctx{&abort_flag, status};
  // Whichever warp runs into the time limit first raises the block's abort flag; the other one sees
  // the flag at its next check and gives up as well.
  const bool done = mbar_wait(bar, 0, wctx, barrier_id);
  if (!done && (threadIdx.x & 31) == 0 && waits_given_up) atomicAdd(waits_given_up, 1);
}

}  // namespace

cudaError_t launch_selftest_wait(int barrier_id, int* status, int* waits_given_up, cudaStream_t stream) {
  fal_selftest_wait_kernel<<<1, 64, 0, stream>>>(barrier_id, status, waits_given_up);
  return cudaGetLastError();
}

}  // namespace fal
