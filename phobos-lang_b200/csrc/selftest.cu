// Self-test of the bounded-wait policy: one CTA initialises an mbarrier that
// nothing ever arrives at and waits on it through the same mbar_wait the leaf
// kernels use, with a caller-chosen limit.  The wait runs out, records
// SITE_SELFTEST in the device's status word and the kernel returns normally:
// no trap, no fault, the context stays usable.  This is how the time-out path
// of the kernels is exercised without breaking a real pipeline.  The reference's
// analogues are host side: the engine's stall detector and the fetch deadline
// (phobos-pod/src/engine.rs:752-775, 825-828).
#include "common.cuh"
#include "kernels.h"

namespace ph {
namespace {

__global__ void __launch_bounds__(32, 1) selftest_wait_kernel(unsigned long long limit_ns, uint32_t* status) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncwarp();
  WaitCtx ctx{&abort_flag, status, limit_ns};
  // every lane takes the whole-warp form the kernels use ahead of collective instructions
  const bool ok = mbar_wait_warp(&bar, 0, SITE_SELFTEST, ctx);
  // a wait that succeeded here would mean the barrier completed by itself: report that as its own code
  if (ok && threadIdx.x == 0) atomicCAS(status, 0u, 0xFFu);
}

}  // namespace

int launch_selftest_wait(unsigned long long limit_ns, uint32_t* status, cudaStream_t stream, const char** err) {
  selftest_wait_kernel<<<1, 32, 0, stream>>>(limit_ns, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    *err = cudaGetErrorString(e);
    return -3;
  }
  return 0;
}

}  // namespace ph
