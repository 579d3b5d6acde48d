// A kernel that does nothing but wait, with the library's bounded mbarrier wait, on a barrier on
// which nothing ever arrives: the wait runs out after its time limit, the kernel sets the status
// word's WAIT_TIMEOUT bit and returns.  It exists so that a test can see the bound work (every
// kernel that copies by TMA or multiplies on tcgen05 waits through the same helper) without a
// fault and without a hang: the wait ends by itself.
#include "tcgen05.cuh"

namespace {

__global__ void wait_probe_kernel(int* status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  if (threadIdx.x == 0 && !mbar_wait(&bar, 0)) atomicOr(status, (int)SPROUT_STATUS_WAIT_TIMEOUT);
}

}  // namespace

SPROUT_API int sprout_wait_probe(int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(status, "wait_probe: null pointer");
  wait_probe_kernel<<<1, 32, 0, stream>>>(status);
  return sprout_check_launch("wait_probe");
}
