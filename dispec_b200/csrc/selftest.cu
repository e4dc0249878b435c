// Self-test entry points: they exercise the kernels' own error reporting in forms that cannot touch
// bad memory and cannot wait without bound.
#include "tcgen05_common.cuh"

namespace {
// One warp waits, with the product kernels' own bounded wait, on an mbarrier at which nothing ever
// arrives.  The wait runs out after `tries` tries, the kernel records DSP_ERR_WAIT_LIMIT in the
// device error word and returns normally: the context stays usable.
__global__ void wait_limit_kernel(uint32_t tries, int* err, int* ran_out) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    tc::mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const bool done = tc::mbar_wait_limit(&bar, 0, tries);
  if (!done && threadIdx.x == 0) {
    atomicOr(err, DSP_ERR_WAIT_LIMIT);
    *ran_out = 1;
  }
}
}  // namespace

// tries: at most 65,536 (each try blocks for a short, hardware-bounded time).  ran_out: a device
// int that is set to 1 when the wait ran out.
extern "C" int dsp_selftest_wait_limit(int tries, int* ran_out, cudaStream_t stream) {
  DSP_REQUIRE(tries > 0 && tries <= 65536, "dsp_selftest_wait_limit: tries=%d outside 1..65536", tries);
  int* err = dsp_device_error_ptr();
  DSP_REQUIRE(err != nullptr && ran_out != nullptr, "dsp_selftest_wait_limit: no device error word or result");
  wait_limit_kernel<<<1, 32, 0, stream>>>((uint32_t)tries, err, ran_out);
  DSP_CHECK_LAUNCH("dsp_selftest_wait_limit");
  return 0;
}
