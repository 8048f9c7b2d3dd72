// Self-test of the bounded device-side waits: a kernel waits on an mbarrier that nothing ever
// arrives at, with a short deadline, and must come back with the give-up code in the status word
// instead of hanging.  Nothing faults: the wait simply runs out and the kernel returns.
#include "mvpa_common.cuh"
#include "tc_ptx.cuh"

namespace mvpa {
namespace {

constexpr int kSelftestCode = 59;

__global__ void __launch_bounds__(32) wait_timeout_kernel(int* status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1);
    ptx::mbar_fence_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) ptx::mbar_wait(&bar, 0, status, kSelftestCode);  // phase 0 never completes
}

}  // namespace

int selftest_wait_timeout(int* status, unsigned limit_us, cudaStream_t s) {
  MVPA_CUDA_CHECK(cudaMemsetAsync(status, 0, 256, s));
  // (this translation unit's copy of the deadline: the product kernels keep their default)
  MVPA_CUDA_CHECK(cudaMemcpyToSymbolAsync(ptx::g_wait_limit_us, &limit_us, sizeof(limit_us), 0,
                                          cudaMemcpyHostToDevice, s));
  wait_timeout_kernel<<<1, 32, 0, s>>>(status);
  count_launch();
  MVPA_CUDA_CHECK(cudaGetLastError());
  const unsigned zero = 0;
  MVPA_CUDA_CHECK(cudaMemcpyToSymbolAsync(ptx::g_wait_limit_us, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, s));
  return MVPA_OK;
}

}  // namespace mvpa
