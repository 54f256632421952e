// Self-test of the failure path: a wait that nothing ever satisfies must end by
// itself, leave the context usable and report through the device status word.
#include "../../include/coda_b200.h"
#include "gemm_host.cuh"

using namespace cb;

namespace {
// One warp waits on an mbarrier that never receives its arrival.  The wait is
// the same bounded wait every GEMM role uses, with a short limit; when it runs
// out the kernel records the code and returns normally.
__global__ void wait_timeout_kernel(int* __restrict__ status, unsigned long long timeout_ns, int* __restrict__ waited_us) {
  __shared__ alignas(8) unsigned long long bar_storage;
  __shared__ int abort_word;
  const uint32_t bar = smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    abort_word = 0;
    mbar_init(bar, 1);
    fence_barrier_init();
  }
  __syncthreads();
  const unsigned long long t0 = globaltimer_ns();
  const bool ok = mbar_wait_for(bar, 0u, &abort_word, kErrTimeoutFull, timeout_ns);
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!ok || abort_word != 0) report_status(status, abort_word != 0 ? abort_word : static_cast<int>(kErrTimeoutFull));
    if (waited_us != nullptr) *waited_us = static_cast<int>((globaltimer_ns() - t0) / 1000ull);
  }
}
}  // namespace

extern "C" int coda_b200_selftest_wait_timeout(int* dev_status, int64_t timeout_us, int* waited_us, void* stream) {
  if (dev_status == nullptr) return fail(kBadArgument, "device status word is required");
  if (timeout_us <= 0 || timeout_us > 1000000) return fail(kBadArgument, "timeout must be between 1 us and 1 s");
  wait_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(dev_status, static_cast<unsigned long long>(timeout_us) * 1000ull,
                                                                      waited_us);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(kCudaError, std::string("selftest launch: ") + cudaGetErrorString(e));
  return kOk;
}
