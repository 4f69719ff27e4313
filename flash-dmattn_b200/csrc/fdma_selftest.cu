// fdma_selftest_wait_timeout: exercises the give-up path of the bounded mbarrier wait that every tcgen05 kernel of
// this library uses, without involving any of those kernels.
//
// One CTA allocates tensor memory, initialises an mbarrier that nothing will ever arrive on, and waits on it with
// a SHORT limit supplied by the caller. The wait must run out, record its code in the per-device status word (and
// its host mirror), raise the CTA's abort flag, and the CTA must then run the same tear-down the attention
// kernels run (free its tensor memory, return). Nothing here can hang: the only wait is the bounded one.
// The reference has no counterpart (its kernels use no asynchronous barriers).
#include <cuda_runtime.h>

#include "fdma_internal.h"
#include "fdma_ptx.cuh"

namespace fdma {
namespace {

constexpr int kSelfTestCode = 901;

__global__ void __launch_bounds__(64, 1) wait_timeout_kernel(int* status, uint64_t limit_ns, int* result) {
  __shared__ uint64_t bar;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&s_tmem, 32);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = s_tmem;
  const WaitCtl ctl{&s_abort, status};
  // phase 0 of a freshly initialised barrier never completes without an arrival
  const bool ok = mbar_wait_limit(&bar, 0, ctl, kSelfTestCode, limit_ns);
  const bool all_gave_up = __syncthreads_and(!ok) != 0;
  if (threadIdx.x == 0) *result = all_gave_up ? 1 : 0;
  // tear-down, as in the attention kernels
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 32);
  }
}

}  // namespace
}  // namespace fdma

extern "C" int fdma_selftest_wait_timeout(uint32_t limit_us, int* result_dev, void* stream_) {
  using namespace fdma;
  if (!result_dev || limit_us == 0 || limit_us > 1000000u) return FDMA_ERR_BAD_ARG;
  int* status = kernel_status_ptr();
  if (!status) return FDMA_ERR_DRIVER;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  wait_timeout_kernel<<<1, 64, 0, stream>>>(status, static_cast<uint64_t>(limit_us) * 1000ull, result_dev);
  return static_cast<int>(cudaGetLastError());
}
