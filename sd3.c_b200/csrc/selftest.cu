// Self-test of the bounded-wait machinery: a kernel that waits on an mbarrier
// nobody ever arrives on, with a short limit, and goes through the same path a
// production kernel takes when a wait runs out (status word, CTA abort flag,
// drain, return).  It touches no TMA, no tensor core and no TMEM, so nothing is
// in flight when it gives up and the context stays usable.  Integrators can
// call it once to check that a device-side timeout surfaces through
// sd3_device_status; the test suite does.  The reference has no counterpart
// (its CUDA path calls exit(EXIT_FAILURE) on errors, cuda/dit.cu:96,460,690,738).
#include "../../include/sd3_b200.h"
#include "kernels.h"
#include "ptx.cuh"

namespace sd3 {
int* device_status_word();

namespace {

__global__ void __launch_bounds__(64, 1) wait_timeout_kernel(int* status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    s_abort = 0;
    fence_barrier_init();
  }
  __syncthreads();
  const WaitCtx wc{&s_abort, status};
  // warp 0 waits for a phase that never completes; warp 1 waits on the same barrier and
  // leaves through the abort flag that warp 0 raises (or through its own limit)
  bool ok = true;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(&bar, 0, wc, DEV_TIMEOUT_SELFTEST, limit_ns);
  __syncthreads();
  if (s_abort) drain_after_abort();
  (void)ok;
}

}  // namespace
}  // namespace sd3

extern "C" int sd3_selftest_wait_timeout(int limit_us, void* stream) {
  using namespace sd3;
  if (limit_us <= 0 || limit_us > 1000000) {
    set_last_error("sd3_selftest_wait_timeout: limit_us must be in (0, 1000000]");
    return SD3_ERR_INVALID_ARG;
  }
  int* status = device_status_word();
  if (!status) {
    set_last_error("device status word unavailable");
    return SD3_ERR_CUDA;
  }
  wait_timeout_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(
      status, static_cast<unsigned long long>(limit_us) * 1000ull);
  return after_launch("wait_timeout_kernel");
}
