// Error reporting shared by all launchers: a thread-local message that the C
// ABI hands out through sd3_last_error().  The reference instead calls
// exit(EXIT_FAILURE) on CUDA errors (cuda/dit.cu:96,460,690,738); here every
// failure becomes a negative return code plus a message.
#include <stdarg.h>
#include <stdio.h>

#include <atomic>

#include "kernels.h"

namespace sd3 {

static thread_local char g_last_error[512] = "";

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

const char* get_last_error() { return g_last_error; }

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return ST_OK;
  set_last_error("%s: %s", what, cudaGetErrorString(e));
  return ST_CUDA_ERROR;
}

static std::atomic<long> g_launches{0};

// Called right after every kernel launch: counts it and picks up launch errors.
int after_launch(const char* kernel_name) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return ST_OK;
  set_last_error("launch of %s failed: %s", kernel_name, cudaGetErrorString(e));
  return ST_CUDA_ERROR;
}

long launch_count(int reset) {
  return reset ? g_launches.exchange(0) : g_launches.load();
}

}  // namespace sd3
