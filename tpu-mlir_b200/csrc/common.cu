// Error reporting and library-level entry points of libb200q.
#include <cstdarg>
#include <cstdio>

#include "internal.h"

namespace b200q {

static thread_local char g_last_error[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_error(cudaError_t e, const char* expr, const char* file, int line) {
  const int code = (e == cudaErrorMemoryAllocation) ? B200Q_ERR_NOMEM
                   : (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) ? B200Q_ERR_NO_DEVICE
                                                                                  : B200Q_ERR_CUDA;
  return set_error(code, "%s failed: %s (%s:%d)", expr, cudaGetErrorString(e), file, line);
}

}  // namespace b200q

extern "C" {

const char* b200q_version(void) { return "b200q 0.1 (sm_100a)"; }

const char* b200q_last_error(void) { return b200q::g_last_error; }

int b200q_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  int ok = 0;
  for (int i = 0; i < n; ++i) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, i) == cudaSuccess && major == 10) ++ok;
  }
  return ok;
}

}  // extern "C"
