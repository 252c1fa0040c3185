// Internal helpers shared by the translation units of libb200q: thread-local error text and CUDA error
// mapping.  Nothing in the library aborts; every failure becomes a negative b200q_status.
#pragma once
#include <cuda_runtime.h>

#include "../../include/b200q.h"

namespace b200q {

// Records a printf-style message for b200q_last_error() and returns `code`.
int set_error(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
int cuda_error(cudaError_t e, const char* expr, const char* file, int line);

#define CUDA_TRY(expr)                                                          \
  do {                                                                          \
    cudaError_t _e = (expr);                                                    \
    if (_e != cudaSuccess) return ::b200q::cuda_error(_e, #expr, __FILE__, __LINE__); \
  } while (0)

#define B200Q_TRY(expr)        \
  do {                         \
    int _rc = (expr);          \
    if (_rc != B200Q_OK) return _rc; \
  } while (0)

inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

}  // namespace b200q
