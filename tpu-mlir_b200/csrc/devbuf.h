// Grow-only device buffer owned by an op handle.
#pragma once
#include <cuda_runtime.h>

#include "internal.h"

namespace b200q {

struct DevBuf {
  void* p = nullptr;
  size_t cap = 0;
  DevBuf() = default;
  DevBuf(const DevBuf&) = delete;
  DevBuf& operator=(const DevBuf&) = delete;
  ~DevBuf() {
    if (p) cudaFree(p);
  }
  // Make room for `bytes` (contents are not preserved when the buffer grows).
  int ensure(size_t bytes) {
    if (bytes <= cap) return B200Q_OK;
    if (p) {
      cudaFree(p);
      p = nullptr;
      cap = 0;
    }
    const size_t want = (bytes + 255) & ~size_t(255);
    cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) {
      p = nullptr;
      return cuda_error(e, "cudaMalloc", __FILE__, __LINE__);
    }
    cap = want;
    return B200Q_OK;
  }
  int upload(const void* host, size_t bytes, cudaStream_t s) {
    B200Q_TRY(ensure(bytes));
    CUDA_TRY(cudaMemcpyAsync(p, host, bytes, cudaMemcpyHostToDevice, s));
    return B200Q_OK;
  }
  template <typename T>
  T* as() const {
    return static_cast<T*>(p);
  }
};

}  // namespace b200q
