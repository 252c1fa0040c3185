// A16MatMul (4-bit group-quantized weights, bf16 activations) kernel launchers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "devbuf.h"

namespace b200q {

int a16_w4_gemv_supported(int M, int N, int K, int group, const char** why, bool f16 = false);
// weights_constant: the caller vouches that no earlier work of the stream writes wq / scale / zp, so the kernel may
// request its first weight rows while the previous kernel of the stream is still running.
// x bf16 [M,K], wq bytes [N,K/2], scale bf16 [N*K/group], zp u8 [N*K/group], bias f32 [N] or null, y bf16 [M,N]
int a16_w4_gemv_launch(const void* x, const void* wq, const void* scale, const void* zp, const float* bias, void* y,
                       int M, int N, int K, int group, int* status, cudaStream_t stream, bool weights_constant = false,
                       bool f16 = false);
// Whether two to eight tokens of this shape run the resident form of the decode kernel (the faster one: then nine to
// sixteen tokens are better served by two decode launches than by the fused tensor-core kernel).
int a16_w4_gemv_resident_applies(int N, int K, int group, bool f16);
// f16 = true: x, scale and y hold IEEE half values instead of bf16 (w4f16); the one-token kernel and the tensor-core
// kernel have that form.

// Tensor-core form (a16_w4_umma.cu): any M; K and the group size multiples of 64.
int a16_w4_umma_supported(long long M, int N, int K, int group, const char** why);
int a16_w4_umma_launch(const void* x, const void* wq, const void* scale, const void* zp, const float* bias, void* y,
                       long long M, int N, int K, int group, int* status, cudaStream_t stream, bool f16 = false);

// Warpgroup form for a handful of tokens (a16_w4_wg.cu): M <= 32; K a multiple of 64; group 32 or a multiple of 64.
int a16_w4_wg_supported(long long M, int N, int K, int group, const char** why);
struct A16WgScratch {   // fp32 partial sums [M][N] and per-tile arrival counters, zero between launches
  DevBuf ws, counters;
  size_t ws_elems = 0;
  int tiles = 0;
};
// scratch: the caller's (a handle's), or null for one kept per (device, stream) by the launcher
int a16_w4_wg_launch(const void* x, const void* wq, const void* scale, const void* zp, const float* bias, void* y,
                     long long M, int N, int K, int group, int* status, cudaStream_t stream, bool f16 = false,
                     A16WgScratch* scratch = nullptr);

}  // namespace b200q
