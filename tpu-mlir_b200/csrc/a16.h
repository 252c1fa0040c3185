// A16MatMul (4-bit group-quantized weights, bf16 activations) kernel launchers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200q {

int a16_w4_gemv_supported(int M, int N, int K, int group, const char** why, bool f16 = false);
// weights_constant: the caller vouches that no earlier work of the stream writes wq / scale / zp, so the kernel may
// request its first weight rows while the previous kernel of the stream is still running.
// x bf16 [M,K], wq bytes [N,K/2], scale bf16 [N*K/group], zp u8 [N*K/group], bias f32 [N] or null, y bf16 [M,N]
int a16_w4_gemv_launch(const void* x, const void* wq, const void* scale, const void* zp, const float* bias, void* y,
                       int M, int N, int K, int group, int* status, cudaStream_t stream, bool weights_constant = false,
                       bool f16 = false);
// f16 = true: x, scale and y hold IEEE half values instead of bf16 (w4f16); the one-token kernel and the tensor-core
// kernel have that form.

// Tensor-core form (a16_w4_umma.cu): any M; K and the group size multiples of 64.
int a16_w4_umma_supported(long long M, int N, int K, int group, const char** why);
int a16_w4_umma_launch(const void* x, const void* wq, const void* scale, const void* zp, const float* bias, void* y,
                       long long M, int N, int K, int group, int* status, cudaStream_t stream, bool f16 = false);

}  // namespace b200q
