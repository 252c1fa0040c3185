// A16MatMul (4-bit group-quantized weights, bf16 activations) kernel launchers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200q {

int a16_w4_gemv_supported(int M, int N, int K, int group, const char** why);
// x bf16 [M,K], wq bytes [N,K/2], scale bf16 [N*K/group], zp u8 [N*K/group], bias f32 [N] or null, y bf16 [M,N]
int a16_w4_gemv_launch(const void* x, const void* wq, const void* scale, const void* zp, const float* bias, void* y,
                       int M, int N, int K, int group, int* status, cudaStream_t stream);

}  // namespace b200q
