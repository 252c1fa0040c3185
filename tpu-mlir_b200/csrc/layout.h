// Layout / dtype conversion launchers (layout.cu).  All asynchronous on the given stream.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200q {

// x NCHW (uint8/int8 bytes, or float holding integers) -> y [N][H+2bh][W+2bw][C] bytes, interior only.
int nchw_to_bordered_nhwc(const void* x, int x_is_f32, void* y, int N, int C, int H, int W, int bh, int bw,
                          cudaStream_t s);
// w [OC][IC][KH][KW] -> [OC][KH*KW][IC] bytes.
int repack_weight_oihw(const void* w, int w_is_f32, void* wr, int OC, int IC, int KH, int KW, cudaStream_t s);
// 64-channel filters, horizontally adjacent taps paired: [OC][64][KH][KW] -> [OC][KH][ceil(KW/2)][2][64]
int repack_weight_pairs64(const void* w, int w_is_f32, void* wr, int OC, int KH, int KW, cudaStream_t s);
// few-channel im2col order: [OC][C][KH][KW] -> [OC][kpad], k = (fy*C + c)*8 + fx
int repack_weight_fy_c_fx8(const void* w, int w_is_f32, void* wr, int OC, int C, int KH, int KW, int kpad, cudaStream_t s);
// [rows][cols] -> [cols][rows] bytes.
int transpose_to_u8(const void* src, int src_is_f32, void* dst, int rows, int cols, cudaStream_t s);
int transpose_f32(const float* src, float* dst, int rows, int cols, cudaStream_t s);
int f32_to_q8(const float* x, void* y, long long n, cudaStream_t s);
int f32_to_i32(const float* x, int32_t* y, long long n, cudaStream_t s);
int q_to_f32(const void* x, int dt, float* y, long long n, cudaStream_t s);

}  // namespace b200q
