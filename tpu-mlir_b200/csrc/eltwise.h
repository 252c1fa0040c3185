// Launchers of eltwise.cu (asynchronous on the given stream).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "requant.cuh"

namespace b200q {

int requant_axis_launch(const int32_t* x, long long outer, int C, long long inner, const int32_t* mult,
                        const int32_t* shift, const int32_t* zp, int per_channel, int in_zp, const Epilogue& e, void* out,
                        cudaStream_t s);
int constop_i8_launch(int form, const void* x, int dt, long long n, int m, double const_val, int sft, int in_zp, int do_relu, float relu_limit,
                      int out_dt, void* out, cudaStream_t s);
int sub_i8_launch(const void* a, int a_dt, const void* b, int b_dt, long long n, int m0, int s0, int m1, int s1, int do_relu, int out_dt,
                  void* out, cudaStream_t s);
int add_i8_launch(const void* a, int a_dt, const void* b, int b_dt, long long n, int m0, int s0, int m1, int s1,
                  int do_relu, int out_dt, void* out, cudaStream_t s);
// mode 0 = max, 1 = average (window sum * multi >> rshift, half up)
int pool2d_i8_launch(const void* x, int dt, int NC, int ih, int iw, int kh, int kw, int sh, int sw, int pht, int phb,
                     int pwl, int pwr, int mode, int multi, int rshift, int do_relu, int out_dt, void* out, cudaStream_t s);
// tpu.Lut / tpu.MulShift / tpu.Mul (8-bit, equal shapes)
int lut_launch(const void* x, long long n, const void* table, int elem_size, void* out, cudaStream_t s);
int requant_fp_launch(const void* x, int in_is_i32, long long n, float scale, float offset, int zp, int tflite, int rmode, int out_dt,
                      void* out, cudaStream_t s);
int prelu_i8_launch(const void* x, int dt, const void* slope, long long n, long long inner, int num_slope, int sft, int out_dt, void* out,
                    cudaStream_t s);
int prelu_f32_launch(const float* x, const float* slope, long long n, long long inner, int num_slope, float* out, cudaStream_t s);
int addconst_i8_launch(const void* x, int dt, long long n, int m, double const_val, int sft, int in_zp, int do_relu, int out_dt,
                       void* out, cudaStream_t s);
int mulshift_i8_launch(const void* x, int dt, long long n, int m, int sft, int in_zp, int out_zp, int out_dt, void* out,
                       cudaStream_t s);
int mul_i8_launch(const void* a, int a_dt, const void* b, int b_dt, long long n, int m, int sft, int do_relu, int out_dt,
                  void* out, cudaStream_t s);
// NHWC-resident graphs: [N][H][W][C] -> interior of the zero-bordered image; pooling on [N][H][W][C]
int nhwc_to_bordered_launch(const void* x, void* y, long long N, int C, int H, int W, int bh, int bw, cudaStream_t s);
int pool2d_i8_nhwc_launch(const void* x, int dt, long long N, int C, int ih, int iw, int kh, int kw, int sh, int sw, int pht,
                          int phb, int pwl, int pwr, int mode, int multi, int rshift, int do_relu, int out_dt, void* out,
                          cudaStream_t s);
int cast_f32_q8_launch(const float* x, long long n, double scale, int zp, int rmode, int out_dt, void* out, cudaStream_t s);
int cast_q8_f32_launch(const void* x, int dt, long long n, double scale, int zp, float* out, cudaStream_t s);
// x: zero-bordered NHWC bytes [N][Hp][Wp][C]; a: rows [N*OH*OW][kpad], k = (fy*KW+fx)*C + c.  (oy0, ox0) = bordered
// coordinate of the first tap of output pixel (0,0), i.e. border - pad.
int im2col_nhwc_launch(const void* x, void* a, long long N, int C, int Hp, int Wp, int OH, int OW, int KH, int KW, int sh,
                       int sw, int dh, int dw, int oy0, int ox0, int kpad, cudaStream_t s);
// im2col straight from NCHW (bytes, or floats holding integers) for few input channels; zero padding
int im2col_nchw_small_c_launch(const void* x, int x_is_f32, void* a, long long N, int C, int H, int W, int OH, int OW, int KH,
                               int KW, int sh, int sw, int dh, int dw, int pht, int pwl, int kpad, cudaStream_t s);
// im2col for at most 4 input channels and filters up to 8 taps wide, straight from NCHW; K order (fy, c, fx padded
// to 8), row length kpad = round16(KH*C*8)
bool im2col_few_channels_ok(int C, int H, int W, int KH, int KW, int sh, int sw, int dh, int dw, int pwl, int OW);
int im2col_few_channels_launch(const void* x, int x_is_f32, void* a, long long N, int C, int H, int W, int OH, int OW, int KH,
                               int sh, int sw, int pht, int pwl, int kpad, cudaStream_t s);

}  // namespace b200q
