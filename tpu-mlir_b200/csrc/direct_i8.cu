// CUDA-core INT8 convolution / GEMM for the shapes the tensor-core implicit GEMM does not take
// (channel counts that are not a multiple of 16, strides, dilation, groups, zero points, batched right
// operands).  One thread per output element, int32 accumulation, the same exact epilogue (requant.cuh).
// Semantics: tpu::Conv2DOp::inference (lib/Dialect/Tpu/Interfaces/Common/Conv2D.cpp:264-341) and
// tpu::MatMulOp::inference (MatMul.cpp:599-728) for uniform-quantized outputs.
#include "igemm.h"
#include "internal.h"

namespace b200q {
namespace {

__device__ __forceinline__ int32_t ld_q8(const void* p, long long i, int is_unsigned) {
  return is_unsigned ? (int32_t) reinterpret_cast<const uint8_t*>(p)[i] : (int32_t) reinterpret_cast<const int8_t*>(p)[i];
}

__device__ __forceinline__ void st_q(void* out, long long i, int dt, int32_t v) {
  switch (dt) {
    case B200Q_DT_I8:
    case B200Q_DT_U8: reinterpret_cast<uint8_t*>(out)[i] = (uint8_t)v; break;
    case B200Q_DT_I16:
    case B200Q_DT_U16: reinterpret_cast<uint16_t*>(out)[i] = (uint16_t)v; break;
    default: reinterpret_cast<int32_t*>(out)[i] = v; break;
  }
}

__device__ __forceinline__ int32_t finish(int32_t acc, int c, const Epilogue& e) {
  if (e.bias) acc += e.bias[c];
  if (e.relu == B200Q_RELU_BEFORE_REQUANT && acc < 0) acc = 0;
  const int qi = e.per_channel ? c : 0;
  const int32_t m = e.multiplier ? e.multiplier[qi] : 1;
  const int32_t s = e.shift ? e.shift[qi] : 0;
  return requant_value<-1, -1>(acc, m, s, e);
}

__global__ void conv2d_i8_direct_kernel(const void* __restrict__ x, int x_unsigned, const int8_t* __restrict__ w,
                                        ConvGeometry g, Epilogue e, void* __restrict__ y, long long total) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int xo = (int)(idx % g.ow);
  const int yo = (int)((idx / g.ow) % g.oh);
  const int oc = (int)((idx / ((long long)g.ow * g.oh)) % g.oc);
  const int n = (int)(idx / ((long long)g.ow * g.oh * g.oc));
  const int icg = g.ic / g.groups, ocg = g.oc / g.groups;
  const int grp = oc / ocg;
  int32_t acc = 0;
  for (int c = 0; c < icg; ++c) {
    const int cin = grp * icg + c;
    for (int fy = 0; fy < g.kh; ++fy) {
      const int iy = yo * g.sh - g.pht + fy * g.dh;
      for (int fx = 0; fx < g.kw; ++fx) {
        const int ix = xo * g.sw - g.pwl + fx * g.dw;
        int32_t xv = g.pad_value;
        if (iy >= 0 && iy < g.ih && ix >= 0 && ix < g.iw)
          xv = ld_q8(x, (((long long)n * g.ic + cin) * g.ih + iy) * g.iw + ix, x_unsigned);
        acc += xv * (int32_t)w[(((long long)oc * icg + c) * g.kh + fy) * g.kw + fx];
      }
    }
  }
  st_q(y, idx, e.out_dtype, finish(acc, oc, e));
}

__global__ void gemm_i8_direct_kernel(const void* __restrict__ a, int a_unsigned, const void* __restrict__ b,
                                      int b_unsigned, int b_is_nk, int m, int n, int k, int input_zp, int right_zp,
                                      Epilogue e, void* __restrict__ out) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)m * n) return;
  const int col = (int)(idx % n);
  const long long row = idx / n;
  int32_t acc = 0;
  for (int kk = 0; kk < k; ++kk) {
    const int32_t av = ld_q8(a, row * k + kk, a_unsigned) - input_zp;
    const int32_t bv = ld_q8(b, b_is_nk ? (long long)col * k + kk : (long long)kk * n + col, b_unsigned) - right_zp;
    acc += av * bv;
  }
  st_q(out, idx, e.out_dtype, finish(acc, col, e));
}

}  // namespace

int conv2d_i8_direct_launch(const void* x, int x_unsigned, const int8_t* w, const ConvGeometry& g, const Epilogue& epi,
                            void* y, cudaStream_t stream) {
  const long long total = (long long)g.n * g.oc * g.oh * g.ow;
  if (total == 0) return B200Q_OK;
  const int threads = 256;
  const long long blocks = (total + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return set_error(B200Q_ERR_UNSUPPORTED, "direct conv: output too large");
  conv2d_i8_direct_kernel<<<(unsigned)blocks, threads, 0, stream>>>(x, x_unsigned, w, g, epi, y, total);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int gemm_i8_direct_launch(const void* a, int a_unsigned, const void* b, int b_unsigned, int b_is_nk, int m, int n,
                          int k, int input_zp, int right_zp, const Epilogue& epi, void* out, cudaStream_t stream) {
  const long long total = (long long)m * n;
  if (total == 0) return B200Q_OK;
  const int threads = 256;
  const long long blocks = (total + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return set_error(B200Q_ERR_UNSUPPORTED, "direct gemm: output too large");
  gemm_i8_direct_kernel<<<(unsigned)blocks, threads, 0, stream>>>(a, a_unsigned, b, b_unsigned, b_is_nk, m, n, k,
                                                                  input_zp, right_zp, epi, out);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

}  // namespace b200q
