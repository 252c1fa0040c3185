// Element-wise and pooling ops of an INT8 graph around the MatMul/Conv2D kernels, on native NCHW tensors:
// stand-alone requantisation, residual Add, max / average pooling, float <-> int8 casts.  All HBM-bound.
//
// Reference semantics (paths inside the tpu-mlir tree):
//   tpu.RequantIntAxis  lib/Dialect/Tpu/Interfaces/Common/RequantIntAxis.cpp:17-123
//   tpu.RequantInt      lib/Dialect/Tpu/Interfaces/Common/RequantInt.cpp:17-71
//   tpu.Add             lib/Dialect/Tpu/Interfaces/Common/Add.cpp:177-207 (symmetric int8, BM168x)
//   tpu.Pool2D          lib/Dialect/Tpu/Interfaces/Common/Pool2D.cpp:160-192
//   tpu.Cast            lib/Dialect/Tpu/Interfaces/Common/Cast.cpp:75-116, lib/Support/CastUtils.cpp:15-47
#include "eltwise.h"
#include "internal.h"
#include "requant.cuh"

namespace b200q {
namespace {
__device__ __forceinline__ uint8_t to_u8(uint8_t v) { return v; }
__device__ __forceinline__ uint8_t to_u8(float v) { return (uint8_t)(int)v; }  // integral by contract

__device__ __forceinline__ uint32_t ld4_as_bytes(const uint8_t* p) { return *reinterpret_cast<const uint32_t*>(p); }
__device__ __forceinline__ uint32_t ld4_as_bytes(const float* p) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  return (uint32_t)((int)v.x & 0xff) | ((uint32_t)((int)v.y & 0xff) << 8) | ((uint32_t)((int)v.z & 0xff) << 16) |
         ((uint32_t)((int)v.w & 0xff) << 24);
}


__device__ __forceinline__ int32_t ld_q(const void* p, long long i, int dt) {
  switch (dt) {
    case B200Q_DT_I8: return reinterpret_cast<const int8_t*>(p)[i];
    case B200Q_DT_U8: return reinterpret_cast<const uint8_t*>(p)[i];
    case B200Q_DT_I16: return reinterpret_cast<const int16_t*>(p)[i];
    case B200Q_DT_U16: return reinterpret_cast<const uint16_t*>(p)[i];
    default: return reinterpret_cast<const int32_t*>(p)[i];
  }
}
__device__ __forceinline__ void st_q(void* p, long long i, int dt, int32_t v) {
  switch (dt) {
    case B200Q_DT_I8:
    case B200Q_DT_U8: reinterpret_cast<uint8_t*>(p)[i] = (uint8_t)v; break;
    case B200Q_DT_I16:
    case B200Q_DT_U16: reinterpret_cast<uint16_t*>(p)[i] = (uint16_t)v; break;
    default: reinterpret_cast<int32_t*>(p)[i] = v; break;
  }
}

// x int32 viewed [outer][C][inner]; per channel {multiplier, shift, zero point}; e carries dialect / rounding /
// output type (its own zero point and per-channel arrays are not used here).
__global__ void requant_axis_kernel(const int32_t* __restrict__ x, long long total, int C, long long inner,
                                    const int32_t* __restrict__ mult, const int32_t* __restrict__ shift,
                                    const int32_t* __restrict__ zp, int per_channel, int in_zp, Epilogue e,
                                    void* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = per_channel ? (int)((i / inner) % C) : 0;
  Epilogue le = e;
  le.out_zp = zp ? zp[c] : e.out_zp;
  st_q(out, i, e.out_dtype, requant_value<-1, -1>(x[i] - in_zp, mult ? mult[c] : 1, shift ? shift[c] : 0, le));
}

__global__ void add_i8_kernel(const void* __restrict__ a, int a_dt, const void* __restrict__ b, int b_dt, long long n,
                              int m0, int s0, int m1, int s1, int do_relu, int out_dt, void* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t l = rshift_round((int64_t)ld_q(a, i, a_dt) * m0, s0, B200Q_ROUND_HALF_UP);
  const int64_t r = rshift_round((int64_t)ld_q(b, i, b_dt) * m1, s1, B200Q_ROUND_HALF_UP);
  int64_t v = l + r;
  if (do_relu && v < 0) v = 0;
  st_q(out, i, out_dt, (int32_t)clamp_dtype(v, out_dt));
}

// tpu.MaxConst / MinConst (MaxConst.cpp:27-42, MinConst.cpp alike) and tpu.SubConst (SubConst.cpp:26-112, symmetric) with a
// uniform-quantized output, in the reference's mix of types: the scaled input (x - in_zp) * m is held in a float, compared
// with / reduced by the constant there, cut to an integer toward zero where applyMultiplierAndRShift takes it, then shifted
// half-up, ReLU'd and saturated.  form 0 max, 1 min, 2 x - c, 3 c - x (SubConst takes no input zero point).
__global__ void __launch_bounds__(256)
constop_i8_kernel(int form, const void* __restrict__ x, int dt, long long n, int m, double const_val, int sft, int in_zp, int do_relu,
                  float relu_limit, int out_dt, void* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float f;
  if (form <= 1) {
    const float pf = (float)((int64_t)(ld_q(x, i, dt) - in_zp) * m), cf = (float)const_val;
    f = form == 0 ? fmaxf(pf, cf) : fminf(pf, cf);
  } else {
    const double prod = (double)((int64_t)ld_q(x, i, dt) * m);
    f = (float)(form == 2 ? prod - const_val : const_val - prod);
    if (do_relu) {
      f = fmaxf(f, 0.f);
      if (relu_limit > 0.f) f = fminf(f, relu_limit);
    }
  }
  int64_t v = rshift_round((int64_t)f, sft, B200Q_ROUND_HALF_UP);
  if (do_relu && v < 0) v = 0;
  st_q(out, i, out_dt, (int32_t)clamp_dtype(v, out_dt));
}

// tpu.Sub, symmetric 8-bit (lib/Dialect/Tpu/Interfaces/Common/Sub.cpp:88-113): each operand is brought to the output's scale
// with its own multiplier and half-up shift, then out = saturate(relu(lhs - rhs)).  (Negating the second multiplier in the
// Add kernel would round its ties the other way.)
__global__ void sub_i8_kernel(const void* __restrict__ a, int a_dt, const void* __restrict__ b, int b_dt, long long n,
                              int m0, int s0, int m1, int s1, int do_relu, int out_dt, void* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t l = rshift_round((int64_t)ld_q(a, i, a_dt) * m0, s0, B200Q_ROUND_HALF_UP);
  const int64_t r = rshift_round((int64_t)ld_q(b, i, b_dt) * m1, s1, B200Q_ROUND_HALF_UP);
  int64_t v = l - r;
  if (do_relu && v < 0) v = 0;
  st_q(out, i, out_dt, (int32_t)clamp_dtype(v, out_dt));
}

// 4 elements per thread for the common 8-bit case
__global__ void add_i8x4_kernel(const uint32_t* __restrict__ a, int a_unsigned, const uint32_t* __restrict__ b,
                                int b_unsigned, long long n4, int m0, int s0, int m1, int s1, int do_relu, int out_dt,
                                uint32_t* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const uint32_t wa = a[i], wb = b[i];
  uint32_t o = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int32_t xa = a_unsigned ? (int32_t)((wa >> (8 * j)) & 0xff) : (int32_t)(int8_t)(wa >> (8 * j));
    const int32_t xb = b_unsigned ? (int32_t)((wb >> (8 * j)) & 0xff) : (int32_t)(int8_t)(wb >> (8 * j));
    int64_t v = rshift_round((int64_t)xa * m0, s0, B200Q_ROUND_HALF_UP) + rshift_round((int64_t)xb * m1, s1, B200Q_ROUND_HALF_UP);
    if (do_relu && v < 0) v = 0;
    o |= ((uint32_t)clamp_dtype(v, out_dt) & 0xffu) << (8 * j);
  }
  out[i] = o;
}

// 16 elements per thread (one 16-byte access per operand) for 8-bit tensors with multipliers / shifts in the range the
// lowering emits (|m| < 2^23, shift in [1, 31]): x*m + 2^(s-1) fits 32 bits, so the half-up shift is one
// multiply-add and one arithmetic shift per input (MathUtils.cpp:474-514 RightShiftRound, ROUNDING_HALF_UP).
template <bool A_UNS, bool B_UNS>
__global__ void __launch_bounds__(256)
add_i8x16_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, long long n16, int m0, int s0, int m1, int s1,
                 int lo, int hi, uint4* __restrict__ out) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // a dependent convolution may set itself up meanwhile
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n16) return;
  const uint4 va = a[i], vb = b[i];
  const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
  const int32_t h0 = 1 << (s0 - 1), h1 = 1 << (s1 - 1);
  uint32_t o[4];
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    uint32_t r = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int32_t xa = A_UNS ? (int32_t)((wa[w] >> (8 * j)) & 0xff) : (int32_t)(int8_t)(wa[w] >> (8 * j));
      const int32_t xb = B_UNS ? (int32_t)((wb[w] >> (8 * j)) & 0xff) : (int32_t)(int8_t)(wb[w] >> (8 * j));
      const int32_t v = ((xa * m0 + h0) >> s0) + ((xb * m1 + h1) >> s1);
      r |= ((uint32_t)min(max(v, lo), hi) & 0xffu) << (8 * j);
    }
    o[w] = r;
  }
  out[i] = make_uint4(o[0], o[1], o[2], o[3]);
}

__global__ void pool2d_i8_kernel(const void* __restrict__ x, int dt, int NC, int ih, int iw, int kh, int kw, int sh,
                                 int sw, int pht, int pwl, int oh, int ow, int mode, int multi, int rshift, int do_relu,
                                 int out_dt, void* __restrict__ out) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)NC * oh * ow;
  if (idx >= total) return;
  const int xo = (int)(idx % ow), yo = (int)((idx / ow) % oh);
  const long long nc = idx / ((long long)ow * oh);
  int64_t best = INT64_MIN, sum = 0;
  for (int fy = 0; fy < kh; ++fy) {
    const int iy = yo * sh - pht + fy;
    if (iy < 0 || iy >= ih) continue;
    for (int fx = 0; fx < kw; ++fx) {
      const int ix = xo * sw - pwl + fx;
      if (ix < 0 || ix >= iw) continue;
      const int64_t v = ld_q(x, (nc * ih + iy) * iw + ix, dt);
      best = v > best ? v : best;
      sum += v;
    }
  }
  int64_t v;
  if (mode == 0) {
    v = best;
    if (do_relu && v < 0) v = 0;
  } else {
    v = rshift_round(sum * multi, rshift, B200Q_ROUND_HALF_UP);
    if (do_relu && v < 0) v = 0;
    v = clamp_dtype(v, out_dt);
  }
  st_q(out, idx, out_dt, (int32_t)v);
}

// 8-bit max pooling, input and output of the same type, no ReLU clamp needed beyond max(v, 0): typed loads and 32-bit
// arithmetic (the general kernel above dispatches on the type per load and works in 64 bits).
template <typename T>
__global__ void __launch_bounds__(256)
maxpool_q8_kernel(const T* __restrict__ x, long long total, int ih, int iw, int kh, int kw, int sh, int sw, int pht, int pwl,
                  int oh, int ow, int do_relu, T* __restrict__ out) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  int xo, yo;
  long long nc;
  if (total < (1ll << 31)) {  // 32-bit index arithmetic (a 64-bit division costs ~100 instructions)
    const uint32_t i32 = (uint32_t)idx, t32 = i32 / (uint32_t)ow;
    xo = (int)(i32 - t32 * (uint32_t)ow);
    const uint32_t n32 = t32 / (uint32_t)oh;
    yo = (int)(t32 - n32 * (uint32_t)oh);
    nc = n32;
  } else {
    xo = (int)(idx % ow);
    const long long t = idx / ow;
    yo = (int)(t % oh);
    nc = t / oh;
  }
  const int y0 = yo * sh - pht, x0 = xo * sw - pwl;
  const int fy0 = max(0, -y0), fy1 = min(kh, ih - y0), fx0 = max(0, -x0), fx1 = min(kw, iw - x0);
  const T* src = x + nc * (long long)ih * iw;
  int best = -2147483647 - 1;
  for (int fy = fy0; fy < fy1; ++fy) {
    const T* row = src + (long long)(y0 + fy) * iw + x0;
    for (int fx = fx0; fx < fx1; ++fx) best = max(best, (int)row[fx]);
  }
  if (do_relu && best < 0) best = 0;
  out[idx] = (T)best;
}

// The same for planes that fit shared memory: a block loads one (n, c) plane with 16-byte accesses, then every
// output reads its window from shared memory (the direct kernel spends its time on strided single-byte global loads).
template <typename T>
__global__ void __launch_bounds__(256)
maxpool_q8_plane_kernel(const T* __restrict__ x, int ih, int iw, int kh, int kw, int sh, int sw, int pht, int pwl, int oh,
                        int ow, int do_relu, T* __restrict__ out) {
  extern __shared__ __align__(16) uint8_t plane_raw[];
  T* plane = reinterpret_cast<T*>(plane_raw);
  const long long nc = blockIdx.x;
  const int n_in = ih * iw;
  const T* src = x + nc * n_in;
  if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    for (int i = threadIdx.x; i < n_in / 16; i += 256)
      reinterpret_cast<uint4*>(plane_raw)[i] = reinterpret_cast<const uint4*>(src)[i];
    for (int i = (n_in / 16) * 16 + threadIdx.x; i < n_in; i += 256) plane[i] = src[i];
  } else {
    for (int i = threadIdx.x; i < n_in; i += 256) plane[i] = src[i];
  }
  __syncthreads();
  T* dst = out + nc * (long long)oh * ow;
  for (int o = threadIdx.x; o < oh * ow; o += 256) {
    const int yo = o / ow, xo = o - yo * ow;
    const int y0 = yo * sh - pht, x0 = xo * sw - pwl;
    const int fy0 = max(0, -y0), fy1 = min(kh, ih - y0), fx0 = max(0, -x0), fx1 = min(kw, iw - x0);
    int best = -2147483647 - 1;
    for (int fy = fy0; fy < fy1; ++fy) {
      const T* row = plane + (y0 + fy) * iw + x0;
      for (int fx = fx0; fx < fx1; ++fx) best = max(best, (int)row[fx]);
    }
    if (do_relu && best < 0) best = 0;
    dst[o] = (T)best;
  }
}

__global__ void cast_f32_q8_kernel(const float* __restrict__ x, long long n, float inv_scale, int zp, int rmode,
                                   int out_dt, void* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = __fadd_rn(roundf(__fmul_rn(x[i], inv_scale)), (float)zp);
  st_q(out, i, out_dt, (int32_t)clamp_dtype(to_int_f32(v, rmode), out_dt));
}

// four elements per thread for 8-bit outputs (16-byte load, 4-byte store), same arithmetic
__global__ void __launch_bounds__(256)
cast_f32_q8x4_kernel(const float4* __restrict__ x, long long n4, float inv_scale, int zp, int rmode, int out_dt,
                     uint32_t* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const float4 v4 = x[i];
  const float f[4] = {v4.x, v4.y, v4.z, v4.w};
  uint32_t o = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float v = __fadd_rn(roundf(__fmul_rn(f[j], inv_scale)), (float)zp);
    o |= ((uint32_t)clamp_dtype(to_int_f32(v, rmode), out_dt) & 0xffu) << (8 * j);
  }
  out[i] = o;
}

__global__ void cast_q8_f32_kernel(const void* __restrict__ x, int dt, long long n, float scale, int zp,
                                   float* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  out[i] = __fmul_rn(scale, __fsub_rn((float)ld_q(x, i, dt), (float)zp));
}

// NHWC [N][Hp][Wp][C] -> im2col rows [N*OH*OW][kpad] with k = (fy*KW + fx)*C + c.  Tap (fy, fx) of output pixel
// (yo, xo) reads position (yo*sh + fy*dh + oy0, xo*sw + fx*dw + ox0); positions outside the image are zeros, so the
// image may carry its padding as a zero border (oy0, ox0 >= 0) or not at all (oy0 = -pad_top, ox0 = -pad_left).
__global__ void im2col_nhwc_kernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ a, int C, int Hp, int Wp, int OH,
                                   int OW, int KH, int KW, int sh, int sw, int dh, int dw, int oy0, int ox0, int kpad,
                                   long long total_units, int vec) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // a dependent convolution may set itself up meanwhile
  // one unit = (row, tap, vec-byte piece of C); vec = 16 when C % 16 == 0, else 1 unit = (row, tap) with a byte loop
  const long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= total_units) return;
  const int pieces = vec == 16 ? C / 16 : 1;
  const int piece = (int)(u % pieces);
  const int tap = (int)((u / pieces) % (KH * KW));
  const long long row = u / ((long long)pieces * KH * KW);
  const int xo = (int)(row % OW), yo = (int)((row / OW) % OH);
  const long long n = row / ((long long)OW * OH);
  const int fy = tap / KW, fx = tap - fy * KW;
  const int iy = yo * sh + fy * dh + oy0, ix = xo * sw + fx * dw + ox0;   // bordered coordinates
  const bool inside = iy >= 0 && iy < Hp && ix >= 0 && ix < Wp;
  const uint8_t* src = x + ((n * Hp + iy) * Wp + ix) * C;
  uint8_t* dst = a + row * kpad + (long long)tap * C;
  if (vec == 16) {
    reinterpret_cast<uint4*>(dst)[piece] = inside ? reinterpret_cast<const uint4*>(src)[piece] : make_uint4(0u, 0u, 0u, 0u);
  } else {
    for (int c = 0; c < C; ++c) dst[c] = inside ? src[c] : (uint8_t)0;
  }
}

// im2col straight from the NCHW input for few input channels (the 3-channel stem of a vision network): no bordered
// NHWC copy in between.  A thread assembles one 16-byte piece of a row [kpad] with k = (fy*KW + fx)*C + c from
// single-byte reads (neighbouring rows share them in L1) and stores it once; positions in the padding and the
// k >= KH*KW*C tail are zero.  The (c, fy, fx) of every k come from a table in shared memory.
template <typename T>
__global__ void __launch_bounds__(256)
im2col_nchw_small_c_kernel(const T* __restrict__ x, uint8_t* __restrict__ a, int C, int H, int W, int OH, int OW, int KH,
                           int KW, int sh, int sw, int dh, int dw, int pht, int pwl, int kpad, long long total_units) {
  extern __shared__ int ktab[];  // per k: c | fy << 8 | fx << 16, or -1 past the filter
  const int kk = KH * KW * C;
  for (int k = threadIdx.x; k < kpad; k += 256) {
    int v = -1;
    if (k < kk) {
      const int tap = k / C, c = k - tap * C;
      const int fy = tap / KW, fx = tap - fy * KW;
      v = c | (fy << 8) | (fx << 16);
    }
    ktab[k] = v;
  }
  __syncthreads();
  const long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (u >= total_units) return;
  const int pieces = kpad / 16;
  const int piece = (int)(u % pieces);
  const long long row = u / pieces;
  const int xo = (int)(row % OW), yo = (int)((row / OW) % OH);
  const long long n = row / ((long long)OW * OH);
  const int y0 = yo * sh - pht, x0 = xo * sw - pwl;
  const T* xn = x + n * (long long)C * H * W;
  uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
  for (int b = 0; b < 16; ++b) {
    const int e = ktab[piece * 16 + b];
    if (e >= 0) {
      const int c = e & 0xff, iy = y0 + ((e >> 8) & 0xff) * dh, ix = x0 + (e >> 16) * dw;
      if (iy >= 0 && iy < H && ix >= 0 && ix < W)
        w[b >> 2] |= (uint32_t)to_u8(xn[((long long)c * H + iy) * W + ix]) << (8 * (b & 3));
    }
  }
  reinterpret_cast<uint4*>(a + row * kpad)[piece] = make_uint4(w[0], w[1], w[2], w[3]);
}

// im2col for few input channels and filters up to 8 taps wide, K order (fy, c, fx padded to 8): the eight input bytes
// of one (fy, c) segment are contiguous in the NCHW row, so a row of A is built from unaligned 8-byte reads instead of
// single bytes.  A block stages the input rows of a band of output rows in shared memory (zero padding included),
// then every thread assembles 16-byte pieces (two segments) with three aligned word reads and two funnel shifts per
// segment.  The eighth byte of a segment is whatever pixel follows; its filter weight is zero.
template <typename T>
__global__ void __launch_bounds__(256)
im2col_few_channels_kernel(const T* __restrict__ x, uint8_t* __restrict__ a, int C, int H, int W, int OH, int OW, int KH,
                           int sh, int sw, int pht, int pwl, int kpad, int band, int wpad, int pwl_s) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // a dependent convolution may set itself up meanwhile
  extern __shared__ __align__(16) uint8_t tile[];  // [C][rows_in][wpad]
  const int n = blockIdx.y, oy0 = blockIdx.x * band;
  const int rows_out = min(band, OH - oy0);
  const int rows_in = (rows_out - 1) * sh + KH;
  const int iy0 = oy0 * sh - pht;
  // ---- fill (zeros first, then the valid parts of the rows)
  const int tile_words = C * rows_in * wpad / 4;
  for (int i = threadIdx.x; i < tile_words; i += 256) reinterpret_cast<uint32_t*>(tile)[i] = 0u;
  __syncthreads();
  const T* xn = x + (long long)n * C * H * W;
  if ((W & 3) == 0) {
    const int wq = W / 4;
    for (int i = threadIdx.x; i < C * rows_in * wq; i += 256) {
      const int q = i % wq, cr = i / wq;
      const int r = cr % rows_in, c = cr / rows_in;
      const int iy = iy0 + r;
      if (iy >= 0 && iy < H)
        *reinterpret_cast<uint32_t*>(tile + (c * rows_in + r) * wpad + pwl_s + 4 * q) = ld4_as_bytes(xn + ((long long)c * H + iy) * W + 4 * q);
    }
  } else {
    for (int i = threadIdx.x; i < C * rows_in * W; i += 256) {
      const int q = i % W, cr = i / W;
      const int r = cr % rows_in, c = cr / rows_in;
      const int iy = iy0 + r;
      if (iy >= 0 && iy < H) tile[(c * rows_in + r) * wpad + pwl_s + q] = to_u8(xn[((long long)c * H + iy) * W + q]);
    }
  }
  __syncthreads();
  // ---- rows of A: piece = 16 bytes = two (fy, c) segments
  const int ppr = kpad / 16, nseg = KH * C;
  uint8_t* an = a + ((long long)n * OH + oy0) * OW * kpad;
  for (int i = threadIdx.x; i < rows_out * OW * ppr; i += 256) {
    const int pp = i % ppr, rl = i / ppr;
    const int ox = rl % OW, oyl = rl / OW;
    const int xs = ox * sw - pwl + pwl_s;  // window start in tile columns
    const int sh8 = (xs & 3) * 8;
    uint32_t w[4];
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      const int seg = 2 * pp + g;
      uint32_t lo = 0, hi = 0;
      if (seg < nseg) {
        const int fy = seg / C, c = seg - fy * C;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(tile + (c * rows_in + oyl * sh + fy) * wpad + (xs & ~3));
        const uint32_t w0 = src[0], w1 = src[1], w2 = src[2];
        lo = __funnelshift_r(w0, w1, sh8);
        hi = __funnelshift_r(w1, w2, sh8);
      }
      w[2 * g] = lo;
      w[2 * g + 1] = hi;
    }
    *reinterpret_cast<uint4*>(an + (long long)rl * kpad + pp * 16) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// ------------------------------------------------------------------------------------------- Lut / MulShift / Mul
// tpu.Lut (Lut.cpp:20-32): out = table[x mod 256].  The 256-entry table sits in shared memory; 8-bit tensors move as
// 16-byte words (16 look-ups per thread).
template <typename E>
__global__ void __launch_bounds__(256)
lut_kernel(const uint8_t* __restrict__ x, long long n, const E* __restrict__ table, E* __restrict__ out, int vec16) {
  __shared__ E tab[256];
  tab[threadIdx.x] = table[threadIdx.x];
  __syncthreads();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (sizeof(E) == 1 && vec16) {
    const long long n16 = n / 16;
    if (i < n16) {
      const uint4 v = reinterpret_cast<const uint4*>(x)[i];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        o[k] = (uint32_t)tab[w[k] & 0xff] | ((uint32_t)tab[(w[k] >> 8) & 0xff] << 8) |
               ((uint32_t)tab[(w[k] >> 16) & 0xff] << 16) | ((uint32_t)tab[w[k] >> 24] << 24);
      reinterpret_cast<uint4*>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    const long long t = n16 * 16 + i;  // the tail, one element per thread of the first blocks
    if (i < n - n16 * 16) out[t] = tab[x[t]];
  } else {
    if (i < n) out[i] = tab[x[i]];
  }
}

// tpu.MulShift (MulShift.cpp:19-41): out = saturate(RSR((x - in_zp) * m, s, half-up) + out_zp)
__global__ void __launch_bounds__(256)
mulshift_i8_kernel(const void* __restrict__ x, int dt, long long n, int m, int sft, int in_zp, int out_zp, int out_dt,
                   void* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t v = rshift_round((int64_t)(ld_q(x, i, dt) - in_zp) * m, sft, B200Q_ROUND_HALF_UP) + out_zp;
  st_q(out, i, out_dt, (int32_t)clamp_dtype(v, out_dt));
}

// tpu.AddConst with a uniform-quantized output (AddConst.cpp:26-47): sum = (x - in_zp) * m; sum += const_val (a double,
// truncated toward zero where applyMultiplierAndRShift takes it as an int64); out = saturate(relu(RSR(sum, s, half-up))).
// With const_val = 0 and in_zp = 0 this is the symmetric tpu.MulConst (MulConst.cpp:50-62).
__global__ void __launch_bounds__(256)
addconst_i8_kernel(const void* __restrict__ x, int dt, long long n, int m, double const_val, int sft, int in_zp, int do_relu,
                   int out_dt, void* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const double sum = (double)((int64_t)(ld_q(x, i, dt) - in_zp) * m) + const_val;
  int64_t v = rshift_round((int64_t)sum, sft, B200Q_ROUND_HALF_UP);
  if (do_relu && v < 0) v = 0;
  st_q(out, i, out_dt, (int32_t)clamp_dtype(v, out_dt));
}

// tpu.RequantFp (lib/Dialect/Tpu/Interfaces/Common/RequantFp.cpp:17-66) to an integer type.  The input is the float the reference's
// interpreter holds (an int32 tensor is converted the way its storage converts it).  tflite != 0: to_int(x * scale) + zp (TFLite,
// TFLite_LShift); else to_int(x * scale + offset) (MultiplierShift); a float multiply and a float add, not fused.
__global__ void __launch_bounds__(256)
requant_fp_kernel(const void* __restrict__ x, int in_is_i32, long long n, float scale, float offset, int zp, int tflite, int rmode,
                  int out_dt, void* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = in_is_i32 ? (float)static_cast<const int32_t*>(x)[i] : static_cast<const float*>(x)[i];
  int64_t r;
  if (tflite) r = (int64_t)(int32_t)to_int_f32(__fmul_rn(v, scale), rmode) + zp;
  else r = (int32_t)to_int_f32(__fadd_rn(__fmul_rn(v, scale), offset), rmode);
  st_q(out, i, out_dt, (int32_t)clamp_dtype((int64_t)(int32_t)r, out_dt));
}

// tpu.PRelu (lib/Dialect/Tpu/Interfaces/Common/PRelu.cpp:35-88).  8-bit symmetric: a negative input becomes
// saturate(RSR(x * slope[c], rshift, half-up)) with int8 slopes, anything else passes through; c = (i / inner) % num_slope.
__global__ void __launch_bounds__(256)
prelu_i8_kernel(const void* __restrict__ x, int dt, const int8_t* __restrict__ slope, long long n, long long inner, int num_slope,
                int sft, int out_dt, void* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int v = ld_q(x, i, dt);
  int64_t r = v;
  if (v < 0) r = clamp_dtype(rshift_round((int64_t)v * slope[(i / inner) % num_slope], sft, B200Q_ROUND_HALF_UP), out_dt);
  st_q(out, i, out_dt, (int32_t)r);
}

// the float form is the library PReLU the reference calls (lib/Support/Dnnl/PRelu.cpp): x > 0 ? x : x * slope[c]
__global__ void __launch_bounds__(256)
prelu_f32_kernel(const float* __restrict__ x, const float* __restrict__ slope, long long n, long long inner, int num_slope,
                 float* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = x[i];
  out[i] = v > 0.f ? v : __fmul_rn(v, slope[(i / inner) % num_slope]);
}

// tpu.Mul, symmetric 8-bit tensors of equal shape (Mul.cpp:23-29,:72-85): the ReLU acts on the product, then
// out = saturate(RSR(prod * m, s, half-up))
__global__ void __launch_bounds__(256)
mul_i8_kernel(const void* __restrict__ a, int a_dt, const void* __restrict__ b, int b_dt, long long n, int m, int sft,
              int do_relu, int out_dt, void* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int64_t prod = (int64_t)ld_q(a, i, a_dt) * ld_q(b, i, b_dt);
  if (do_relu && prod < 0) prod = 0;
  const int64_t v = rshift_round(prod * m, sft, B200Q_ROUND_HALF_UP);
  st_q(out, i, out_dt, (int32_t)clamp_dtype(v, out_dt));
}

// ------------------------------------------------------------------------------------------- NHWC-resident graphs
// [N][H][W][C] -> the interior of the zero-bordered [N][H+2bh][W+2bw][C] (16 channels per thread)
__global__ void __launch_bounds__(256)
nhwc_to_bordered_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, long long total16, int c16, int H, int W, int bh, int bw) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // a dependent convolution may set itself up meanwhile
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total16) return;
  const int c = (int)(i % c16);
  const long long p = i / c16;
  const int w = (int)(p % W);
  const long long t = p / W;
  const int h = (int)(t % H);
  const long long n = t / H;
  y[((n * (H + 2 * bh) + h + bh) * (W + 2 * bw) + w + bw) * c16 + c] = x[i];
}

// 8-bit max pooling on NHWC: one thread per (output pixel, 16 channels)
template <bool SIGNED>
__global__ void __launch_bounds__(256)
maxpool_nhwc_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, long long total16, int c16, int ih, int iw, int kh, int kw,
                    int sh, int sw, int pht, int pwl, int oh, int ow, int do_relu) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // a dependent convolution may set itself up meanwhile
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total16) return;
  const int c = (int)(i % c16);
  const long long p = i / c16;
  const int xo = (int)(p % ow);
  const long long t = p / ow;
  const int yo = (int)(t % oh);
  const long long n = t / oh;
  const int y0 = yo * sh - pht, x0 = xo * sw - pwl;
  const uint32_t lowest = SIGNED ? 0x80808080u : 0u;
  uint32_t b0 = lowest, b1 = lowest, b2 = lowest, b3 = lowest;
  for (int fy = max(0, -y0); fy < min(kh, ih - y0); ++fy)
    for (int fx = max(0, -x0); fx < min(kw, iw - x0); ++fx) {
      const uint4 v = x[((n * ih + y0 + fy) * iw + x0 + fx) * c16 + c];
      if (SIGNED) {
        b0 = __vmaxs4(b0, v.x); b1 = __vmaxs4(b1, v.y); b2 = __vmaxs4(b2, v.z); b3 = __vmaxs4(b3, v.w);
      } else {
        b0 = __vmaxu4(b0, v.x); b1 = __vmaxu4(b1, v.y); b2 = __vmaxu4(b2, v.z); b3 = __vmaxu4(b3, v.w);
      }
    }
  if (SIGNED && do_relu) {
    b0 = __vmaxs4(b0, 0u); b1 = __vmaxs4(b1, 0u); b2 = __vmaxs4(b2, 0u); b3 = __vmaxs4(b3, 0u);
  }
  y[i] = make_uint4(b0, b1, b2, b3);
}

// average pooling over the whole kh x kw window grid on NHWC (Pool2D.cpp:162-200: the window sum, MultiplierShift
// half-up, optional ReLU, saturate); one thread per (output pixel, channel), channels along the warp
__global__ void __launch_bounds__(256)
avgpool_nhwc_kernel(const void* __restrict__ x, int dt, long long total, int C, int ih, int iw, int kh, int kw, int sh, int sw,
                    int pht, int pwl, int oh, int ow, int multi, int rshift, int do_relu, int out_dt, void* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = (int)(i % C);
  const long long p = i / C;
  const int xo = (int)(p % ow);
  const long long t = p / ow;
  const int yo = (int)(t % oh);
  const long long n = t / oh;
  const int y0 = yo * sh - pht, x0 = xo * sw - pwl;
  int64_t sum = 0;
  for (int fy = max(0, -y0); fy < min(kh, ih - y0); ++fy)
    for (int fx = max(0, -x0); fx < min(kw, iw - x0); ++fx) sum += ld_q(x, ((n * ih + y0 + fy) * iw + x0 + fx) * C + c, dt);
  int64_t v = rshift_round(sum * multi, rshift, B200Q_ROUND_HALF_UP);
  if (do_relu && v < 0) v = 0;
  st_q(out, i, out_dt, (int32_t)clamp_dtype(v, out_dt));
}

inline unsigned nblk(long long n, int t) { return (unsigned)((n + t - 1) / t); }

}  // namespace

int requant_axis_launch(const int32_t* x, long long outer, int C, long long inner, const int32_t* mult,
                        const int32_t* shift, const int32_t* zp, int per_channel, int in_zp, const Epilogue& e, void* out,
                        cudaStream_t s) {
  const long long total = outer * C * inner;
  if (total == 0) return B200Q_OK;
  requant_axis_kernel<<<nblk(total, 256), 256, 0, s>>>(x, total, C, inner, mult, shift, zp, per_channel, in_zp, e, out);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int add_i8_launch(const void* a, int a_dt, const void* b, int b_dt, long long n, int m0, int s0, int m1, int s1,
                  int do_relu, int out_dt, void* out, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  const bool q8 = a_dt <= B200Q_DT_U8 && b_dt <= B200Q_DT_U8 && out_dt <= B200Q_DT_U8;
  const bool al = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 3) == 0;
  const bool al16 = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  const bool small = m0 > -(1 << 23) && m0 < (1 << 23) && m1 > -(1 << 23) && m1 < (1 << 23) && s0 >= 1 && s0 <= 31 &&
                     s1 >= 1 && s1 <= 31;
  if (q8 && al16 && small && n % 16 == 0) {
    // output range with the ReLU floor folded in
    const int lo = out_dt == B200Q_DT_U8 ? 0 : (do_relu ? 0 : -128), hi = out_dt == B200Q_DT_U8 ? 255 : 127;
    const long long n16 = n / 16;
    const bool au = a_dt == B200Q_DT_U8, bu = b_dt == B200Q_DT_U8;
    const uint4 *pa = (const uint4*)a, *pb = (const uint4*)b;
    uint4* po = (uint4*)out;
    if (au && bu) add_i8x16_kernel<true, true><<<nblk(n16, 256), 256, 0, s>>>(pa, pb, n16, m0, s0, m1, s1, lo, hi, po);
    else if (au) add_i8x16_kernel<true, false><<<nblk(n16, 256), 256, 0, s>>>(pa, pb, n16, m0, s0, m1, s1, lo, hi, po);
    else if (bu) add_i8x16_kernel<false, true><<<nblk(n16, 256), 256, 0, s>>>(pa, pb, n16, m0, s0, m1, s1, lo, hi, po);
    else add_i8x16_kernel<false, false><<<nblk(n16, 256), 256, 0, s>>>(pa, pb, n16, m0, s0, m1, s1, lo, hi, po);
  } else if (q8 && al && n % 4 == 0) {
    add_i8x4_kernel<<<nblk(n / 4, 256), 256, 0, s>>>((const uint32_t*)a, a_dt == B200Q_DT_U8, (const uint32_t*)b,
                                                     b_dt == B200Q_DT_U8, n / 4, m0, s0, m1, s1, do_relu, out_dt, (uint32_t*)out);
  } else {
    add_i8_kernel<<<nblk(n, 256), 256, 0, s>>>(a, a_dt, b, b_dt, n, m0, s0, m1, s1, do_relu, out_dt, out);
  }
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int constop_i8_launch(int form, const void* x, int dt, long long n, int m, double const_val, int sft, int in_zp, int do_relu, float relu_limit,
                      int out_dt, void* out, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  constop_i8_kernel<<<nblk(n, 256), 256, 0, s>>>(form, x, dt, n, m, const_val, sft, in_zp, do_relu, relu_limit, out_dt, out);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int sub_i8_launch(const void* a, int a_dt, const void* b, int b_dt, long long n, int m0, int s0, int m1, int s1, int do_relu, int out_dt,
                  void* out, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  sub_i8_kernel<<<nblk(n, 256), 256, 0, s>>>(a, a_dt, b, b_dt, n, m0, s0, m1, s1, do_relu, out_dt, out);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int pool2d_i8_launch(const void* x, int dt, int NC, int ih, int iw, int kh, int kw, int sh, int sw, int pht, int phb,
                     int pwl, int pwr, int mode, int multi, int rshift, int do_relu, int out_dt, void* out, cudaStream_t s) {
  const int oh = (ih + pht + phb - kh) / sh + 1, ow = (iw + pwl + pwr - kw) / sw + 1;
  const long long total = (long long)NC * oh * ow;
  if (total <= 0) return B200Q_OK;
  if (mode == 0 && dt == out_dt && (dt == B200Q_DT_I8 || dt == B200Q_DT_U8) && (long long)ih * iw <= 48 * 1024 && NC > 0) {
    const size_t smem = (size_t)ih * iw;
    if (dt == B200Q_DT_I8)
      maxpool_q8_plane_kernel<int8_t><<<(unsigned)NC, 256, smem, s>>>((const int8_t*)x, ih, iw, kh, kw, sh, sw, pht, pwl, oh, ow,
                                                                      do_relu, (int8_t*)out);
    else
      maxpool_q8_plane_kernel<uint8_t><<<(unsigned)NC, 256, smem, s>>>((const uint8_t*)x, ih, iw, kh, kw, sh, sw, pht, pwl, oh, ow,
                                                                       do_relu, (uint8_t*)out);
    CUDA_TRY(cudaGetLastError());
    return B200Q_OK;
  }
  if (mode == 0 && dt == out_dt && (dt == B200Q_DT_I8 || dt == B200Q_DT_U8)) {
    if (dt == B200Q_DT_I8)
      maxpool_q8_kernel<int8_t><<<nblk(total, 256), 256, 0, s>>>((const int8_t*)x, total, ih, iw, kh, kw, sh, sw, pht, pwl, oh, ow,
                                                                 do_relu, (int8_t*)out);
    else
      maxpool_q8_kernel<uint8_t><<<nblk(total, 256), 256, 0, s>>>((const uint8_t*)x, total, ih, iw, kh, kw, sh, sw, pht, pwl, oh,
                                                                  ow, do_relu, (uint8_t*)out);
    CUDA_TRY(cudaGetLastError());
    return B200Q_OK;
  }
  pool2d_i8_kernel<<<nblk(total, 256), 256, 0, s>>>(x, dt, NC, ih, iw, kh, kw, sh, sw, pht, pwl, oh, ow, mode, multi, rshift,
                                                    do_relu, out_dt, out);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int cast_f32_q8_launch(const float* x, long long n, double scale, int zp, int rmode, int out_dt, void* out, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  if (out_dt <= B200Q_DT_U8 && n % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 3) == 0)
    cast_f32_q8x4_kernel<<<nblk(n / 4, 256), 256, 0, s>>>((const float4*)x, n / 4, (float)(1.0 / scale), zp, rmode, out_dt,
                                                          (uint32_t*)out);
  else
    cast_f32_q8_kernel<<<nblk(n, 256), 256, 0, s>>>(x, n, (float)(1.0 / scale), zp, rmode, out_dt, out);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int cast_q8_f32_launch(const void* x, int dt, long long n, double scale, int zp, float* out, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  cast_q8_f32_kernel<<<nblk(n, 256), 256, 0, s>>>(x, dt, n, (float)scale, zp, out);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int im2col_nhwc_launch(const void* x, void* a, long long N, int C, int Hp, int Wp, int OH, int OW, int KH, int KW, int sh,
                       int sw, int dh, int dw, int oy0, int ox0, int kpad, cudaStream_t s) {
  const bool v16 = (C % 16 == 0) && (kpad % 16 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(a) & 15) == 0);
  const long long units = N * OH * OW * KH * KW * (v16 ? C / 16 : 1);
  if (units == 0) return B200Q_OK;
  if ((units + 255) / 256 > 0x7fffffffLL) return set_error(B200Q_ERR_UNSUPPORTED, "im2col: too large");
  im2col_nhwc_kernel<<<nblk(units, 256), 256, 0, s>>>((const uint8_t*)x, (uint8_t*)a, C, Hp, Wp, OH, OW, KH, KW, sh, sw, dh,
                                                      dw, oy0, ox0, kpad, units, v16 ? 16 : 1);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int im2col_nchw_small_c_launch(const void* x, int x_is_f32, void* a, long long N, int C, int H, int W, int OH, int OW, int KH,
                               int KW, int sh, int sw, int dh, int dw, int pht, int pwl, int kpad, cudaStream_t s) {
  if (kpad % 16 != 0 || (reinterpret_cast<uintptr_t>(a) & 15) != 0 || KH > 255 || KW > 255 || C > 255)
    return set_error(B200Q_ERR_INVALID, "im2col (small C): row length and buffer must be 16-byte aligned");
  const long long units = N * OH * OW * (kpad / 16);
  if (units == 0) return B200Q_OK;
  if ((units + 255) / 256 > 0x7fffffffLL) return set_error(B200Q_ERR_UNSUPPORTED, "im2col: too large");
  const size_t smem = (size_t)kpad * sizeof(int);
  if (x_is_f32)
    im2col_nchw_small_c_kernel<float><<<nblk(units, 256), 256, smem, s>>>((const float*)x, (uint8_t*)a, C, H, W, OH, OW, KH, KW,
                                                                            sh, sw, dh, dw, pht, pwl, kpad, units);
  else
    im2col_nchw_small_c_kernel<uint8_t><<<nblk(units, 256), 256, smem, s>>>((const uint8_t*)x, (uint8_t*)a, C, H, W, OH, OW, KH,
                                                                              KW, sh, sw, dh, dw, pht, pwl, kpad, units);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

// K order (fy, c, fx padded to 8), kpad = round16(KH*C*8).  Geometry limits are checked by im2col_few_channels_ok.
bool im2col_few_channels_ok(int C, int H, int W, int KH, int KW, int sh, int sw, int dh, int dw, int pwl, int OW) {
  if (C < 1 || C > 4 || KW > 8 || dh != 1 || dw != 1 || W < 1) return false;
  const int pwl_s = (pwl + 3) & ~3;
  const int wpad = ((max((OW - 1) * sw - pwl + pwl_s + 8, pwl_s + W) + 3) & ~3) + 4;
  const int rows_in = 7 * sh + KH;  // band of 8 output rows
  return (size_t)C * rows_in * wpad <= 96 * 1024;
}

int im2col_few_channels_launch(const void* x, int x_is_f32, void* a, long long N, int C, int H, int W, int OH, int OW, int KH,
                               int sh, int sw, int pht, int pwl, int kpad, cudaStream_t s) {
  if (N == 0) return B200Q_OK;
  if (N > 65535) return set_error(B200Q_ERR_UNSUPPORTED, "im2col (few channels): at most 65535 images per call");
  if ((reinterpret_cast<uintptr_t>(a) & 15) != 0 || kpad % 16 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0)
    return set_error(B200Q_ERR_INVALID, "im2col (few channels): buffers must be 16-byte aligned");
  const int band = 8;
  const int pwl_s = (pwl + 3) & ~3;
  const int wpad = ((max((OW - 1) * sw - pwl + pwl_s + 8, pwl_s + W) + 3) & ~3) + 4;  // + one word: the third read of a window
  const size_t smem = (size_t)C * ((band - 1) * sh + KH) * wpad;
  dim3 grid((OH + band - 1) / band, (unsigned)N);
  if (x_is_f32) {
    auto k = im2col_few_channels_kernel<float>;
    if (smem > 48 * 1024) CUDA_TRY(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k<<<grid, 256, smem, s>>>((const float*)x, (uint8_t*)a, C, H, W, OH, OW, KH, sh, sw, pht, pwl, kpad, band, wpad, pwl_s);
  } else {
    auto k = im2col_few_channels_kernel<uint8_t>;
    if (smem > 48 * 1024) CUDA_TRY(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k<<<grid, 256, smem, s>>>((const uint8_t*)x, (uint8_t*)a, C, H, W, OH, OW, KH, sh, sw, pht, pwl, kpad, band, wpad, pwl_s);
  }
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int lut_launch(const void* x, long long n, const void* table, int elem_size, void* out, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  if (elem_size == 1) {
    const bool al = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    const long long threads = al ? (n / 16 > 16 ? n / 16 : 16) : n;  // vector form: at least the (< 16 element) tail
    lut_kernel<uint8_t><<<nblk(threads, 256), 256, 0, s>>>((const uint8_t*)x, n, (const uint8_t*)table, (uint8_t*)out, al ? 1 : 0);
  } else if (elem_size == 2) {
    lut_kernel<uint16_t><<<nblk(n, 256), 256, 0, s>>>((const uint8_t*)x, n, (const uint16_t*)table, (uint16_t*)out, 0);
  } else if (elem_size == 4) {
    lut_kernel<uint32_t><<<nblk(n, 256), 256, 0, s>>>((const uint8_t*)x, n, (const uint32_t*)table, (uint32_t*)out, 0);
  } else {
    return set_error(B200Q_ERR_INVALID, "lut: table entries are 1, 2 or 4 bytes");
  }
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int addconst_i8_launch(const void* x, int dt, long long n, int m, double const_val, int sft, int in_zp, int do_relu, int out_dt,
                       void* out, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  addconst_i8_kernel<<<nblk(n, 256), 256, 0, s>>>(x, dt, n, m, const_val, sft, in_zp, do_relu, out_dt, out);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int requant_fp_launch(const void* x, int in_is_i32, long long n, float scale, float offset, int zp, int tflite, int rmode, int out_dt,
                      void* out, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  requant_fp_kernel<<<nblk(n, 256), 256, 0, s>>>(x, in_is_i32, n, scale, offset, zp, tflite, rmode, out_dt, out);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int prelu_i8_launch(const void* x, int dt, const void* slope, long long n, long long inner, int num_slope, int sft, int out_dt, void* out,
                    cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  prelu_i8_kernel<<<nblk(n, 256), 256, 0, s>>>(x, dt, static_cast<const int8_t*>(slope), n, inner, num_slope, sft, out_dt, out);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int prelu_f32_launch(const float* x, const float* slope, long long n, long long inner, int num_slope, float* out, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  prelu_f32_kernel<<<nblk(n, 256), 256, 0, s>>>(x, slope, n, inner, num_slope, out);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int mulshift_i8_launch(const void* x, int dt, long long n, int m, int sft, int in_zp, int out_zp, int out_dt, void* out,
                       cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  mulshift_i8_kernel<<<nblk(n, 256), 256, 0, s>>>(x, dt, n, m, sft, in_zp, out_zp, out_dt, out);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int mul_i8_launch(const void* a, int a_dt, const void* b, int b_dt, long long n, int m, int sft, int do_relu, int out_dt,
                  void* out, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  mul_i8_kernel<<<nblk(n, 256), 256, 0, s>>>(a, a_dt, b, b_dt, n, m, sft, do_relu, out_dt, out);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int nhwc_to_bordered_launch(const void* x, void* y, long long N, int C, int H, int W, int bh, int bw, cudaStream_t s) {
  if (C % 16 != 0 || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) != 0)
    return set_error(B200Q_ERR_UNSUPPORTED, "nhwc_to_bordered: channels must be a multiple of 16 and the buffers 16-byte aligned");
  const long long total16 = N * H * W * (C / 16);
  if (total16 == 0) return B200Q_OK;
  nhwc_to_bordered_kernel<<<nblk(total16, 256), 256, 0, s>>>((const uint4*)x, (uint4*)y, total16, C / 16, H, W, bh, bw);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int pool2d_i8_nhwc_launch(const void* x, int dt, long long N, int C, int ih, int iw, int kh, int kw, int sh, int sw, int pht,
                          int phb, int pwl, int pwr, int mode, int multi, int rshift, int do_relu, int out_dt, void* out,
                          cudaStream_t s) {
  const int oh = (ih + pht + phb - kh) / sh + 1, ow = (iw + pwl + pwr - kw) / sw + 1;
  const long long total = N * oh * ow * C;
  if (total <= 0) return B200Q_OK;
  const bool al = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  if (mode == 0 && dt == out_dt && (dt == B200Q_DT_I8 || dt == B200Q_DT_U8) && C % 16 == 0 && al) {
    const long long t16 = total / 16;
    if (dt == B200Q_DT_I8)
      maxpool_nhwc_kernel<true><<<nblk(t16, 256), 256, 0, s>>>((const uint4*)x, (uint4*)out, t16, C / 16, ih, iw, kh, kw, sh, sw, pht,
                                                               pwl, oh, ow, do_relu);
    else
      maxpool_nhwc_kernel<false><<<nblk(t16, 256), 256, 0, s>>>((const uint4*)x, (uint4*)out, t16, C / 16, ih, iw, kh, kw, sh, sw, pht,
                                                                pwl, oh, ow, do_relu);
  } else if (mode == 1) {
    avgpool_nhwc_kernel<<<nblk(total, 256), 256, 0, s>>>(x, dt, total, C, ih, iw, kh, kw, sh, sw, pht, pwl, oh, ow, multi, rshift,
                                                         do_relu, out_dt, out);
  } else {
    return set_error(B200Q_ERR_UNSUPPORTED, "pool2d (NHWC): max pooling needs equal 8-bit types and channels %% 16 == 0");
  }
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

}  // namespace b200q
