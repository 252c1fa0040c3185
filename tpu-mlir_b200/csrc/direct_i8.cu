// CUDA-core INT8 convolution / GEMM for the shapes the tensor-core implicit GEMM does not take
// (channel counts that are not a multiple of 16, strides, dilation, groups, zero points, batched right
// operands).  One thread per output element, int32 accumulation, the same exact epilogue (requant.cuh); depthwise 3 x 3 and
// 5 x 5 convolutions have a kernel of their own (a patch of outputs per thread).
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

// RSR(a * m, s, half up) for 1 <= s <= 62, saturated to int32, in 32-bit operations: floor((a * m + 2^(s-1)) / 2^s)
// (the identity requant.cuh uses; |a * m| < 2^62, so adding the half cannot overflow).
__device__ __forceinline__ int rshift_half_up_sat32(int a, int m, int s, unsigned half_lo, int half_hi) {
  const unsigned lo = (unsigned)a * (unsigned)m;
  int hi = __mulhi(a, m);
  const unsigned lo2 = lo + half_lo;
  hi += half_hi + (lo2 < lo ? 1 : 0);
  const int k1 = s < 31 ? s : 31, k2 = s - k1;      // an arithmetic 64-bit shift by s as two shifts of at most 31
  const unsigned l1 = __funnelshift_r(lo2, (unsigned)hi, k1);
  const int h1 = hi >> k1;
  const unsigned l2 = __funnelshift_r(l1, (unsigned)h1, k2);
  const int h2 = h1 >> k2;
  return h2 == ((int)l2 >> 31) ? (int)l2 : (h2 < 0 ? (int)0x80000000 : 0x7fffffff);
}

template <bool XU>
__device__ __forceinline__ int dot4(uint32_t a, uint32_t b, int c) {   // four input bytes (u8 or s8) times four s8 weights
  int d;
  if (XU) asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  else asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// Depthwise convolution (groups == ic == oc), square K x K filter, stride S, no dilation: the memory-bound case of the
// mobile networks.  One thread owns a patch of R rows x 4 columns of one plane's output and walks the (R - 1) * S + K input
// rows the patch needs once.  A row is read as aligned 32-bit words, shifted to the window's first byte, its out-of-image
// bytes replaced by the pad value through a per-thread byte mask, and fed four bytes at a time to dp4a against the packed
// filter row (bytes a word holds beyond the filter's width meet zero weights); rows outside the image are the pad word.
// The words reach up to three bytes before the window and 4 * (NV + 1) bytes past its start, which lies inside the tensor
// for every patch but the few at its two ends; those (and a tensor that is not 4-byte aligned) take a compact
// one-output-at-a-time loop.  The code is kept small on purpose: fully unrolled tested byte loads and an inlined general
// requantisation made the first version wait on instruction fetch more than on anything else.
__device__ __noinline__ int requant_general(int a, int m, int s, const Epilogue& e) { return requant_value<-1, -1>(a, m, s, e); }

template <int K, int S, int R, int CW, bool FAST_RQ, bool XU>
__global__ void __launch_bounds__(256)
dwconv_i8_kernel(const uint8_t* __restrict__ x, long long x_bytes, const int8_t* __restrict__ w, ConvGeometry g, Epilogue e,
                 void* __restrict__ y, unsigned per_plane, unsigned planes_per_block, unsigned inv_per_plane, unsigned xq_per_row,
                 unsigned inv_xq) {
  // grid (blocks of one plane, channel groups, images): a plane with at most 256 patches shares its block with the next
  // channels' planes; divisions are multiplications by the reciprocals the launcher rounded up (exact for these ranges)
  unsigned pl = 0, rem = blockIdx.x * 256u + threadIdx.x;
  if (planes_per_block > 1) {
    pl = per_plane == 1 ? threadIdx.x : __umulhi(threadIdx.x, inv_per_plane);
    rem = threadIdx.x - pl * per_plane;
    if (pl >= planes_per_block) return;
  }
  const int c = (int)(blockIdx.y * planes_per_block + pl);
  if (c >= g.oc || rem >= per_plane) return;
  const unsigned plane = blockIdx.z * (unsigned)g.oc + (unsigned)c;     // n * C + c
  const int yt = (int)(xq_per_row == 1 ? rem : __umulhi(rem, inv_xq)), xq = (int)(rem - (unsigned)yt * xq_per_row);
  constexpr int ROWS = (R - 1) * S + K;
  constexpr int T = (K + 3) / 4, LASTB = (CW - 1) * S + 4 * (T - 1) + 3, NV = LASTB / 4 + 1;
  const int x0 = xq * CW, y0 = yt * R;
  const int ix0 = x0 * S - g.pwl, iy0 = y0 * S - g.pht;
  const int bias = e.bias ? e.bias[c] : 0;
  const int qi = e.per_channel ? c : 0;
  const int32_t m = e.multiplier ? e.multiplier[qi] : 1;
  const int32_t sft = e.shift ? e.shift[qi] : 0;
  const long long plane_off = (long long)plane * (g.ih * g.iw);
  const int iy_first = iy0 > 0 ? iy0 : 0, iy_last = iy0 + ROWS - 1 < g.ih - 1 ? iy0 + ROWS - 1 : g.ih - 1;
  const bool words_ok = plane_off + (long long)iy_first * g.iw + ix0 >= 0 &&
                        plane_off + (long long)iy_last * g.iw + ix0 + 4 * (NV + 1) <= x_bytes;
  if (!words_ok) {
    // the ends of the tensor: one output at a time, tested byte loads
    const uint8_t* xp = x + plane_off;
#pragma unroll 1
    for (int i = 0; i < R * CW; ++i) {
      const int yo = y0 + i / CW, xo = x0 + i % CW;
      if (yo >= g.oh || xo >= g.ow) continue;
      int a = bias;
#pragma unroll 1
      for (int f = 0; f < K * K; ++f) {
        const int iy = yo * S - g.pht + f / K, ix = xo * S - g.pwl + f % K;
        int v = g.pad_value;
        if ((unsigned)iy < (unsigned)g.ih && (unsigned)ix < (unsigned)g.iw) v = XU ? (int)xp[iy * g.iw + ix] : (int)(int8_t)xp[iy * g.iw + ix];
        a += v * (int)w[c * K * K + f];
      }
      if (e.relu == B200Q_RELU_BEFORE_REQUANT && a < 0) a = 0;
      st_q(y, ((long long)plane * g.oh + yo) * g.ow + xo, e.out_dtype, requant_general(a, m, sft, e));
    }
    return;
  }
  uint32_t wp[K][T];
#pragma unroll
  for (int i = 0; i < K; ++i)
#pragma unroll
    for (int t = 0; t < T; ++t) {
      uint32_t v = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b)
        if (4 * t + b < K) v |= (uint32_t)((int)w[c * K * K + i * K + 4 * t + b] & 255) << (8 * b);
      wp[i][t] = v;
    }
  // byte masks of the window's columns that lie inside the image, and the pad value in the others
  const uint32_t padw = (uint32_t)(g.pad_value & 255) * 0x01010101u;
  uint32_t keep[NV], fill[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    uint32_t k = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b)
      if ((unsigned)(ix0 + 4 * i + b) < (unsigned)g.iw) k |= 0xffu << (8 * b);
    keep[i] = k;
    fill[i] = padw & ~k;
  }
  int acc[R][CW];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int o = 0; o < CW; ++o) acc[r][o] = 0;
  const uintptr_t first = reinterpret_cast<uintptr_t>(x) + (uintptr_t)(plane_off + (long long)iy0 * g.iw + ix0);
#pragma unroll
  for (int rel = 0; rel < ROWS; ++rel) {
    uint32_t V[NV];
    if ((unsigned)(iy0 + rel) < (unsigned)g.ih) {
      const uintptr_t ap = first + (uintptr_t)((long long)rel * g.iw);
      const uint32_t* a32 = reinterpret_cast<const uint32_t*>(ap & ~(uintptr_t)3);
      const unsigned sh8 = (unsigned)(ap & 3) * 8;
      uint32_t W[NV + 1];
#pragma unroll
      for (int i = 0; i <= NV; ++i) W[i] = a32[i];
#pragma unroll
      for (int i = 0; i < NV; ++i) V[i] = (__funnelshift_r(W[i], W[i + 1], sh8) & keep[i]) | fill[i];
    } else {
#pragma unroll
      for (int i = 0; i < NV; ++i) V[i] = padw;
    }
    uint32_t word[CW][T];
#pragma unroll
    for (int o = 0; o < CW; ++o)
#pragma unroll
      for (int t = 0; t < T; ++t) {
        const int p_ = o * S + 4 * t;
        word[o][t] = (p_ % 4 == 0) ? V[p_ / 4] : __funnelshift_r(V[p_ / 4], V[(p_ / 4 + 1) < NV ? (p_ / 4 + 1) : (NV - 1)], 8 * (p_ % 4));
      }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int fy = rel - r * S;      // compile-time after unrolling
      if (fy >= 0 && fy < K) {
#pragma unroll
        for (int o = 0; o < CW; ++o)
#pragma unroll
          for (int t = 0; t < T; ++t) acc[r][o] = dot4<XU>(word[o][t], wp[fy][t], acc[r][o]);
      }
    }
  }
  const bool out8 = e.out_dtype == B200Q_DT_I8 || e.out_dtype == B200Q_DT_U8;
  // FAST_RQ (MultiplierShift, half up, 8-bit output): floor((a * m + 2^(s-1)) / 2^s) is the HIGH word of one 64-bit
  // multiply-add when the binary point sits at bit 32: for s >= 32 that is hi32(a * m + 2^(s-1)) >> (s - 32); for a smaller
  // s the multiplier is scaled by 2^(32-s) first, which is exact while it still fits 32 bits (|m| < 2^(s-1)).  The high
  // word cannot overflow, and the clamp bounds carry the zero point and the ReLU.  Other shifts and multipliers take the
  // 32-bit sequence above, other dialects the general function.
  int mode = 0;                                  // 0 general, 1 high-word form, 2 two-shift form
  int mx = m, post = 0;
  long long half64 = 0;
  if (FAST_RQ && sft >= 32 && sft <= 62) {
    mode = 1;
    half64 = 1ll << (sft - 1);
    post = sft - 32;
  } else if (FAST_RQ && sft >= 1 && sft <= 31) {
    const int lim = 1 << (sft - 1);
    if (m > -lim && m < lim) {
      mode = 1;
      mx = m * (1 << (32 - sft));               // |m| < 2^(s-1): the product stays below 2^31
      half64 = 1ll << 31;
    } else {
      mode = 2;
    }
  }
  const unsigned half_lo = (mode == 2) ? (1u << (sft - 1)) : 0u;
  const int q_lo = e.out_dtype == B200Q_DT_U8 ? 0 : -128, q_hi = e.out_dtype == B200Q_DT_U8 ? 255 : 127;
  const int ozp = e.out_zp;
  const bool relu_before = e.relu == B200Q_RELU_BEFORE_REQUANT;
  const int floor_q = (e.relu == B200Q_RELU_AFTER_REQUANT && ozp > q_lo) ? ozp : q_lo;
  const int b_lo = floor_q - ozp, b_hi = q_hi - ozp;      // bounds of the value before the zero point is added
  // the form is chosen once per thread, outside the unrolled loops (inside, every output paid its own tests and branches)
  int q[R][CW];
  if (mode == 1) {
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int o = 0; o < CW; ++o) {
        int a = acc[r][o] + bias;
        if (relu_before) a = max(a, 0);
        const int v = (int)(((long long)a * mx + half64) >> 32) >> post;
        q[r][o] = min(min(max(v, b_lo), b_hi) + ozp, q_hi);      // the last bound acts only when the zero point lies above the type
      }
  } else if (mode == 2) {
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int o = 0; o < CW; ++o) {
        int a = acc[r][o] + bias;
        if (relu_before) a = max(a, 0);
        const int v = rshift_half_up_sat32(a, m, sft, half_lo, 0);
        q[r][o] = min(min(max(max(min(v, 1 << 24), -(1 << 24)), b_lo), b_hi) + ozp, q_hi);
      }
  } else {
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int o = 0; o < CW; ++o) {
        int a = acc[r][o] + bias;
        if (relu_before) a = max(a, 0);
        q[r][o] = requant_general(a, m, sft, e);
      }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int yo = y0 + r;
    if (yo >= g.oh) break;
    const long long at = ((long long)plane * g.oh + yo) * g.ow + x0;
#pragma unroll
    for (int j = 0; j < CW; j += 4) {
      if (out8 && x0 + j + 3 < g.ow && ((at + j) & 3) == 0) {
        const uint32_t lo16 = __byte_perm((uint32_t)q[r][j], (uint32_t)q[r][j + 1], 0x0040), hi16 = __byte_perm((uint32_t)q[r][j + 2], (uint32_t)q[r][j + 3], 0x0040);
        reinterpret_cast<uint32_t*>(y)[(at + j) >> 2] = __byte_perm(lo16, hi16, 0x5410);
      } else {
#pragma unroll
        for (int o = j; o < j + 4; ++o)
          if (x0 + o < g.ow) st_q(y, at + o, e.out_dtype, q[r][o]);
      }
    }
  }
}

template <int K, int S, int R, int CW>
int dwconv_launch_krs(const void* x, int x_unsigned, const int8_t* w, const ConvGeometry& g, const Epilogue& epi, void* y, cudaStream_t stream) {
  const unsigned xq = (unsigned)((g.ow + CW - 1) / CW), yt = (unsigned)((g.oh + R - 1) / R);
  const unsigned per_plane = xq * yt;
  if ((long long)g.n * g.oc * per_plane == 0) return B200Q_OK;
  const unsigned ppb = per_plane <= 128 ? 256u / per_plane : 1u;      // planes per block
  const dim3 grid(ppb > 1 ? 1u : (per_plane + 255u) / 256u, ((unsigned)g.oc + ppb - 1) / ppb, (unsigned)g.n);
  if (grid.y > 65535u || grid.z > 65535u) return set_error(B200Q_ERR_UNSUPPORTED, "depthwise conv: more than 65535 channel groups or images");
  // ceil(2^32 / d): __umulhi(v, that) == v / d while v * (d - 1) < 2^32; v stays below 2^16 here (d == 1 is tested apart)
  auto recip = [](unsigned d) { return d <= 1 ? 0u : (unsigned)((0x100000000ull + d - 1) / d); };
  if (per_plane >= 65536u) return set_error(B200Q_ERR_UNSUPPORTED, "depthwise conv: plane too large");
  const bool fast = epi.dialect == B200Q_RQ_MULTIPLIER_SHIFT && epi.round_mode == B200Q_ROUND_HALF_UP &&
                    (epi.out_dtype == B200Q_DT_I8 || epi.out_dtype == B200Q_DT_U8);
  // the word-wise path needs a 4-byte aligned tensor; a misaligned one takes the tested byte loads everywhere (x_bytes = 0)
  const long long x_bytes = (reinterpret_cast<uintptr_t>(x) & 3) == 0 ? (long long)g.n * g.ic * g.ih * g.iw : 0;
  const uint8_t* xb = static_cast<const uint8_t*>(x);
  const unsigned ipp = recip(per_plane), ixq = recip(xq);
  if (fast && x_unsigned) dwconv_i8_kernel<K, S, R, CW, true, true><<<grid, 256, 0, stream>>>(xb, x_bytes, w, g, epi, y, per_plane, ppb, ipp, xq, ixq);
  else if (fast) dwconv_i8_kernel<K, S, R, CW, true, false><<<grid, 256, 0, stream>>>(xb, x_bytes, w, g, epi, y, per_plane, ppb, ipp, xq, ixq);
  else if (x_unsigned) dwconv_i8_kernel<K, S, R, CW, false, true><<<grid, 256, 0, stream>>>(xb, x_bytes, w, g, epi, y, per_plane, ppb, ipp, xq, ixq);
  else dwconv_i8_kernel<K, S, R, CW, false, false><<<grid, 256, 0, stream>>>(xb, x_bytes, w, g, epi, y, per_plane, ppb, ipp, xq, ixq);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

// 1 = launched, 0 = not a shape this kernel takes
template <int K, int S>
int dwconv_launch_ks(const void* x, int x_unsigned, const int8_t* w, const ConvGeometry& g, const Epilogue& epi, void* y, cudaStream_t stream,
                     int* rc) {
  // four columns per thread: eight (CW = 8) were measured slower on 56- and 112-wide planes (79 registers instead of 58)
  if (g.oh >= 12) *rc = dwconv_launch_krs<K, S, 4, 4>(x, x_unsigned, w, g, epi, y, stream);
  else *rc = dwconv_launch_krs<K, S, 2, 4>(x, x_unsigned, w, g, epi, y, stream);
  return 1;
}

int dwconv_try(const void* x, int x_unsigned, const int8_t* w, const ConvGeometry& g, const Epilogue& epi, void* y, cudaStream_t stream, int* rc) {
  if (g.groups != g.ic || g.oc != g.ic || g.kh != g.kw || g.sh != g.sw || g.dh != 1 || g.dw != 1) return 0;
  if ((long long)g.ih * g.iw > 0x3fffffffLL) return 0;
  if (g.kh == 3 && g.sh == 1) return dwconv_launch_ks<3, 1>(x, x_unsigned, w, g, epi, y, stream, rc);
  if (g.kh == 3 && g.sh == 2) return dwconv_launch_ks<3, 2>(x, x_unsigned, w, g, epi, y, stream, rc);
  if (g.kh == 5 && g.sh == 1) return dwconv_launch_ks<5, 1>(x, x_unsigned, w, g, epi, y, stream, rc);
  if (g.kh == 5 && g.sh == 2) return dwconv_launch_ks<5, 2>(x, x_unsigned, w, g, epi, y, stream, rc);
  return 0;
}

}  // namespace

int conv2d_i8_direct_launch(const void* x, int x_unsigned, const int8_t* w, const ConvGeometry& g, const Epilogue& epi,
                            void* y, cudaStream_t stream) {
  const long long total = (long long)g.n * g.oc * g.oh * g.ow;
  if (total == 0) return B200Q_OK;
  int rc = B200Q_OK;
  if (dwconv_try(x, x_unsigned, w, g, epi, y, stream, &rc)) return rc;
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
