// fp32 forward of the Top-dialect ops a calibration pass runs: Conv (+ bias, ReLU), MatMul, Add, MaxPool, AvgPool, Relu.
//
// Semantics: top::ConvOp::inference (lib/Dialect/Top/Interfaces/Conv.cpp:222-231: fp32 convolution, bias, optional ReLU
// with relu_limit), top::MatMulOp, top::AddOp::inference (Add.cpp:45-85), top::MaxPoolOp / top::AvgPoolOp (the pooling
// of lib/Support/Dnnl/Pool.cpp: pad value -inf for max, count_include_pad for avg), top::ReluOp (Relu.cpp:17-24 over
// function_relu, lib/Support/MathUtils.cpp:891-903).  Tensors are NCHW fp32 like the interpreter's buffers.
//
// The convolution is an implicit GEMM on the CUDA cores in full fp32 (calibration statistics should not depend on a
// reduced-precision product): C[co][pixel] = sum_k Wt[k][co] * X[k][pixel], k = (c, kh, kw).  A block computes 128 (or
// 64) output channels x 128 pixels, K in slices of 8 through a four-stage ring in shared memory; a thread owns 8 x 8 (4 x 8)
// results; the tiles travel by cp.async, three slices ahead.  The weight is kept transposed [K][oc] so its tile loads
// are contiguous; the activation tile is gathered
// with a per-k table (offset of (c, kh, kw) inside an image and the two shifts for the border test), the pixel's own
// decomposition (image, row, column) is computed once per thread.  In NCHW consecutive pixels are consecutive
// addresses for a fixed k, so both the gather and the store run along the fast axis.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "internal.h"
#include "requant.cuh"
#include "top_f32.h"

namespace b200q {
namespace {

constexpr int TN = 128;   // pixels per block
constexpr int TK = 8;     // k per slice
constexpr int CONV_THREADS = 256;
constexpr int STAGES = 4;   // slices of K in flight (shared memory: 4 x 8 KB at 128 output channels)

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// asynchronous global -> shared copies; src_bytes < the copy size zero-fills the rest (0: nothing is read)
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ float relu_f(float v, int do_relu, float limit) {
  if (do_relu) {
    v = v > 0.f ? v : 0.f;
    if (limit > 0.f && v > limit) v = limit;
  }
  return v;
}

// KHW: 1 = 1x1 filter, 9 = 3x3 filter (the position of k inside the image comes from arithmetic on k, so the gather
// does not wait for a table entry first); 0 = any filter, through the table.
template <int TM, int KHW>
__global__ void __launch_bounds__(CONV_THREADS) conv2d_f32_kernel(const float* __restrict__ x, const float* __restrict__ wt,
                                                                   const int2* __restrict__ ktab, const float* __restrict__ bias,
                                                                   float* __restrict__ y, const TopConvPlan p) {
  constexpr int RM = TM / 16;   // output channels per thread: 8 or 4
  __shared__ __align__(16) float As[STAGES][TK][TM];
  __shared__ __align__(16) float Bs[STAGES][TK][TN];
  const int tid = threadIdx.x;
  // blockIdx.z = group * splits + split: with splits > 1 every split sums its own range of K into its own plane of the
  // output buffer (which is then a workspace: no bias, no ReLU; splitk_reduce_kernel adds the planes in a fixed order)
  const int g = blockIdx.z / p.splits, split = blockIdx.z - g * p.splits;
  const int k_begin = split * p.k_per_split, k_end = min(p.K, k_begin + p.k_per_split);
  const int co0 = blockIdx.y * TM;                 // inside the group
  const long long pix0 = (long long)blockIdx.x * TN;
  const int ohow = p.oh * p.ow;
  const long long P = (long long)p.n * ohow;
  const float* wg = wt + (size_t)g * p.K * p.ocg;

  // ---- this thread's pixel for the gather
  const int bp = tid & (TN - 1);
  const int bk = tid >> 7;                         // 0 / 1: k rows bk, bk + 2, bk + 4, bk + 6
  const long long pix = pix0 + bp;
  const bool pvalid = pix < P;
  int hi0 = 0, wi0 = 0;
  long long xbase = 0;
  if (pvalid) {
    const int b = (int)(pix / ohow), r = (int)(pix - (long long)b * ohow);
    const int ho = r / p.ow, wo = r - ho * p.ow;
    hi0 = ho * p.sh - p.pht;
    wi0 = wo * p.sw - p.pwl;
    xbase = ((long long)b * p.ic + (long long)g * p.icg) * p.ih * p.iw + (long long)hi0 * p.iw + wi0;
  }
  // ---- this thread's piece of the weight tile: one float4 of row ak
  constexpr int A_VECS = TK * TM / 4;              // 256 or 128
  const int ak = tid / (TM / 4), ac = (tid % (TM / 4)) * 4;
  const bool a_active = tid < A_VECS;
  const bool a_vec = (p.ocg & 3) == 0;

  // Tiles go from global to shared memory with cp.async (no staging registers), STAGES - 1 slices ahead of the
  // arithmetic: 16 bytes per thread of the weight tile, four 4-byte gathers of the activation tile whose source size
  // is 0 outside the image (the copy then writes zeros).
  auto issue = [&](int k0, int buf) {
    if (a_active) {
      const int k = k0 + ak;
      const uint32_t dst = smem_addr(&As[buf][ak][ac]);
      const float* src = wg + (size_t)(k < k_end ? k : 0) * p.ocg + co0 + ac;
      if (a_vec) {
        const bool ok = k < k_end && co0 + ac + 3 < p.ocg;
        cp_async_16(dst, ok ? src : wg, ok ? 16 : 0);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const bool ok = k < k_end && co0 + ac + e < p.ocg;
          cp_async_4(dst + 4 * e, ok ? src + e : wg, ok ? 4 : 0);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + bk + 2 * i;
      const float* src = x;
      int bytes = 0;
      if (pvalid && k < k_end) {
        int koff, khd, kwd;
        if (KHW == 1) {
          koff = k * p.ih * p.iw;
          khd = kwd = 0;
        } else if (KHW == 9) {
          const int c = k / 9, r = k - c * 9, a = r / 3, b = r - a * 3;
          khd = a * p.dh;
          kwd = b * p.dw;
          koff = c * p.ih * p.iw + khd * p.iw + kwd;
        } else {
          const int2 t = __ldg(ktab + k);
          koff = t.x;
          khd = t.y & 0xffff;
          kwd = t.y >> 16;
        }
        if ((unsigned)(hi0 + khd) < (unsigned)p.ih && (unsigned)(wi0 + kwd) < (unsigned)p.iw) {
          src = x + xbase + koff;
          bytes = 4;
        }
      }
      cp_async_4(smem_addr(&Bs[buf][bk + 2 * i][bp]), src, bytes);
    }
  };

  const int tx = tid & 15, ty = tid >> 4;
  float acc[RM][8];
#pragma unroll
  for (int i = 0; i < RM; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  const int nslices = (k_end - k_begin + TK - 1) / TK;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < nslices) issue(k_begin + s * TK, s);
    cp_async_commit();
  }
  for (int s = 0; s < nslices; ++s) {
    const int buf = s % STAGES;
    cp_async_wait<STAGES - 2>();   // slice s has landed (for this thread's copies; the barrier extends that to all)
    __syncthreads();               // ... and everybody is done with the buffer that the next copies overwrite
    if (s + STAGES - 1 < nslices) issue(k_begin + (s + STAGES - 1) * TK, (s + STAGES - 1) % STAGES);
    cp_async_commit();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[RM], b[8];
      {
        const float4 v = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
        a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
        if (RM == 8) {
          const float4 u = *reinterpret_cast<const float4*>(&As[buf][kk][(TM / 2) + ty * 4]);
          a[RM - 4] = u.x; a[RM - 3] = u.y; a[RM - 2] = u.z; a[RM - 1] = u.w;
        }
      }
      {
        const float4 v = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
        const float4 u = *reinterpret_cast<const float4*>(&Bs[buf][kk][64 + tx * 4]);
        b[0] = v.x; b[1] = v.y; b[2] = v.z; b[3] = v.w; b[4] = u.x; b[5] = u.y; b[6] = u.z; b[7] = u.w;
      }
#pragma unroll
      for (int i = 0; i < RM; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
  }
  cp_async_wait<0>();

  // ---- bias, ReLU, store: rows ty * 4 + {0..3} (and TM / 2 + the same), pixels tx * 4 + {0..3} and 64 + the same
  const bool vec_store = (ohow & 3) == 0;
  const bool partial = p.splits > 1;
  if (partial) y += (size_t)split * P * p.oc;
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    const int co = co0 + (i < 4 ? ty * 4 + i : (TM / 2) + ty * 4 + (i - 4));
    if (co >= p.ocg) continue;
    const int oc = g * p.ocg + co;
    const float bv = (bias && !partial) ? __ldg(bias + oc) : 0.f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const long long q0 = pix0 + h * 64 + tx * 4;
      if (q0 >= P) continue;
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = relu_f(acc[i][h * 4 + j] + bv, partial ? 0 : p.do_relu, p.relu_limit);
      if (vec_store && q0 + 3 < P) {
        const long long b = q0 / ohow, r = q0 - b * ohow;
        *reinterpret_cast<float4*>(y + (b * p.oc + oc) * ohow + r) = make_float4(v[0], v[1], v[2], v[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const long long q = q0 + j;
          if (q < P) {
            const long long b = q / ohow, r = q - b * ohow;
            y[(b * p.oc + oc) * ohow + r] = v[j];
          }
        }
      }
    }
  }
}

// y = relu(sum over the splits' planes, in plane order, + bias): 4 outputs per thread (count is a multiple of 4 or the
// tail runs element by element)
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, const float* __restrict__ bias, float* __restrict__ y,
                                     long long count, int splits, int oc, int ohow, int do_relu, float relu_limit) {
  const long long i4 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i4 >= count) return;
  const int n = (int)min((long long)4, count - i4);
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (n == 4 && (ohow & 3) == 0) {
    for (int s = 0; s < splits; ++s) {
      const float4 u = __ldg(reinterpret_cast<const float4*>(ws + (size_t)s * count + i4));
      v[0] += u.x; v[1] += u.y; v[2] += u.z; v[3] += u.w;
    }
    const float bv = bias ? __ldg(bias + (int)((i4 / ohow) % oc)) : 0.f;   // the four share a channel: ohow % 4 == 0
    *reinterpret_cast<float4*>(y + i4) = make_float4(relu_f(v[0] + bv, do_relu, relu_limit), relu_f(v[1] + bv, do_relu, relu_limit),
                                                     relu_f(v[2] + bv, do_relu, relu_limit), relu_f(v[3] + bv, do_relu, relu_limit));
    return;
  }
  for (int e = 0; e < n; ++e) {
    float a = 0.f;
    for (int s = 0; s < splits; ++s) a += __ldg(ws + (size_t)s * count + i4 + e);
    const float bv = bias ? __ldg(bias + (int)(((i4 + e) / ohow) % oc)) : 0.f;
    y[i4 + e] = relu_f(a + bv, do_relu, relu_limit);
  }
}

// (c, kh, kw) of every k: offset inside an image and the two border shifts
__global__ void conv_ktab_kernel(int2* ktab, int K, int kh, int kw, int ih, int iw, int dh, int dw) {
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= K) return;
  const int c = k / (kh * kw), r = k - c * kh * kw, a = r / kw, b = r - a * kw;
  ktab[k] = make_int2(c * ih * iw + a * dh * iw + b * dw, (a * dh) | ((b * dw) << 16));
}

// OIHW [groups * ocg][K] -> [groups][K][ocg]
__global__ void conv_wt_kernel(const float* __restrict__ w, float* __restrict__ wt, int groups, int ocg, int K) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)groups * ocg * K;
  if (i >= total) return;
  const int co = (int)(i % ocg);
  const long long r = i / ocg;
  const int k = (int)(r % K), g = (int)(r / K);
  wt[i] = w[((size_t)g * ocg + co) * K + k];
}

__global__ void pool2d_f32_kernel(const float* __restrict__ x, float* __restrict__ y, long long total, int ih, int iw, int oh,
                                  int ow, int kh, int kw, int sh, int sw, int pht, int pwl, int is_max,
                                  int count_include_pad, int phb, int pwr, int do_relu, float relu_limit) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int wo = (int)(i % ow);
  const long long r = i / ow;
  const int ho = (int)(r % oh);
  const long long nc = r / oh;
  const float* src = x + nc * ih * iw;
  const int h0 = ho * sh - pht, w0 = wo * sw - pwl;
  float acc = is_max ? -INFINITY : 0.f;
  int inside = 0;
  for (int a = 0; a < kh; ++a) {
    const int h = h0 + a;
    if ((unsigned)h >= (unsigned)ih) continue;
    for (int b = 0; b < kw; ++b) {
      const int w = w0 + b;
      if ((unsigned)w >= (unsigned)iw) continue;
      const float v = __ldg(src + (size_t)h * iw + w);
      acc = is_max ? fmaxf(acc, v) : acc + v;
      ++inside;
    }
  }
  if (!is_max) {
    int div = inside;
    if (count_include_pad) {   // the window clipped to the padded image
      const int he = min(h0 + kh, ih + phb), we = min(w0 + kw, iw + pwr);
      div = (he - h0) * (we - w0);
    }
    acc = div > 0 ? acc / (float)div : 0.f;
  }
  y[i] = relu_f(acc, do_relu, relu_limit);
}

__global__ void add_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ y, long long n,
                               int do_relu, float relu_limit) {
  const long long i4 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i4 + 3 < n) {
    const float4 u = *reinterpret_cast<const float4*>(a + i4);
    const float4 v = b ? *reinterpret_cast<const float4*>(b + i4) : make_float4(0.f, 0.f, 0.f, 0.f);
    *reinterpret_cast<float4*>(y + i4) = make_float4(relu_f(u.x + v.x, do_relu, relu_limit), relu_f(u.y + v.y, do_relu, relu_limit),
                                                     relu_f(u.z + v.z, do_relu, relu_limit), relu_f(u.w + v.w, do_relu, relu_limit));
  } else {
    for (long long i = i4; i < n; ++i) y[i] = relu_f(a[i] + (b ? b[i] : 0.f), do_relu, relu_limit);
  }
}

// import_quant_bias of the threshold tuner (python/calibration/simple_tunner.py:43-50): the value on the int8 grid of
// `threshold`, round(v * 127 / th) clipped to [-128, 127], back in float.  np.round rounds halves to even.
__global__ void fake_quant_f32_kernel(const float* __restrict__ x, float* __restrict__ y, long long n, float scale) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = rintf(x[i] * scale);
  v = fminf(fmaxf(v, -128.f), 127.f);
  y[i] = v / scale;
}

// sums for the tuner's distance and cosine similarity (simple_tunner.py:334-358): out[0] += sum (ref - x)^2,
// out[1] += sum |ref|, out[2] += sum x * ref, out[3] += sum x^2, out[4] += sum ref^2; double accumulation
__global__ void distance_f32_kernel(const float* __restrict__ x, const float* __restrict__ ref, long long n, double* out) {
  double s[5] = {0, 0, 0, 0, 0};
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const double a = x[i], r = ref[i], d = r - a;
    s[0] += d * d;
    s[1] += fabs(r);
    s[2] += a * r;
    s[3] += a * a;
    s[4] += r * r;
  }
  __shared__ double sh[5][8];
#pragma unroll
  for (int k = 0; k < 5; ++k) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s[k] += __shfl_xor_sync(0xffffffffu, s[k], o);
    if ((threadIdx.x & 31) == 0) sh[k][threadIdx.x >> 5] = s[k];
  }
  __syncthreads();
  if (threadIdx.x < 5) {
    double t = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += sh[threadIdx.x][w];
    atomicAdd(out + threadIdx.x, t);
  }
}

// ---- elementwise float ops of the Top dialect (lib/Dialect/Top/Interfaces/<Op>.cpp, each op's inference loop): the
// arithmetic type of every expression follows the reference's C++ (float unless a double constant promotes it)
__global__ void eltwise_f32_kernel(int op, const float* __restrict__ a, const float* __restrict__ b, double cd,
                                   float* __restrict__ y, long long n, int do_relu, float relu_limit) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float x = a[i];
  const float c = (float)cd;
  float v;
  switch (op) {
    case TOP_ADD_CONST: v = __fadd_rn(x, c); break;                                   // AddConst.cpp:26
    case TOP_SUB_CONST: v = __fsub_rn(x, c); break;                                   // SubConst.cpp:31
    case TOP_RSUB_CONST: v = __fsub_rn(c, x); break;                                  // SubConst.cpp:26 (is_reverse)
    case TOP_MUL_CONST: v = (float)((double)x * cd); break;                           // MulConst.cpp:25: float * double
    case TOP_MAX_CONST: v = fmaxf(x, c); break;                                       // MaxConst.cpp:26
    case TOP_MIN_CONST: v = fminf(x, c); break;                                       // MinConst.cpp:26
    case TOP_MUL: v = __fmul_rn(x, b[i]); break;
    case TOP_SUB: v = __fsub_rn(x, b[i]); break;
    case TOP_RSUB: v = __fsub_rn(b[i], x); break;
    case TOP_DIV: v = __fdiv_rn(x, b[i]); break;
    case TOP_RDIV: v = __fdiv_rn(b[i], x); break;
    case TOP_SIGMOID: v = __fdiv_rn(1.f, __fadd_rn(1.f, expf(-x))); break;            // Sigmoid.cpp:28
    case TOP_LOG_SIGMOID: v = logf(__fdiv_rn(1.f, __fadd_rn(1.f, expf(-x)))); break;
    case TOP_SILU: v = __fdiv_rn(x, __fadd_rn(1.f, expf(-x))); break;                 // SiLU.cpp:26
    case TOP_GELU: v = (float)(0.5 * (double)x * (1.0 + erf((double)x / sqrt(2.0)))); break;   // GELU.cpp:24: double
    case TOP_FLOOR: v = floorf(x); break;                                             // Floor.cpp:24
    default: v = x;
  }
  y[i] = relu_f(v, do_relu, relu_limit);
}

// tpu::ActiveOp (lib/Dialect/Tpu/Interfaces/Common/Active.cpp:20-32): out = (float)func((double)in) with func from
// lib/Support/ActiveUtils.cpp:16-181; `mode` is the dialect's ActiveMode number.  Everything is evaluated in double, as
// there, except MISH, whose helper works in float (lib/Support/GenericCpuFunc.cpp:25-33).  Modes the reference's switch
// does not hold (RELU, IS_FINITE, ARCSIN, ARCSINH, ARCCOSH) are refused by the launcher.
__global__ void active_f32_kernel(int mode, const float* __restrict__ x, double c0, double c1, float* __restrict__ y, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const double v = (double)x[i];
  double r;
  switch (mode) {
    case 0: r = tanh(v); break;
    case 1: r = 1.0 / (1.0 + exp(-v)); break;
    case 3: r = exp(v); break;
    case 4: r = v > 0 ? v : c0 * (exp(v) - 1.0); break;                                  // ELU, alpha = coeffs[0]
    case 5: r = sqrt(v); break;
    case 6: r = v * v; break;
    case 7: r = 1.0 / sqrt(v); break;                                                    // RSQRT: `1.f / std::sqrt(val)` divides in double
    case 8: r = fabs(v); break;
    case 9: r = log(v); break;
    case 10: r = round(v); break;
    case 11: r = ceil(v); break;
    case 12: r = floor(v); break;
    case 13: r = sin(v); break;
    case 14: r = cos(v); break;
    case 16: {                                                                           // MISH in float
      const float xf = x[i];
      const float sp = logf(__fadd_rn(expf(xf), 1.f));
      const float th = __fsub_rn(__fdiv_rn(2.f, __fadd_rn(1.f, expf(__fmul_rn(-2.f, sp)))), 1.f);
      r = (double)__fmul_rn(xf, th);
      break;
    }
    case 17: r = v / (1.0 + exp(-v * c0)); break;                                        // SWISH, beta = coeffs[0]
    case 18: r = v * fmax(0.0, fmin(1.0, (v + 3.0) / 6.0)); break;                       // HSWISH
    case 19: r = v / (1.0 + exp(-v)); break;                                             // SILU
    case 21: r = acos(v); break;
    case 24: r = atanh(v); break;
    case 25: r = sinh(v); break;
    case 26: r = cosh(v); break;
    case 27: r = tan(v); break;
    case 28: r = v < 0 ? -1.0 : 1.0; break;                                              // SIGN as the reference evaluates it: 1 at 0
    case 29: r = 0.5 * v * (1.0 + erf(v / sqrt(2.0))); break;                            // GELU
    case 30: r = erf(v); break;
    case 31: r = fmax(0.0, fmin(1.0, c1 * v + c0)); break;                               // HSIGMOID: alpha = coeffs[1], beta = coeffs[0]
    case 32: r = log(1.0 / (1.0 + exp(-v))); break;                                      // LOG_SIGMOID
    case 33: r = v > 20 ? v : log(exp(v) + 1.0); break;                                  // SOFT_PLUS
    case 34: r = v / (1.0 + fabs(v)); break;                                             // SOFT_SIGN
    case 35: r = log2(v); break;
    case 36: r = 0.5 * v * (1.0 + tanh(v * 0.7978845608 * (1.0 + 0.044715 * v * v))); break;   // TGELU
    case 37: r = v * (1.0 / (1.0 + exp(-(1.702 * v)))); break;                           // QGELU
    default: r = v;
  }
  y[i] = (float)r;
}

// top::ScaleOp (Scale.cpp:19-44): y = x * scale[c] + bias[c], a multiply and an add (no fused multiply-add)
__global__ void scale_f32_kernel(const float* __restrict__ x, const float* __restrict__ sc, const float* __restrict__ bi,
                                 float* __restrict__ y, long long n, int channels, long long inner, int do_relu, float relu_limit) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int c = (int)((i / inner) % channels);
  y[i] = relu_f(__fadd_rn(__fmul_rn(x[i], sc[c]), bi ? bi[c] : 0.f), do_relu, relu_limit);
}

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float u = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, u) : v + u;
  }
  __syncthreads();   // the previous use of `sh` is over
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = sh[0];
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) r = is_max ? fmaxf(r, sh[w]) : r + sh[w];
  return r;
}

// top::SoftmaxOp (Softmax.cpp:53-80, oneDNN softmax over the middle dimension of [outer, channels, inner]): one block per
// (outer, inner) pair; the usual max-subtracted form, log_softmax when `log`.
__global__ void softmax_f32_kernel(const float* __restrict__ x, float* __restrict__ y, int channels, long long inner, int log_form) {
  __shared__ float sh[8];
  const long long o = blockIdx.x / inner, i = blockIdx.x - o * inner;
  const float* src = x + o * channels * inner + i;
  float* dst = y + o * channels * inner + i;
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < channels; c += blockDim.x) mx = fmaxf(mx, src[(long long)c * inner]);
  mx = block_reduce(mx, true, sh);
  float sum = 0.f;
  for (int c = threadIdx.x; c < channels; c += blockDim.x) sum += expf(src[(long long)c * inner] - mx);
  sum = block_reduce(sum, false, sh);
  const float lsum = logf(sum);
  for (int c = threadIdx.x; c < channels; c += blockDim.x) {
    const float d = src[(long long)c * inner] - mx;
    dst[(long long)c * inner] = log_form ? d - lsum : expf(d) / sum;
  }
}

// top::LayerNormOp (LayerNorm.cpp:24-78): per row of `inner` values mean, biased variance + eps, (x - mean) * rstd, then
// the optional weight and bias of the normalised shape.  One block per row; the sums are tree reductions (the reference
// adds sequentially: agreement to rounding).
__global__ void layernorm_f32_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                     float* __restrict__ y, long long inner, float eps) {
  __shared__ float sh[8];
  const float* src = x + (long long)blockIdx.x * inner;
  float* dst = y + (long long)blockIdx.x * inner;
  float s = 0.f;
  for (long long j = threadIdx.x; j < inner; j += blockDim.x) s += src[j];
  const float mean = block_reduce(s, false, sh) / (float)inner;
  float v = 0.f;
  for (long long j = threadIdx.x; j < inner; j += blockDim.x) {
    const float d = src[j] - mean;
    v += d * d;
  }
  const float rstd = 1.0f / sqrtf(block_reduce(v, false, sh) / (float)inner + eps);
  for (long long j = threadIdx.x; j < inner; j += blockDim.x) {
    float r = __fmul_rn(src[j] - mean, rstd);
    if (w) r = __fmul_rn(r, w[j]);
    if (b) r = __fadd_rn(r, b[j]);
    dst[j] = r;
  }
}

// top::ReduceOp over one run of adjacent axes (Reduce.cpp:59-108): [outer, axis, inner] -> [outer, inner].  One thread per
// output walks the axis in order, as the reference's loop does (sequential float sums: the same rounding).
__global__ void reduce_f32_kernel(int mode, const float* __restrict__ x, float* __restrict__ y, long long outer, int axis,
                                  long long inner) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= outer * inner) return;
  const long long o = i / inner, in = i - o * inner;
  const float* src = x + o * axis * inner + in;
  float v;
  if (mode == TOP_REDUCE_MAX || mode == TOP_REDUCE_MIN || mode == TOP_REDUCE_PROD) {
    v = src[0];
    for (int a = 1; a < axis; ++a) {
      const float u = src[(long long)a * inner];
      if (mode == TOP_REDUCE_MAX) v = u > v ? u : v;
      else if (mode == TOP_REDUCE_MIN) v = u < v ? u : v;
      else v = __fmul_rn(v, u);
    }
  } else {
    v = 0.f;
    for (int a = 0; a < axis; ++a) {
      const float u = src[(long long)a * inner];
      if (mode == TOP_REDUCE_L2) v = __fadd_rn(v, (float)pow((double)u, 2.0));      // std::pow(float, int) computes in double
      else if (mode == TOP_REDUCE_L1) v = __fadd_rn(v, fabsf(u));
      else v = __fadd_rn(v, u);
    }
    if (mode == TOP_REDUCE_MEAN) v = __fdiv_rn(v, (float)axis);
    if (mode == TOP_REDUCE_MEAN_RCP) v = __fmul_rn(v, (float)(1.0 / (double)axis));     // tpu::ReduceOp, Reduce.cpp:132-138
    if (mode == TOP_REDUCE_L2) v = (float)pow((double)v, 0.5);
  }
  y[i] = v;
}

// top::InterpOp / tpu::InterpOp, modes nearest and linear (interp_core, lib/Dialect/Top/Interfaces/Interp.cpp:28-181): per output
// row / column the source coordinate comes from backward_map (:52-98); linear blends rows first (buf = a + dy * (b - a)), then
// columns, each a subtract, a multiply and an add in float, with the last row / column copied.
enum { INTERP_PYTORCH_SUPPORT = 0, INTERP_CAFFE_SUPPORT, INTERP_TENSORFLOW_NEAREST, INTERP_PYTORCH_NEAREST, INTERP_ONNX_NEAREST,
       INTERP_CAFFE_NEAREST };
__device__ __forceinline__ void interp_map(int o, float scale, int d, int align, int half_pixel, int sp, float& xs, int& xi) {
  const float of = (float)o, hi = (float)(d - 1);
  switch (sp) {
    case INTERP_TENSORFLOW_NEAREST:
      xs = half_pixel ? __fmul_rn(__fadd_rn(of, 0.5f), scale) : __fmul_rn(of, scale);
      xs = fminf(fmaxf(xs, 0.f), hi);
      xi = align ? (int)roundf(xs) : (int)floorf(xs);
      break;
    case INTERP_PYTORCH_SUPPORT:
      xs = align ? __fmul_rn(of, scale) : __fsub_rn(__fmul_rn(__fadd_rn(of, 0.5f), scale), 0.5f);
      xs = fminf(fmaxf(xs, 0.f), hi);
      xi = (int)floorf(xs);
      break;
    case INTERP_ONNX_NEAREST:
      if (half_pixel) {
        xs = fminf(fmaxf(__fsub_rn(__fmul_rn(__fadd_rn(of, 0.5f), scale), 0.5f), 0.f), hi);
        xi = (int)floorf(xs);
      } else {
        xs = fminf(fmaxf(__fmul_rn(of, scale), 0.f), hi);
        xi = align ? (int)roundf(xs) : (int)floorf(xs);
      }
      break;
    default:   // PYTORCH_NEAREST, CAFFE_SUPPORT, CAFFE_NEAREST
      xs = fminf(fmaxf(__fmul_rn(of, scale), 0.f), hi);
      xi = (int)floorf(xs);
  }
}
__global__ void interp_f32_kernel(const float* __restrict__ x, float* __restrict__ y, long long nc, int ih, int iw, int oh, int ow,
                                  float h_scale, float w_scale, int align, int half_pixel, int sp) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nc * oh * ow) return;
  const int xo = (int)(i % ow), yo = (int)((i / ow) % oh);
  const float* in = x + (i / ((long long)ow * oh)) * ih * iw;
  float ys, xs;
  int yi, xi;
  interp_map(yo, h_scale, ih, align, half_pixel, sp, ys, yi);
  interp_map(xo, w_scale, iw, align, half_pixel, sp, xs, xi);
  if (sp != INTERP_PYTORCH_SUPPORT && sp != INTERP_CAFFE_SUPPORT) {
    y[i] = in[(long long)yi * iw + xi];
    return;
  }
  const float dy = __fsub_rn(ys, (float)yi), dx = __fsub_rn(xs, (float)xi);
  auto row_blend = [&](int xf) {
    if (yi == ih - 1) return in[(long long)(ih - 1) * iw + xf];
    const float a = in[(long long)yi * iw + xf], b = in[(long long)(yi + 1) * iw + xf];
    return __fadd_rn(a, __fmul_rn(dy, __fsub_rn(b, a)));
  };
  if (xi == iw - 1) {
    y[i] = row_blend(iw - 1);
  } else {
    const float a = row_blend(xi), b = row_blend(xi + 1);
    y[i] = __fadd_rn(a, __fmul_rn(dx, __fsub_rn(b, a)));
  }
}

// top::GridSamplerOp / tpu::GridSamplerOp with a 4-D grid [N, OH, OW, 2] (GridSamplerFunc, lib/Support/GenericCpuFunc.cpp:3332-3455):
// mode 0 bilinear, 1 nearest (nearbyint); padding 0 zeros, 1 border, 2 reflection.  Float arithmetic in the reference's order,
// products and sums kept apart.
__device__ __forceinline__ float grid_clip(float v, int limit) { return fminf((float)(limit - 1), fmaxf(v, 0.f)); }
__device__ __forceinline__ float grid_reflect(float v, int twice_low, int twice_high) {
  if (twice_low == twice_high) return 0.f;
  const float mn = __fdiv_rn((float)twice_low, 2.f), span = __fdiv_rn((float)(twice_high - twice_low), 2.f);
  v = fabsf(__fsub_rn(v, mn));
  const float extra = fmodf(v, span);
  const int flips = (int)floorf(__fdiv_rn(v, span));
  return (flips % 2 == 0) ? __fadd_rn(extra, mn) : __fadd_rn(__fsub_rn(span, extra), mn);
}
__device__ __forceinline__ float grid_index(float coord, int size, int padding, int align) {
  float r = align ? __fmul_rn(__fmul_rn(__fadd_rn(coord, 1.f), .5f), (float)(size - 1))
                  : __fmul_rn(__fsub_rn(__fmul_rn(__fadd_rn(coord, 1.f), (float)size), 1.f), .5f);
  if (padding == 1) r = grid_clip(r, size);
  else if (padding == 2) r = grid_clip(align ? grid_reflect(r, 0, 2 * (size - 1)) : grid_reflect(r, -1, 2 * size - 1), size);
  return r;
}
__global__ void grid_sampler_f32_kernel(const float* __restrict__ x, const float* __restrict__ grid, float* __restrict__ y, int N, int C,
                                        int IH, int IW, int OH, int OW, int mode, int padding, int align) {
  const long long total = (long long)N * C * OH * OW;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int w = (int)(i % OW), h = (int)((i / OW) % OH), c = (int)((i / ((long long)OW * OH)) % C), n = (int)(i / ((long long)OW * OH * C));
  const float* g = grid + (((long long)n * OH + h) * OW + w) * 2;
  const float fx = grid_index(g[0], IW, padding, align), fy = grid_index(g[1], IH, padding, align);
  const float* in = x + ((long long)n * C + c) * IH * IW;
  float o = 0.f;
  if (mode == 0) {
    const int xx = (int)floorf(fx), yy = (int)floorf(fy);
    const float dx = __fsub_rn(fx, (float)xx), dy = __fsub_rn(fy, (float)yy), tx = __fsub_rn(1.f, dx), ty = __fsub_rn(1.f, dy);
    const bool y0 = yy >= 0 && yy < IH, y1 = yy + 1 >= 0 && yy + 1 < IH, x0 = xx >= 0 && xx < IW, x1 = xx + 1 >= 0 && xx + 1 < IW;
    const long long at = (long long)yy * IW + xx;
    if (y0 && x0) o = __fadd_rn(o, __fmul_rn(in[at], __fmul_rn(tx, ty)));
    if (y0 && x1) o = __fadd_rn(o, __fmul_rn(in[at + 1], __fmul_rn(dx, ty)));
    if (y1 && x0) o = __fadd_rn(o, __fmul_rn(in[at + IW], __fmul_rn(tx, dy)));
    if (y1 && x1) o = __fadd_rn(o, __fmul_rn(in[at + IW + 1], __fmul_rn(dx, dy)));
  } else {
    const int xx = (int)rintf(fx), yy = (int)rintf(fy);
    if (yy >= 0 && yy < IH && xx >= 0 && xx < IW) o = in[(long long)yy * IW + xx];
  }
  y[i] = o;
}

// top::ArgOp / tpu::ArgOp (lib/Dialect/Top/Interfaces/Arg.cpp:39-83): along the middle dimension of [outer, axis, inner] the index
// (and, if asked, the value) of the maximum or minimum; a tie keeps the first index, or the last with select_last_index (the
// comparison is then >= / <=).  One thread per output walks the axis in order, like the reference's loop.
__global__ void arg_f32_kernel(const float* __restrict__ x, long long outer, int axis, long long inner, int is_max, int select_last,
                               void* __restrict__ idx_out, int idx_is_float, float* __restrict__ val_out) {
  const long long n = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= outer * inner) return;
  const float* p = x + (n / inner) * axis * inner + (n % inner);
  float best = p[0];
  int at = 0;
  for (int a = 1; a < axis; ++a) {
    const float v = p[(long long)a * inner];
    const bool take = is_max ? (select_last ? v >= best : v > best) : (select_last ? v <= best : v < best);
    if (take) {
      best = v;
      at = a;
    }
  }
  if (idx_is_float) static_cast<float*>(idx_out)[n] = (float)at;
  else static_cast<int*>(idx_out)[n] = at;
  if (val_out) val_out[n] = best;
}

// top::CastOp (lib/Dialect/Top/Interfaces/Cast.cpp:18-68): to an integer type, saturate(to_int(x, round_mode)); the result is
// written as a float (the reference's storage) or in the integer type itself.  `to` F32 copies.
__global__ void top_cast_kernel(const float* __restrict__ x, long long n, int to_dt, int rmode, int out_dt, void* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = x[i];
  if (to_dt == B200Q_DT_F32) {
    static_cast<float*>(out)[i] = v;
    return;
  }
  const long long r = clamp_dtype(to_int_f32(v, rmode), to_dt);
  switch (out_dt) {
    case B200Q_DT_F32: static_cast<float*>(out)[i] = (float)r; break;
    case B200Q_DT_I8: static_cast<int8_t*>(out)[i] = (int8_t)r; break;
    case B200Q_DT_U8: static_cast<uint8_t*>(out)[i] = (uint8_t)r; break;
    case B200Q_DT_I16: static_cast<int16_t*>(out)[i] = (int16_t)r; break;
    case B200Q_DT_U16: static_cast<uint16_t*>(out)[i] = (uint16_t)r; break;
    default: static_cast<int32_t*>(out)[i] = (int32_t)r; break;
  }
}

// top::GatherOp / tpu::GatherOp (lib/Dialect/Top/Interfaces/Gather.cpp:17-49): dst[o, j, k] = src[o, idx[j], k], a negative
// index counts from the end of the axis.  Indices are floats (the interpreter's storage) or int32.  An index outside the axis
// writes zero instead of reading outside the tensor.
template <typename T>
__global__ void gather_kernel(const T* __restrict__ src, const void* __restrict__ indices, int index_is_float, T* __restrict__ dst,
                              long long outer, long long axis_dim, long long num_indices, long long inner) {
  const long long total = outer * num_indices * inner;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long k = i % inner, j = (i / inner) % num_indices, o = i / (inner * num_indices);
    long long ix;
    if (index_is_float) {
      const float f = static_cast<const float*>(indices)[j];
      ix = (long long)(f < 0 ? f + (float)axis_dim : f);
    } else {
      ix = static_cast<const int*>(indices)[j];
      if (ix < 0) ix += axis_dim;
    }
    dst[i] = (ix >= 0 && ix < axis_dim) ? src[(o * axis_dim + ix) * inner + k] : T(0);
  }
}

// top::GatherElementsOp (GatherElements.cpp:20-79): the output has the shape of `indices`; the source coordinate equals the
// output's except on `axis`, where it is the index.  Up to eight dimensions, as there.
struct GatherElemDims { long long idx_shape[8], src_stride[8]; int ndim, axis; long long axis_dim; };
template <typename T>
__global__ void gather_elements_kernel(const T* __restrict__ src, const void* __restrict__ indices, int index_is_float,
                                       T* __restrict__ dst, const GatherElemDims d, long long total) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    long long rem = i, at = 0;
    for (int k = d.ndim - 1; k >= 0; --k) {
      const long long c = rem % d.idx_shape[k];
      rem /= d.idx_shape[k];
      if (k != d.axis) at += c * d.src_stride[k];
    }
    long long ix = index_is_float ? (long long)static_cast<const float*>(indices)[i] : (long long)static_cast<const int*>(indices)[i];
    if (ix < 0) ix += d.axis_dim;
    dst[i] = (ix >= 0 && ix < d.axis_dim) ? src[at + ix * d.src_stride[d.axis]] : T(0);
  }
}

// Data movement by index arithmetic (Slice, Permute, Tile, Upsample, Pad, Concat of either dialect): the output (or, for
// Concat, one input's region of it) is walked in up to six dimensions; per dimension the source coordinate is
// ((i / div) % mod) * mul + off (mod 0 = no wrap), valid inside [0, extent); an invalid coordinate writes the pad value.
template <typename T>
__global__ void remap_kernel(const T* __restrict__ src, T* __restrict__ dst, const TopRemap m, T pad, long long total) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  long long so = 0, dofs = m.dst_offset;
  bool ok = true;
#pragma unroll
  for (int d = TOP_REMAP_DIMS - 1; d >= 0; --d) {
    const long long dim = m.dims[d];
    const long long id = i % dim;
    i /= dim;
    long long sidx = id / m.div[d];
    if (m.mod[d] > 0) sidx %= m.mod[d];
    sidx = sidx * m.mul[d] + m.off[d];
    ok = ok && sidx >= 0 && sidx < m.extent[d];
    so += sidx * m.src_stride[d];
    dofs += id * m.dst_stride[d];
  }
  dst[dofs] = ok ? src[so] : pad;
}

}  // namespace

int top_eltwise_launch(int op, const float* a, const float* b, double c, float* y, long long n, bool do_relu, float relu_limit,
                       cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  if (op < 0 || op >= TOP_ELTWISE_OPS) return set_error(B200Q_ERR_INVALID, "top eltwise: unknown op %d", op);
  const bool binary = op == TOP_MUL || op == TOP_SUB || op == TOP_RSUB || op == TOP_DIV || op == TOP_RDIV;
  if (binary && !b) return set_error(B200Q_ERR_INVALID, "top eltwise: the op needs a second operand");
  eltwise_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(op, a, b, c, y, n, do_relu ? 1 : 0, relu_limit);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int top_active_launch(int mode, const float* x, double c0, double c1, float* y, long long n, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  const bool known = mode >= 0 && mode <= 37 && mode != 2 && mode != 15 && mode != 20 && mode != 22 && mode != 23;
  if (!known) return set_error(B200Q_ERR_UNSUPPORTED, "active: mode %d has no function in the reference", mode);
  active_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(mode, x, c0, c1, y, n);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int top_scale_launch(const float* x, const float* scale, const float* bias, float* y, long long outer, int channels, long long inner,
                     bool do_relu, float relu_limit, cudaStream_t s) {
  const long long n = outer * channels * inner;
  if (n == 0) return B200Q_OK;
  scale_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(x, scale, bias, y, n, channels, inner, do_relu ? 1 : 0, relu_limit);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int top_reduce_launch(int mode, const float* x, float* y, long long outer, int axis, long long inner, cudaStream_t s) {
  const long long n = outer * inner;
  if (n == 0) return B200Q_OK;
  if (mode < 0 || mode >= TOP_REDUCE_MODES || axis < 1) return set_error(B200Q_ERR_INVALID, "reduce: bad mode or empty axis");
  reduce_f32_kernel<<<(unsigned)((n + 127) / 128), 128, 0, s>>>(mode, x, y, outer, axis, inner);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int top_softmax_launch(const float* x, float* y, long long outer, int channels, long long inner, bool log_form, cudaStream_t s) {
  const long long rows = outer * inner;
  if (rows == 0 || channels == 0) return B200Q_OK;
  if (rows > 0x7fffffffLL) return set_error(B200Q_ERR_UNSUPPORTED, "softmax: too many rows");
  softmax_f32_kernel<<<(unsigned)rows, 256, 0, s>>>(x, y, channels, inner, log_form ? 1 : 0);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int top_layernorm_launch(const float* x, const float* w, const float* b, float* y, long long outer, long long inner, float eps,
                         cudaStream_t s) {
  if (outer == 0 || inner == 0) return B200Q_OK;
  if (outer > 0x7fffffffLL) return set_error(B200Q_ERR_UNSUPPORTED, "layernorm: too many rows");
  layernorm_f32_kernel<<<(unsigned)outer, 256, 0, s>>>(x, w, b, y, inner, eps);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

// calc_resize_scale (Interp.cpp:28-50)
static float interp_scale(int in_size, int out_size, bool align, int sp) {
  const bool caffe = sp == INTERP_CAFFE_NEAREST || sp == INTERP_CAFFE_SUPPORT;
  const bool may_align = sp == INTERP_TENSORFLOW_NEAREST || sp == INTERP_PYTORCH_SUPPORT || sp == INTERP_ONNX_NEAREST;
  if (caffe || (may_align && align)) {
    if (out_size <= 1) return 0.f;
    --in_size;
    --out_size;
  }
  return in_size / (float)out_size;
}

// mode 0 nearest / 1 linear; coord_mode 0 half_pixel, 1 pytorch_half_pixel, 2 align_corners, 3 asymmetric; platform 0 ONNX (and any
// other), 1 TORCH, 2 TFLITE, 3 CAFFE: the resolution of Interp.cpp:226-279
int top_interp_launch(const float* x, float* y, long long nc, int ih, int iw, int oh, int ow, int mode, int coord_mode, int platform,
                      cudaStream_t s) {
  if (mode < 0 || mode > 1 || coord_mode < 0 || coord_mode > 3) return set_error(B200Q_ERR_UNSUPPORTED, "interp: mode %d, coord mode %d", mode, coord_mode);
  int sp;
  bool align, half_pixel;
  if (mode == 0) {
    sp = platform == 3 ? INTERP_CAFFE_NEAREST : platform == 1 ? INTERP_PYTORCH_NEAREST : platform == 2 ? INTERP_TENSORFLOW_NEAREST : INTERP_ONNX_NEAREST;
    align = coord_mode != 3;
    half_pixel = false;
  } else {
    sp = platform == 3 ? INTERP_CAFFE_SUPPORT : INTERP_PYTORCH_SUPPORT;
    align = coord_mode == 2;
    half_pixel = coord_mode == 0 || coord_mode == 1;
  }
  const long long total = nc * oh * ow;
  if (total == 0) return B200Q_OK;
  interp_f32_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(x, y, nc, ih, iw, oh, ow, interp_scale(ih, oh, align, sp),
                                                                     interp_scale(iw, ow, align, sp), align, half_pixel, sp);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int top_grid_sampler_launch(const float* x, const float* grid, float* y, int N, int C, int IH, int IW, int OH, int OW, int mode, int padding,
                            bool align_corners, cudaStream_t s) {
  const long long total = (long long)N * C * OH * OW;
  if (total == 0) return B200Q_OK;
  if (mode < 0 || mode > 1 || padding < 0 || padding > 2) return set_error(B200Q_ERR_INVALID, "grid_sampler: mode %d, padding %d", mode, padding);
  grid_sampler_f32_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(x, grid, y, N, C, IH, IW, OH, OW, mode, padding, align_corners);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int top_arg_launch(const float* x, long long outer, int axis, long long inner, bool is_max, bool select_last, void* idx_out,
                   bool idx_is_float, float* val_out, cudaStream_t s) {
  const long long n = outer * inner;
  if (n == 0) return B200Q_OK;
  arg_f32_kernel<<<(unsigned)((n + 127) / 128), 128, 0, s>>>(x, outer, axis, inner, is_max, select_last, idx_out, idx_is_float, val_out);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int top_cast_launch(const float* x, long long n, int to_dt, int rmode, int out_dt, void* out, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  top_cast_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(x, n, to_dt, rmode, out_dt, out);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int top_gather_launch(const void* src, int elem_bytes, const void* indices, bool index_is_float, void* dst, long long outer,
                      long long axis_dim, long long num_indices, long long inner, cudaStream_t s) {
  const long long total = outer * num_indices * inner;
  if (total == 0) return B200Q_OK;
  const unsigned blocks = (unsigned)std::min<long long>((total + 255) / 256, 148LL * 32);
  if (elem_bytes == 4)
    gather_kernel<uint32_t><<<blocks, 256, 0, s>>>(static_cast<const uint32_t*>(src), indices, index_is_float, static_cast<uint32_t*>(dst),
                                                    outer, axis_dim, num_indices, inner);
  else if (elem_bytes == 2)
    gather_kernel<uint16_t><<<blocks, 256, 0, s>>>(static_cast<const uint16_t*>(src), indices, index_is_float, static_cast<uint16_t*>(dst),
                                                    outer, axis_dim, num_indices, inner);
  else if (elem_bytes == 1)
    gather_kernel<uint8_t><<<blocks, 256, 0, s>>>(static_cast<const uint8_t*>(src), indices, index_is_float, static_cast<uint8_t*>(dst),
                                                   outer, axis_dim, num_indices, inner);
  else
    return set_error(B200Q_ERR_INVALID, "gather: element size %d", elem_bytes);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int top_gather_elements_launch(const void* src, int elem_bytes, const void* indices, bool index_is_float, void* dst, int ndim,
                               const long long* src_shape, const long long* idx_shape, int axis, cudaStream_t s) {
  if (ndim < 1 || ndim > 8 || axis < 0 || axis >= ndim) return set_error(B200Q_ERR_INVALID, "gather_elements: rank %d, axis %d", ndim, axis);
  GatherElemDims d{};
  d.ndim = ndim;
  d.axis = axis;
  d.axis_dim = src_shape[axis];
  long long acc = 1, total = 1;
  for (int k = ndim - 1; k >= 0; --k) {
    d.src_stride[k] = acc;
    acc *= src_shape[k];
    d.idx_shape[k] = idx_shape[k];
    total *= idx_shape[k];
    if (k != axis && idx_shape[k] > src_shape[k]) return set_error(B200Q_ERR_INVALID, "gather_elements: indices exceed the source on dimension %d", k);
  }
  if (total == 0) return B200Q_OK;
  const unsigned blocks = (unsigned)std::min<long long>((total + 255) / 256, 148LL * 32);
  if (elem_bytes == 4)
    gather_elements_kernel<uint32_t><<<blocks, 256, 0, s>>>(static_cast<const uint32_t*>(src), indices, index_is_float,
                                                             static_cast<uint32_t*>(dst), d, total);
  else if (elem_bytes == 2)
    gather_elements_kernel<uint16_t><<<blocks, 256, 0, s>>>(static_cast<const uint16_t*>(src), indices, index_is_float,
                                                             static_cast<uint16_t*>(dst), d, total);
  else if (elem_bytes == 1)
    gather_elements_kernel<uint8_t><<<blocks, 256, 0, s>>>(static_cast<const uint8_t*>(src), indices, index_is_float,
                                                            static_cast<uint8_t*>(dst), d, total);
  else
    return set_error(B200Q_ERR_INVALID, "gather_elements: element size %d", elem_bytes);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int top_remap_launch(const void* src, void* dst, int elem_bytes, const TopRemap& m, const void* pad_value, cudaStream_t s) {
  long long total = 1;
  for (int d = 0; d < TOP_REMAP_DIMS; ++d) {
    if (m.dims[d] < 0 || m.div[d] < 1 || m.mod[d] < 0) return set_error(B200Q_ERR_INVALID, "remap: bad dimension %d", d);
    total *= m.dims[d];
  }
  if (total == 0) return B200Q_OK;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (elem_bytes == 4) {
    uint32_t pad = 0;
    if (pad_value) memcpy(&pad, pad_value, 4);
    remap_kernel<uint32_t><<<blocks, 256, 0, s>>>(static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst), m, pad, total);
  } else if (elem_bytes == 2) {
    uint16_t pad = 0;
    if (pad_value) memcpy(&pad, pad_value, 2);
    remap_kernel<uint16_t><<<blocks, 256, 0, s>>>(static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst), m, pad, total);
  } else if (elem_bytes == 1) {
    uint8_t pad = 0;
    if (pad_value) memcpy(&pad, pad_value, 1);
    remap_kernel<uint8_t><<<blocks, 256, 0, s>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), m, pad, total);
  } else {
    return set_error(B200Q_ERR_INVALID, "remap: element size %d", elem_bytes);
  }
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int top_fake_quant_launch(const float* x, float* y, long long n, double threshold, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  if (!(threshold > 0.0)) return set_error(B200Q_ERR_INVALID, "fake quant: the threshold must be positive");
  fake_quant_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(x, y, n, (float)(127.0 / threshold));   // the scale is formed in double and used as a float, like numpy does
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int top_distance_launch(const float* x, const float* ref, long long n, double* sums5, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  long long blocks = (n + 256 * 8 - 1) / (256 * 8);
  if (blocks > 148 * 8) blocks = 148 * 8;
  distance_f32_kernel<<<(unsigned)blocks, 256, 0, s>>>(x, ref, n, sums5);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int top_conv_prepare(const TopConvPlan& p, const float* w_oihw, float* wt, int2* ktab, cudaStream_t s) {
  const long long total = (long long)p.groups * p.ocg * p.K;
  conv_wt_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(w_oihw, wt, p.groups, p.ocg, p.K);
  conv_ktab_kernel<<<(p.K + 255) / 256, 256, 0, s>>>(ktab, p.K, p.kh, p.kw, p.ih, p.iw, p.dh, p.dw);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

// K splits for a launch whose grid would leave SMs idle.  Model: the launch takes `waves` rounds of (k per split + a
// fixed cost per block worth about 128 k); the split count with the smallest product wins, each split at least 256 k.
int top_conv_splits(const TopConvPlan& p, int sms) {
  const long long P = (long long)p.n * p.oh * p.ow;
  const long long ptiles = (P + TN - 1) / TN;
  const int tm = p.ocg > 64 ? 128 : 64;
  const long long blocks = ptiles * ((p.ocg + tm - 1) / tm) * p.groups;
  const long long slots = 2LL * sms;
  if (blocks <= 0 || blocks >= slots) return 1;   // (grids of one to four waves were tried too: no gain in the sum)
  int best = 1;
  long long best_cost = 0, cost1 = 0;
  for (int sp = 1; sp <= 8; ++sp) {
    if (sp > 1 && p.K / sp < 256) break;
    const long long waves = (blocks * sp + slots - 1) / slots;
    const long long cost = waves * ((p.K + sp - 1) / sp + 128);
    if (sp == 1) cost1 = cost;
    if (sp == 1 || cost < best_cost) {
      best = sp;
      best_cost = cost;
    }
  }
  return best_cost * 10 <= cost1 * 9 ? best : 1;   // the partial sums cost a pass over the output: worth it from 10 % on
}

int top_conv_launch(const TopConvPlan& plan, const float* x, const float* wt, const int2* ktab, const float* bias, float* y,
                    float* workspace, cudaStream_t s) {
  TopConvPlan p = plan;
  const long long P = (long long)p.n * p.oh * p.ow;
  if (P == 0) return B200Q_OK;
  const long long ptiles = (P + TN - 1) / TN;
  if (ptiles > 0x7fffffffLL) return set_error(B200Q_ERR_UNSUPPORTED, "top conv: too many pixels");
  if ((reinterpret_cast<uintptr_t>(x) & 3) || (reinterpret_cast<uintptr_t>(wt) & 15) || (reinterpret_cast<uintptr_t>(y) & 15))
    return set_error(B200Q_ERR_INVALID, "top conv: operands must be 16-byte aligned");
  const int khw = (p.kh == 1 && p.kw == 1) ? 1 : (p.kh == 3 && p.kw == 3) ? 9 : 0;
  if (khw == 0 && !ktab) return set_error(B200Q_ERR_INVALID, "top conv: this filter size needs the gather table");
  if (p.splits < 1 || !workspace) p.splits = 1;
  p.k_per_split = p.splits > 1 ? ((p.K + p.splits - 1) / p.splits + TK - 1) / TK * TK : p.K;
  if (p.splits > 1) p.splits = (p.K + p.k_per_split - 1) / p.k_per_split;
  float* out = p.splits > 1 ? workspace : y;
  if ((long long)p.groups * p.splits > 65535) return set_error(B200Q_ERR_UNSUPPORTED, "top conv: too many groups");
  // (64-channel tiles for the layers whose 128-channel grid does not fill the GPU were measured: no faster - those
  // layers are bound by the length of their K loop, which the K splits shorten)
  if (p.ocg > 64) {
    dim3 grid((unsigned)ptiles, (unsigned)((p.ocg + 127) / 128), (unsigned)(p.groups * p.splits));
    if (khw == 1) conv2d_f32_kernel<128, 1><<<grid, CONV_THREADS, 0, s>>>(x, wt, ktab, bias, out, p);
    else if (khw == 9) conv2d_f32_kernel<128, 9><<<grid, CONV_THREADS, 0, s>>>(x, wt, ktab, bias, out, p);
    else conv2d_f32_kernel<128, 0><<<grid, CONV_THREADS, 0, s>>>(x, wt, ktab, bias, out, p);
  } else {
    dim3 grid((unsigned)ptiles, (unsigned)((p.ocg + 63) / 64), (unsigned)(p.groups * p.splits));
    if (khw == 1) conv2d_f32_kernel<64, 1><<<grid, CONV_THREADS, 0, s>>>(x, wt, ktab, bias, out, p);
    else if (khw == 9) conv2d_f32_kernel<64, 9><<<grid, CONV_THREADS, 0, s>>>(x, wt, ktab, bias, out, p);
    else conv2d_f32_kernel<64, 0><<<grid, CONV_THREADS, 0, s>>>(x, wt, ktab, bias, out, p);
  }
  CUDA_TRY(cudaGetLastError());
  if (p.splits > 1) {
    const long long count = P * p.oc;
    const long long vecs = (count + 3) / 4;
    splitk_reduce_kernel<<<(unsigned)((vecs + 255) / 256), 256, 0, s>>>(workspace, bias, y, count, p.splits, p.oc, p.oh * p.ow,
                                                                        p.do_relu, p.relu_limit);
    CUDA_TRY(cudaGetLastError());
  }
  return B200Q_OK;
}

int top_pool2d_launch(const float* x, float* y, long long nc, int ih, int iw, int oh, int ow, int kh, int kw, int sh, int sw,
                      int pht, int phb, int pwl, int pwr, bool is_max, bool count_include_pad, bool do_relu, float relu_limit,
                      cudaStream_t s) {
  const long long total = nc * oh * ow;
  if (total == 0) return B200Q_OK;
  pool2d_f32_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(x, y, total, ih, iw, oh, ow, kh, kw, sh, sw, pht, pwl,
                                                                    is_max ? 1 : 0, count_include_pad ? 1 : 0, phb, pwr,
                                                                    do_relu ? 1 : 0, relu_limit);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int top_add_launch(const float* a, const float* b, float* y, long long n, bool do_relu, float relu_limit, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) || (reinterpret_cast<uintptr_t>(y) & 15))
    return set_error(B200Q_ERR_INVALID, "top add: operands must be 16-byte aligned");
  const long long vecs = (n + 3) / 4;
  add_f32_kernel<<<(unsigned)((vecs + 255) / 256), 256, 0, s>>>(a, b, y, n, do_relu ? 1 : 0, relu_limit);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

}  // namespace b200q
