// C ABI for tpu.A16MatMul with 4-bit weights (lib/Dialect/Tpu/Interfaces/Common/A16MatMul.cpp:16-249):
// operator face over host float buffers and device face over native bf16 / packed-nibble tensors.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <new>

#include "a16.h"
#include "igemm.h"
#include "devbuf.h"
#include "internal.h"
#include "layout.h"

namespace b200q {
namespace {

__global__ void f32_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = __float2bfloat16_rn(x[i]);  // exact: the interpreter's bf16 tensors hold bf16-representable floats
}
__global__ void bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ y, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = __bfloat162float(x[i]);
}

__global__ void f32_to_f16_kernel(const float* __restrict__ x, __half* __restrict__ y, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = __float2half_rn(x[i]);  // exact: the interpreter's f16 tensors hold f16-representable floats
}
__global__ void f16_to_f32_kernel(const __half* __restrict__ x, float* __restrict__ y, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = __half2float(x[i]);
}

// float <-> the op's 16-bit storage type (bf16, or IEEE half for w4f16)
int f32_to_16(const float* x, void* y, long long n, bool f16, cudaStream_t s);
int f16_or_bf16_to_f32(const void* x, float* y, long long n, bool f16, cudaStream_t s);

int f32_to_bf16(const float* x, void* y, long long n, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  f32_to_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(x, static_cast<__nv_bfloat16*>(y), n);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}
int bf16_to_f32(const void* x, float* y, long long n, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  bf16_to_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), y, n);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int f32_to_16(const float* x, void* y, long long n, bool f16, cudaStream_t s) {
  if (!f16) return f32_to_bf16(x, y, n, s);
  if (n == 0) return B200Q_OK;
  f32_to_f16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(x, static_cast<__half*>(y), n);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}
int f16_or_bf16_to_f32(const void* x, float* y, long long n, bool f16, cudaStream_t s) {
  if (!f16) return bf16_to_f32(x, y, n, s);
  if (n == 0) return B200Q_OK;
  f16_to_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(static_cast<const __half*>(x), y, n);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

// W[n,k] = bf16((q - zp) * scale): the dequantised weight the prefill GEMM reads (A16MatMul.cpp:190-198 builds
// the same matrix in fp32 on every call; here it is built once per weight version and kept in bf16).
__global__ void dequant_w4_bf16_kernel(const uint32_t* __restrict__ wq, const __nv_bfloat16* __restrict__ scale,
                                       const uint8_t* __restrict__ zp, uint4* __restrict__ W, long long words, int K,
                                       int group) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one 32-bit word = 8 consecutive k
  if (i >= words) return;
  const long long e0 = i * 8;
  const long long n = e0 / K;
  const int k = (int)(e0 - n * K);
  const long long gi = n * (K / group) + k / group;   // group % 8 == 0: the 8 weights share a group
  const float s = __bfloat162float(scale[gi]);
  const int z = zp[gi];
  const uint32_t w = wq[i];
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float a = (float)((int)((w >> (8 * j)) & 0xF) - z) * s;
    const float b = (float)((int)((w >> (8 * j + 4)) & 0xF) - z) * s;
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    o[j] = *reinterpret_cast<const uint32_t*>(&h);
  }
  W[i] = make_uint4(o[0], o[1], o[2], o[3]);
}

int dequant_w4_bf16(const void* wq, const void* scale, const void* zp, void* W, long long N, int K, int group,
                    cudaStream_t s) {
  const long long words = N * K / 8;
  if (words == 0) return B200Q_OK;
  dequant_w4_bf16_kernel<<<(unsigned)((words + 255) / 256), 256, 0, s>>>(
      static_cast<const uint32_t*>(wq), static_cast<const __nv_bfloat16*>(scale), static_cast<const uint8_t*>(zp),
      static_cast<uint4*>(W), words, K, group);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

// 8-bit weights: W[n,k] = bf16((q - zp) * scale), which is the matrix the reference itself multiplies with
// (A16MatMul.cpp:213-232 rounds the dequantised weight with BF16() before its matmul).  The weight and the zero points
// are read as the interpreter stores them (floats holding integers, signed or unsigned); 8 weights per thread.
template <bool F16>
__global__ void dequant_w8_bf16_kernel(const float4* __restrict__ wq, const uint16_t* __restrict__ scale,
                                       const float* __restrict__ zp, uint4* __restrict__ W, long long octets, int K,
                                       int group) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= octets) return;
  const long long e0 = i * 8;
  const long long n = e0 / K;
  const int k = (int)(e0 - n * K);
  const long long gi = n * (K / group) + k / group;   // group % 8 == 0: the 8 weights share a group
  const float s = F16 ? __half2float(__ushort_as_half(scale[gi])) : __uint_as_float((uint32_t)scale[gi] << 16);
  const float z = zp[gi];
  const float4 lo = wq[2 * i], hi = wq[2 * i + 1];
  const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (F16) {   // F16() of the dequantised weight (A16MatMul.cpp:226-227)
      const __half2 h = __floats2half2_rn((v[2 * j] - z) * s, (v[2 * j + 1] - z) * s);
      o[j] = *reinterpret_cast<const uint32_t*>(&h);
    } else {
      const __nv_bfloat162 h = __floats2bfloat162_rn((v[2 * j] - z) * s, (v[2 * j + 1] - z) * s);
      o[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
  W[i] = make_uint4(o[0], o[1], o[2], o[3]);
}

int dequant_w8_bf16(const float* wq_f32, const void* scale, const float* zp_f32, void* W, long long N, int K, int group, bool f16,
                    cudaStream_t s) {
  const long long octets = N * K / 8;
  if (octets == 0) return B200Q_OK;
  if (f16)
    dequant_w8_bf16_kernel<true><<<(unsigned)((octets + 255) / 256), 256, 0, s>>>(
        reinterpret_cast<const float4*>(wq_f32), static_cast<const uint16_t*>(scale), zp_f32, static_cast<uint4*>(W), octets, K, group);
  else
    dequant_w8_bf16_kernel<false><<<(unsigned)((octets + 255) / 256), 256, 0, s>>>(
        reinterpret_cast<const float4*>(wq_f32), static_cast<const uint16_t*>(scale), zp_f32, static_cast<uint4*>(W), octets, K, group);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

// Prefill: y = x * W^T on the bf16 tensor cores (tcgen05 kind::f16, fp32 accumulation in TMEM).
int a16_prefill_gemm(const void* x, const void* W16, const float* bias, void* y, long long M, int N, int K, int* status,
                     cudaStream_t s, bool f16 = false) {
  IGemmProblem p{};
  p.kind = f16 ? IGEMM_KIND_F16 : IGEMM_KIND_BF16;
  p.a = x;
  p.b = W16;
  p.a_pitch = p.b_pitch = 2LL * K;
  p.rows = (int)M;
  p.n = N;
  p.k_per_tap = 2 * K;
  p.taps_h = p.taps_w = 1;
  p.out_mode = IGEMM_OUT_ROWMAJOR;
  p.ldc = N;
  p.out = y;
  p.bias_f32 = bias;
  Epilogue e{};
  return igemm_i8_tcgen05_launch(p, e, status, s);
}

int validate(const b200q_a16matmul_desc& d) {
  if (d.M < 0 || d.K < 1 || d.N < 1 || d.M > 0x7fffffffLL || d.K > 0x7fffffffLL || d.N > 0x7fffffffLL)
    return set_error(B200Q_ERR_INVALID, "a16matmul: bad shape");
  if (d.weight_bits != 4 && d.weight_bits != 8) return set_error(B200Q_ERR_UNSUPPORTED, "a16matmul: weight_bits must be 4 or 8");
  if (!d.w_transpose) return set_error(B200Q_ERR_UNSUPPORTED, "a16matmul: only w_transpose = true (weight stored [N, K/2]) is implemented");
  if (d.q_group_size < 0) return set_error(B200Q_ERR_INVALID, "a16matmul: negative q_group_size");
  if (d.out_dtype != B200Q_DT_BF16 && d.out_dtype != B200Q_DT_F16)
    return set_error(B200Q_ERR_UNSUPPORTED, "a16matmul: activations/outputs are bf16 (w4bf16) or f16 (w4f16)");
  if (d.weight_bits == 8) {
    const int64_t g = d.q_group_size ? d.q_group_size : d.K;
    if (d.K % 8 != 0 || g % 8 != 0 || d.K % g != 0) return set_error(B200Q_ERR_UNSUPPORTED, "a16matmul: w8 needs K and the group size to be multiples of 8, the group dividing K");
  }
  return B200Q_OK;
}

// Route of b200q_a16_*: 0 = chosen per call; 1 = CUDA-core / mma.sync decode kernels (8 tokens at a time);
// 2 = fused-dequantisation tensor-core kernel; 3 = one-time bf16 copy of the weight + bf16 GEMM (handle API, M > 8);
// 4 = warpgroup kernel (M <= 32).
int g_a16_route = 0;

// Decode shapes go to the GEMV kernel; larger M is processed in slices of 8 tokens.
int a16_dispatch(const void* x, const void* wq, const void* scale, const void* zp, const float* bias, void* y,
                 long long M, int N, int K, int group, int* status, cudaStream_t s, DevBuf* w16 = nullptr,
                 bool* w16_ready = nullptr, bool weights_constant = false, bool f16 = false,
                 A16WgScratch* wg_scratch = nullptr) {
  const char* why = nullptr;
  // both routes index scales and zero points as [n][k / group]: the group must tile K exactly, and a byte holds
  // two consecutive k of one row
  if (group < 1 || K % group != 0 || (K & 1)) return set_error(B200Q_ERR_UNSUPPORTED, "a16matmul: K must be even and a multiple of the group size");
  const int route = g_a16_route;
  if (M == 0) return B200Q_OK;
  const bool umma_ok = a16_w4_umma_supported(M, N, K, group, nullptr) != 0;
  // w4f16: the one-token CUDA-core kernel (two tokens where it applies) and the fused tensor-core kernel have the form
  const bool gemv_ok = M <= 8 && a16_w4_gemv_supported((int)M, N, K, group, nullptr, f16) != 0;
  // the one-time bf16 copy + bf16 GEMM: only through a handle (which owns the copy), only for prefill-sized M
  const bool resident_ok = !f16 && M > 8 && w16 && K % 8 == 0 && group % 8 == 0 && M <= 0x7fffffffLL;
  bool use_umma = false, use_resident = false;
  switch (route) {
    case 1: break;
    case 2:
      if (!umma_ok) return set_error(B200Q_ERR_UNSUPPORTED, "a16matmul: the tensor-core kernel needs K and the group size to be multiples of 64");
      use_umma = true;
      break;
    case 4:
      if (!a16_w4_wg_supported(M, N, K, group, &why)) return set_error(B200Q_ERR_UNSUPPORTED, "a16matmul: %s", why);
      return a16_w4_wg_launch(x, wq, scale, zp, bias, y, M, N, K, group, status, s, f16, wg_scratch);
    case 3: use_resident = resident_ok; use_umma = !resident_ok && !gemv_ok && umma_ok; break;
    default:
      // up to 8 tokens: the decode kernels.  Above: the fused kernel (exact group scaling, no copy of the weight);
      // from 64 tokens on a handle trades 2^-9 of relative weight rounding for the plain bf16 GEMM's speed (measured
      // at N = 11008, K = 4096: 16 / 32 tokens 29.7 us either way, 64 tokens 30.8 against 32-38 us, 128 tokens 33.4
      // against 46-53 us, 512 tokens 56 against 150 us).
      if (gemv_ok) break;
      // 9 to 16 tokens: two launches of the resident decode kernel (23 us at N = 11008, K = 4096) beat the fused kernel
      // (28.8 us); three launches (35 us at 24 tokens) do not
      // (the same holds for long rows, K >= 8192, where the fused kernel's time grows with K: 53 us and more against
      // decode launches of about 18 us each: up to three of them win at K = 11008)
      if (!f16 && ((M <= 16 && a16_w4_gemv_resident_applies(N, K, group, f16)) || (M <= 24 && K >= 8192)) &&
          a16_w4_gemv_supported(8, N, K, group, nullptr, f16) && a16_w4_gemv_supported((int)(M % 8 ? M % 8 : 8), N, K, group, nullptr, f16))
        break;
      if (resident_ok && M >= 64) use_resident = true;
      else use_umma = umma_ok;
  }
  if (use_umma) return a16_w4_umma_launch(x, wq, scale, zp, bias, y, M, N, K, group, status, s, f16);
  if (use_resident) {
    // dequantise once (kept for the life of the handle / weight version), then a bf16 GEMM
    if (!*w16_ready) {
      B200Q_TRY(w16->ensure((size_t)N * K * 2));
      B200Q_TRY(dequant_w4_bf16(wq, scale, zp, w16->p, N, K, group, s));
      *w16_ready = true;
    }
    return a16_prefill_gemm(x, w16->p, bias, y, M, N, K, status, s);
  }
  // decode kernels, 8 tokens per launch (also the fallback for shapes the tensor-core kernel does not take)
  if (!a16_w4_gemv_supported((int)(M < 8 ? M : 8), N, K, group, &why, f16) || (M > 8 && !a16_w4_gemv_supported(8, N, K, group, &why, f16))) return set_error(B200Q_ERR_UNSUPPORTED, "a16matmul: %s", why);
  for (long long m0 = 0; m0 < M; m0 += 8) {
    const int mm = (int)((M - m0) < 8 ? (M - m0) : 8);
    B200Q_TRY(a16_w4_gemv_launch(static_cast<const uint8_t*>(x) + (size_t)m0 * K * 2, wq, scale, zp, bias,
                                 static_cast<uint8_t*>(y) + (size_t)m0 * N * 2, mm, N, K, group, status, s,
                                 weights_constant, f16));
  }
  return B200Q_OK;
}

struct A16Handle {
  DevBuf stage, x16, wq, scale, zp, bias, y16, y32, status, w16;
  A16WgScratch wg_scratch;
  bool w16_ready = false;
  // device face: the caller's tensors (not owned)
  const void *d_wq = nullptr, *d_scale = nullptr, *d_zp = nullptr;
  const float* d_bias = nullptr;
  int N = 0, K = 0, group = 0;
  bool f16 = false;   // device face: the tensors are IEEE half instead of bf16
  bool weights_ready = false;
  int weight_version = -1;
  const float* weight_ptr = nullptr;
};

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_a16matmul_init(const b200q_a16matmul_desc* desc, void** handle) {
  if (!desc || !handle) return set_error(B200Q_ERR_INVALID, "a16matmul_init: null argument");
  B200Q_TRY(validate(*desc));
  auto* h = new (std::nothrow) A16Handle();
  if (!h) return set_error(B200Q_ERR_NOMEM, "a16matmul_init: out of host memory");
  *handle = h;
  return B200Q_OK;
}

void b200q_a16matmul_deinit(void** handle) {
  if (handle && *handle) {
    delete static_cast<A16Handle*>(*handle);
    *handle = nullptr;
  }
}

int b200q_a16matmul_inference(const b200q_a16matmul_desc* desc, float* const* inputs, int n_inputs,
                              float* const* outputs, int n_outputs, void** handle) {
  if (!desc || !inputs || !outputs || !handle || n_inputs < 4 || n_outputs < 1 || !inputs[0] || !inputs[1] ||
      !inputs[2] || !inputs[3] || !outputs[0])
    return set_error(B200Q_ERR_INVALID, "a16matmul_inference: null argument");
  const b200q_a16matmul_desc& d = *desc;
  B200Q_TRY(validate(d));
  const bool own = (*handle == nullptr);
  if (own) B200Q_TRY(b200q_a16matmul_init(desc, handle));
  A16Handle* h = static_cast<A16Handle*>(*handle);
  cudaStream_t s = 0;
  int rc = B200Q_OK;
  const bool f16 = d.out_dtype == B200Q_DT_F16;
  do {
    // q_group_size = 0: one scale and zero point per output channel (A16MatMul.cpp:176-187,:216-222) = a group of K
    const int group = d.q_group_size ? d.q_group_size : (int)d.K;
    const bool w8 = d.weight_bits == 8;
    const size_t w_elems = w8 ? (size_t)d.N * d.K : (size_t)d.N * (d.K / 2), q_elems = (size_t)d.N * (d.K / group);
    const float* bias_f = (d.with_bias && n_inputs > 4) ? inputs[4] : nullptr;
    if (d.with_bias && !bias_f) { rc = set_error(B200Q_ERR_INVALID, "a16matmul: with_bias but inputs[4] is null"); break; }
    const bool cached = h->weights_ready && h->weight_version == d.weight_version && h->weight_ptr == inputs[1];
    if (!cached) {
      // weight bytes, scales and zero points arrive float-stored (WeightOp::read_as_float)
      if (w8) {
        // the reference multiplies with the bf16-rounded dequantised weight: build that matrix once per weight version
        if ((rc = h->stage.ensure(w_elems * 4))) break;
        if ((rc = h->scale.ensure(q_elems * 2))) break;
        if ((rc = h->zp.ensure(q_elems * 4))) break;
        if ((rc = h->w16.ensure(w_elems * 2))) break;
        if (cudaMemcpyAsync(h->stage.p, inputs[2], q_elems * 4, cudaMemcpyHostToDevice, s) != cudaSuccess) { rc = cuda_error(cudaGetLastError(), "H2D scale", __FILE__, __LINE__); break; }
        if ((rc = f32_to_16(h->stage.as<float>(), h->scale.p, (long long)q_elems, f16, s))) break;
        if (cudaMemcpyAsync(h->zp.p, inputs[3], q_elems * 4, cudaMemcpyHostToDevice, s) != cudaSuccess) { rc = cuda_error(cudaGetLastError(), "H2D zp", __FILE__, __LINE__); break; }
        if (cudaMemcpyAsync(h->stage.p, inputs[1], w_elems * 4, cudaMemcpyHostToDevice, s) != cudaSuccess) { rc = cuda_error(cudaGetLastError(), "H2D weight", __FILE__, __LINE__); break; }
        if ((rc = dequant_w8_bf16(h->stage.as<float>(), h->scale.p, h->zp.as<float>(), h->w16.p, d.N, (int)d.K, group, f16, s))) break;
        if (bias_f && (rc = h->bias.upload(bias_f, (size_t)d.N * 4, s))) break;
        h->weights_ready = true;
        h->w16_ready = true;
        h->weight_version = d.weight_version;
        h->weight_ptr = inputs[1];
      } else {
      if ((rc = h->stage.ensure(w_elems * 4))) break;
      if ((rc = h->wq.ensure(w_elems))) break;
      if ((rc = h->scale.ensure(q_elems * 2))) break;
      if ((rc = h->zp.ensure(q_elems))) break;
      if (cudaMemcpyAsync(h->stage.p, inputs[1], w_elems * 4, cudaMemcpyHostToDevice, s) != cudaSuccess) { rc = cuda_error(cudaGetLastError(), "H2D weight", __FILE__, __LINE__); break; }
      if ((rc = f32_to_q8(h->stage.as<float>(), h->wq.p, (long long)w_elems, s))) break;
      if (cudaMemcpyAsync(h->stage.p, inputs[2], q_elems * 4, cudaMemcpyHostToDevice, s) != cudaSuccess) { rc = cuda_error(cudaGetLastError(), "H2D scale", __FILE__, __LINE__); break; }
      if ((rc = f32_to_16(h->stage.as<float>(), h->scale.p, (long long)q_elems, f16, s))) break;
      if (cudaMemcpyAsync(h->stage.p, inputs[3], q_elems * 4, cudaMemcpyHostToDevice, s) != cudaSuccess) { rc = cuda_error(cudaGetLastError(), "H2D zp", __FILE__, __LINE__); break; }
      if ((rc = f32_to_q8(h->stage.as<float>(), h->zp.p, (long long)q_elems, s))) break;
      if (bias_f && (rc = h->bias.upload(bias_f, (size_t)d.N * 4, s))) break;
      h->weights_ready = true;
      h->w16_ready = false;
      h->weight_version = d.weight_version;
      h->weight_ptr = inputs[1];
      }
    }
    const size_t x_elems = (size_t)d.M * d.K, y_elems = (size_t)d.M * d.N;
    if (x_elems == 0) break;
    if ((rc = h->stage.ensure(x_elems * 4 > w_elems * 4 ? x_elems * 4 : w_elems * 4))) break;
    if ((rc = h->x16.ensure(x_elems * 2))) break;
    if ((rc = h->y16.ensure(y_elems * 2))) break;
    if ((rc = h->y32.ensure(y_elems * 4))) break;
    if ((rc = h->status.ensure(4))) break;
    if (cudaMemsetAsync(h->status.p, 0, 4, s) != cudaSuccess) { rc = cuda_error(cudaGetLastError(), "memset", __FILE__, __LINE__); break; }
    if (cudaMemcpyAsync(h->stage.p, inputs[0], x_elems * 4, cudaMemcpyHostToDevice, s) != cudaSuccess) { rc = cuda_error(cudaGetLastError(), "H2D input", __FILE__, __LINE__); break; }
    if ((rc = f32_to_16(h->stage.as<float>(), h->x16.p, (long long)x_elems, f16, s))) break;
    if (w8) {
      if ((rc = a16_prefill_gemm(h->x16.p, h->w16.p, bias_f ? h->bias.as<float>() : nullptr, h->y16.p, d.M, (int)d.N, (int)d.K,
                                 h->status.as<int>(), s, f16))) break;
    } else if ((rc = a16_dispatch(h->x16.p, h->wq.p, h->scale.p, h->zp.p, bias_f ? h->bias.as<float>() : nullptr, h->y16.p,
                                  d.M, (int)d.N, (int)d.K, group, h->status.as<int>(), s, &h->w16, &h->w16_ready, false, f16, &h->wg_scratch))) break;
    if ((rc = f16_or_bf16_to_f32(h->y16.p, h->y32.as<float>(), (long long)y_elems, f16, s))) break;
    if (cudaMemcpyAsync(outputs[0], h->y32.p, y_elems * 4, cudaMemcpyDeviceToHost, s) != cudaSuccess) { rc = cuda_error(cudaGetLastError(), "D2H output", __FILE__, __LINE__); break; }
    int hstat = 0;
    if (cudaMemcpyAsync(&hstat, h->status.p, 4, cudaMemcpyDeviceToHost, s) != cudaSuccess) { rc = cuda_error(cudaGetLastError(), "D2H status", __FILE__, __LINE__); break; }
    if (cudaStreamSynchronize(s) != cudaSuccess) { rc = cuda_error(cudaGetLastError(), "sync", __FILE__, __LINE__); break; }
    if (hstat != 0) { rc = set_error(B200Q_ERR_TIMEOUT, "a16matmul: a bounded wait inside the kernel ran out (wait site %d)", hstat); break; }
  } while (0);
  if (rc != B200Q_OK) cudaStreamSynchronize(s);
  if (own) b200q_a16matmul_deinit(handle);
  return rc;
}

void b200q_a16_set_route(int32_t route) { g_a16_route = (route >= 0 && route <= 4) ? route : 0; }

int b200q_a16_w4_dev_dt(const void* x, const void* wq, const void* scale, const void* zp_u8, const float* bias_f32, void* y,
                        int64_t M, int64_t N, int64_t K, int32_t group, int32_t dtype, int32_t* status, void* stream) {
  if (!x || !wq || !scale || !zp_u8 || !y) return set_error(B200Q_ERR_INVALID, "a16_w4_dev: null argument");
  if (M < 0 || N < 1 || K < 1 || N > 0x7fffffffLL || K > 0x7fffffffLL || group < 1) return set_error(B200Q_ERR_INVALID, "a16_w4_dev: bad shape");
  if (dtype != B200Q_DT_BF16 && dtype != B200Q_DT_F16) return set_error(B200Q_ERR_INVALID, "a16_w4_dev: dtype must be bf16 or f16");
  return a16_dispatch(x, wq, scale, zp_u8, bias_f32, y, M, (int)N, (int)K, group, status, static_cast<cudaStream_t>(stream),
                      nullptr, nullptr, false, dtype == B200Q_DT_F16);
}

int b200q_a16_w4_dev(const void* x_bf16, const void* wq, const void* scale_bf16, const void* zp_u8,
                     const float* bias_f32, void* y_bf16, int64_t M, int64_t N, int64_t K, int32_t group,
                     int32_t* status, void* stream) {
  return b200q_a16_w4_dev_dt(x_bf16, wq, scale_bf16, zp_u8, bias_f32, y_bf16, M, N, K, group, B200Q_DT_BF16, status, stream);
}

}  // extern "C"

extern "C" {

int b200q_a16_dev_create(const void* wq, const void* scale_bf16, const void* zp_u8, const float* bias_f32, int64_t N,
                         int64_t K, int32_t group, void** handle) {
  return b200q_a16_dev_create_dt(wq, scale_bf16, zp_u8, bias_f32, N, K, group, B200Q_DT_BF16, handle);
}

int b200q_a16_dev_create_dt(const void* wq, const void* scale_bf16, const void* zp_u8, const float* bias_f32, int64_t N,
                            int64_t K, int32_t group, int32_t dtype, void** handle) {
  if (!wq || !scale_bf16 || !zp_u8 || !handle) return set_error(B200Q_ERR_INVALID, "a16_dev_create: null argument");
  if (N < 1 || K < 1 || group < 1 || N > 0x7fffffffLL || K > 0x7fffffffLL) return set_error(B200Q_ERR_INVALID, "a16_dev_create: bad shape");
  if (dtype != B200Q_DT_BF16 && dtype != B200Q_DT_F16) return set_error(B200Q_ERR_INVALID, "a16_dev_create: dtype must be bf16 or f16");
  const char* why = nullptr;
  if (!a16_w4_gemv_supported(1, (int)N, (int)K, group, &why, dtype == B200Q_DT_F16)) return set_error(B200Q_ERR_UNSUPPORTED, "a16_dev_create: %s", why);
  auto* h = new (std::nothrow) A16Handle();
  if (!h) return set_error(B200Q_ERR_NOMEM, "a16_dev_create: out of host memory");
  h->d_wq = wq;
  h->d_scale = scale_bf16;
  h->d_zp = zp_u8;
  h->d_bias = bias_f32;
  h->N = (int)N;
  h->K = (int)K;
  h->group = group;
  h->f16 = dtype == B200Q_DT_F16;
  int rc = h->status.ensure(4);
  if (rc == B200Q_OK && cudaMemset(h->status.p, 0, 4) != cudaSuccess) rc = cuda_error(cudaGetLastError(), "memset", __FILE__, __LINE__);
  if (rc != B200Q_OK) {
    delete h;
    return rc;
  }
  *handle = h;
  return B200Q_OK;
}

int b200q_a16_dev_run(void* handle, const void* x_bf16, void* y_bf16, int64_t M, void* stream) {
  if (!handle || !x_bf16 || !y_bf16 || M < 0) return set_error(B200Q_ERR_INVALID, "a16_dev_run: bad argument");
  A16Handle* h = static_cast<A16Handle*>(handle);
  return a16_dispatch(x_bf16, h->d_wq, h->d_scale, h->d_zp, h->d_bias, y_bf16, M, h->N, h->K, h->group,
                      h->status.as<int>(), static_cast<cudaStream_t>(stream), &h->w16, &h->w16_ready, true, h->f16, &h->wg_scratch);
}

int b200q_a16_dev_status(void* handle, void* stream) {
  if (!handle) return set_error(B200Q_ERR_INVALID, "a16_dev_status: null handle");
  A16Handle* h = static_cast<A16Handle*>(handle);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int hstat = 0;
  CUDA_TRY(cudaMemcpyAsync(&hstat, h->status.p, 4, cudaMemcpyDeviceToHost, s));
  CUDA_TRY(cudaStreamSynchronize(s));
  if (hstat != 0) {
    cudaMemsetAsync(h->status.p, 0, 4, s);
    return set_error(B200Q_ERR_TIMEOUT, "a16: a bounded wait inside the kernel ran out (wait site %d)", hstat);
  }
  return B200Q_OK;
}

void b200q_a16_dev_destroy(void** handle) { b200q_a16matmul_deinit(handle); }

}  // extern "C"
