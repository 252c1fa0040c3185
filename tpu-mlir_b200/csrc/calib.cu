// Calibration math on the GPU: per-sample min/max, the activation histogram, histogram folding and the
// KLD threshold search.
//
// Reference semantics (paths inside the tpu-mlir tree):
//   histogram            python/calibration/cali_math.py:68-80 (CaliMathCpu.histogram; float32 arithmetic,
//                        zeros excluded, numpy.histogram on float32 input with its float32 bin edges)
//   min/max bookkeeping  python/calibration/kld_calibrator.py:391-398
//   pad + fold           python/calibration/kld_calibrator.py:329-342
//   KLD search           bindings/kld/calibration_math.cpp:158-212 (kl_calc_thread), :273-323, :71-83
#include <math.h>

#include "calib.h"
#include "internal.h"

namespace b200q {
namespace {

// ------------------------------------------------------------------------------------------- min / max
constexpr int MM_THREADS = 256;

__device__ __forceinline__ float warp_min(float v) {
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// grid (blocks_per_sample, samples).  Block partials go to scratch; the last block of a sample to finish
// (ticket counter in scratch) reduces them, writes out[s] = {min, max} and re-arms the counter.
// NaNs are ignored (fminf/fmaxf), where numpy would propagate them.
__global__ void __launch_bounds__(MM_THREADS)
minmax_kernel(const float* __restrict__ x, long long n, float* __restrict__ out, float* __restrict__ partial,
              unsigned int* __restrict__ tickets) {
  const int s = blockIdx.y, nb = gridDim.x;
  const float* xs = x + (long long)s * n;
  float lo = INFINITY, hi = -INFINITY;
  const long long n4 = ((reinterpret_cast<uintptr_t>(xs) & 15) == 0) ? n / 4 : 0;
  const float4* x4 = reinterpret_cast<const float4*>(xs);
  for (long long i = (long long)blockIdx.x * MM_THREADS + threadIdx.x; i < n4; i += (long long)nb * MM_THREADS) {
    const float4 v = x4[i];
    lo = fminf(fminf(lo, v.x), fminf(v.y, fminf(v.z, v.w)));
    hi = fmaxf(fmaxf(hi, v.x), fmaxf(v.y, fmaxf(v.z, v.w)));
  }
  for (long long i = n4 * 4 + (long long)blockIdx.x * MM_THREADS + threadIdx.x; i < n; i += (long long)nb * MM_THREADS) {
    lo = fminf(lo, xs[i]);
    hi = fmaxf(hi, xs[i]);
  }
  __shared__ float slo[MM_THREADS / 32], shi[MM_THREADS / 32];
  __shared__ bool last;
  lo = warp_min(lo);
  hi = warp_max(hi);
  if ((threadIdx.x & 31) == 0) {
    slo[threadIdx.x >> 5] = lo;
    shi[threadIdx.x >> 5] = hi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < MM_THREADS / 32; ++w) {
      lo = fminf(lo, slo[w]);
      hi = fmaxf(hi, shi[w]);
    }
    partial[((long long)s * nb + blockIdx.x) * 2] = lo;
    partial[((long long)s * nb + blockIdx.x) * 2 + 1] = hi;
    __threadfence();
    last = atomicAdd(&tickets[s], 1u) == (unsigned)(nb - 1);
  }
  __syncthreads();
  if (last) {
    __threadfence();
    lo = INFINITY;
    hi = -INFINITY;
    for (int b = threadIdx.x; b < nb; b += MM_THREADS) {
      lo = fminf(lo, partial[((long long)s * nb + b) * 2]);
      hi = fmaxf(hi, partial[((long long)s * nb + b) * 2 + 1]);
    }
    lo = warp_min(lo);
    hi = warp_max(hi);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) {
      slo[threadIdx.x >> 5] = lo;
      shi[threadIdx.x >> 5] = hi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < MM_THREADS / 32; ++w) {
        lo = fminf(lo, slo[w]);
        hi = fmaxf(hi, shi[w]);
      }
      out[2 * s] = lo;
      out[2 * s + 1] = hi;
      tickets[s] = 0;  // ready for the next launch
    }
  }
}

// ------------------------------------------------------------------------------------------- histogram
constexpr int HIST_THREADS = 512;

// Bin of the integer-valued float k in [0, bins-1] under numpy.histogram(k, bins, range=(0, bins-1)) on
// float32 input: bin k, moved up by one when k >= (float)((k+1) * ((bins-1)/bins)) (float32 bin edges).
__device__ __forceinline__ int numpy_bin(float k, int bins, float binsf, double step) {
  int idx = (int)k;
  if (idx >= bins - 1) return bins - 1;
  // the fix-up can only trigger when 1 - (idx+1)/bins <= ulp(idx)/2 <= idx * 2^-24; test with a 2x margin
  if ((float)(bins - 1 - idx) > binsf * k * 1.2e-7f) return idx;
  const float edge = (float)((double)(idx + 1) * step);
  return idx + (k >= edge ? 1 : 0);
}

// grid (blocks_per_sample, samples).  Sample s is histogrammed with its own (threshold th[s], bins nb[s]) and
// ADDED into the first nb[s] entries of hist; nb[s] == 0 skips the sample.  Counts are privatised in shared
// memory when nb[s] fits, else they go to global memory directly.
__global__ void __launch_bounds__(HIST_THREADS)
histogram_kernel(const float* __restrict__ x, long long n, const float* __restrict__ th, const int* __restrict__ nbv,
                 int* __restrict__ hist, int smem_bins) {
  extern __shared__ int sh[];
  const int s = blockIdx.y;
  const int bins = nbv[s];
  if (bins <= 0) return;
  const bool priv = bins <= smem_bins;
  if (priv) {
    for (int i = threadIdx.x; i < bins; i += HIST_THREADS) sh[i] = 0;
    __syncthreads();
  }
  int* dst = priv ? sh : hist;
  const float binsm1 = (float)(bins - 1), binsf = (float)bins;
  const float width = __fdiv_rn(th[s], binsm1);
  const double step = (double)(bins - 1) / (double)bins;
  const float* xs = x + (long long)s * n;
  const long long n4 = ((reinterpret_cast<uintptr_t>(xs) & 15) == 0) ? n / 4 : 0;
  const float4* x4 = reinterpret_cast<const float4*>(xs);
  // t / width, correctly rounded, without a division per element: with r = RN(1/width), q0 = RN(t*r),
  // rem = t - q0*width (exact in an FMA) and q = RN(q0 + rem*r) is the correctly rounded quotient (Markstein) unless
  // width's significand is all ones; that case, and widths whose reciprocal is not a normal number, divide.
  const float rw = __frcp_rn(width);
  const uint32_t wbits = __float_as_uint(width);
  const bool quick = (wbits & 0x007fffffu) != 0x007fffffu && width >= 1e-30f && width <= 1e30f;
  auto one = [&](float v) {
    const float t = fabsf(v);
    if (!(t > 0.f)) return;  // zeros are excluded (cali_math.py:70); NaN falls out here too
    float q;
    if (quick) {
      const float q0 = __fmul_rn(t, rw);
      q = __fmaf_rn(__fmaf_rn(-q0, width, t), rw, q0);
    } else {
      q = __fdiv_rn(t, width);
    }
    const float k = floorf(__fadd_rn(q, 0.5f));
    if (!(k <= binsm1)) return;  // outside range=(0, bins-1): dropped by numpy.histogram
    atomicAdd(&dst[numpy_bin(k, bins, binsf, step)], 1);
  };
  for (long long i = (long long)blockIdx.x * HIST_THREADS + threadIdx.x; i < n4; i += (long long)gridDim.x * HIST_THREADS) {
    const float4 v = x4[i];
    one(v.x);
    one(v.y);
    one(v.z);
    one(v.w);
  }
  for (long long i = n4 * 4 + (long long)blockIdx.x * HIST_THREADS + threadIdx.x; i < n; i += (long long)gridDim.x * HIST_THREADS)
    one(xs[i]);
  if (priv) {
    __syncthreads();
    for (int i = threadIdx.x; i < bins; i += HIST_THREADS) {
      const int c = sh[i];
      if (c) atomicAdd(&hist[i], c);
    }
  }
}

// real_multi_thread_kl_diversity's own histogram (calibration_math.cpp:229-236): every value counts,
// index = floor(fabs(x) / width + 0.5) with the + 0.5 in double.
__global__ void kl_raw_histogram_kernel(const float* __restrict__ x, long long n, float width, int bins, int* hist) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const double k = floor((double)__fdiv_rn(fabsf(x[i]), width) + 0.5);
    if (k >= 0.0 && k < (double)bins) atomicAdd(&hist[(long long)k], 1);
  }
}

// out[i] = in[2i] + in[2i+1] (missing entries are zero), i < n_out: one folding step of find_threshold
__global__ void fold_kernel(const int* __restrict__ in, long long n_in, int* __restrict__ out, long long n_out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_out) return;
  const long long a = 2 * i, b = 2 * i + 1;
  out[i] = (a < n_in ? in[a] : 0) + (b < n_in ? in[b] : 0);
}

// ------------------------------------------------------------------------------------------- KLD
// One block per histogram, one thread per candidate threshold i = (m+1)*BINS.  Every float sum runs in the
// reference's order (sequential, left to right) because the counts exceed 2^24 and float addition is not
// associative; the log10 terms are formed in double and folded into a float accumulator like the reference.
__global__ void __launch_bounds__(1024)
kld_kernel(const int* __restrict__ hist_all, const long long* __restrict__ offsets, const float* __restrict__ widths,
           int BINS, float* __restrict__ thresholds, float* __restrict__ kl_all) {
  const int t = blockIdx.x;
  const int* hist = hist_all + offsets[t];
  const long long N = offsets[t + 1] - offsets[t];
  const int KL_NUM = (int)(N / BINS);
  __shared__ long long scount[32];
  __shared__ float skl[1024];
  // total count (exact, int64)
  long long c = 0;
  for (long long j = threadIdx.x; j < N; j += blockDim.x) c += hist[j];
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) scount[threadIdx.x >> 5] = c;
  __syncthreads();
  long long count = 0;
  for (int w = 0; w < (blockDim.x + 31) / 32; ++w) count += scount[w];
  const float fcount = (float)count;

  const int m = threadIdx.x;
  if (m < KL_NUM) {
    const long long i = (long long)(m + 1) * BINS;
    float tail = 0.f;  // P[i-1]: hist[i-1 .. N-1] summed left to right
    for (long long j = i - 1; j < N; ++j) tail = __fadd_rn(tail, (float)hist[j]);
    float sum = 0.f;
    for (long long j = 0; j < i; ++j) sum = __fadd_rn(sum, (float)hist[j]);
    const long long expand = i / BINS;
    float acc = 0.f;
    long long idx = 0;
    for (int b = 0; b < BINS; ++b) {
      float sum_bin = 0.f, positive = 0.f;
      for (long long k = 0; k < expand; ++k) {
        const int h = hist[idx + k];
        sum_bin = __fadd_rn(sum_bin, (float)h);
        positive = __fadd_rn(positive, h > 0 ? 1.f : 0.f);
      }
      if (positive == 0.f) positive = 1.f;
      const float q_base = __fdiv_rn(__fdiv_rn(sum_bin, positive), sum);
      for (long long k = 0; k < expand; ++k, ++idx) {
        const int h = hist[idx];
        const float p = __fdiv_rn(idx == i - 1 ? tail : (float)h, fcount);
        if (p == 0.f) continue;  // the term is exactly +-0 and leaves the accumulator unchanged
        const float q = h ? q_base : 0.f;
        const double term = __dmul_rn((double)p, __dsub_rn(log10(__dadd_rn((double)p, 1e-30)),
                                                           log10(__dadd_rn((double)q, 1e-30))));
        acc = (float)__dadd_rn((double)acc, term);
      }
    }
    skl[m] = acc;
    if (kl_all) kl_all[(long long)t * 1024 + m] = acc;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // the_min_index (calibration_math.cpp:71-83): first strict minimum
    float best = skl[0];
    int best_m = 0;
    for (int k = 1; k < KL_NUM; ++k)
      if (best > skl[k]) {
        best = skl[k];
        best_m = k;
      }
    thresholds[t] = __fmul_rn(__fmul_rn(widths[t], (float)(best_m + 1)), (float)BINS);
  }
}

}  // namespace

size_t minmax_scratch_bytes(long long samples, int blocks_per_sample) {
  return (size_t)samples * blocks_per_sample * 2 * sizeof(float) + (size_t)samples * sizeof(unsigned int);
}

int minmax_blocks_per_sample(long long n, long long samples) {
  long long want = (n + MM_THREADS * 16 - 1) / (MM_THREADS * 16);  // >= 16 float4 per thread... at most
  long long cap = 148LL * 8 / (samples > 0 ? samples : 1);
  if (cap < 1) cap = 1;
  if (want > cap) want = cap;
  if (want < 1) want = 1;
  return (int)want;
}

int minmax_launch(const float* x, long long n, long long samples, float* out, void* scratch, int blocks_per_sample,
                  cudaStream_t s) {
  if (samples == 0) return B200Q_OK;
  if (samples > 65535) return set_error(B200Q_ERR_UNSUPPORTED, "minmax: at most 65535 samples per call");
  float* partial = static_cast<float*>(scratch);
  unsigned int* tickets = reinterpret_cast<unsigned int*>(partial + (size_t)samples * blocks_per_sample * 2);
  dim3 grid(blocks_per_sample, (unsigned)samples);
  minmax_kernel<<<grid, MM_THREADS, 0, s>>>(x, n, out, partial, tickets);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}


// ------------------------------------------------------------------------------------------- min/max without allocation
// Scratch of the min/max kernel for callers that must not allocate: a fixed array that lives in the module
// image of every GPU that loads this library (36 KB per GPU, held until the process exits).
// Layout: [STATIC_MM_MAX_SAMPLES ticket counters][STATIC_MM_MAX_PARTIALS {min, max} pairs].
constexpr int STATIC_MM_MAX_SAMPLES = 1024;
constexpr int STATIC_MM_MAX_PARTIALS = 4096;
constexpr size_t STATIC_MM_TICKET_BYTES = STATIC_MM_MAX_SAMPLES * sizeof(unsigned int);
constexpr size_t STATIC_MM_BYTES = STATIC_MM_TICKET_BYTES + (size_t)STATIC_MM_MAX_PARTIALS * 2 * sizeof(float);
static __device__ __align__(256) unsigned char g_static_minmax_scratch[STATIC_MM_BYTES];

constexpr int MAX_DEVICES = 64;
static void* g_static_scratch_addr[MAX_DEVICES];  // device address of the array, per device ordinal

// In host code the array's name is only a handle for the runtime, not a device address: the address a
// kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.
int static_scratch_for_current_device(void** out) {
  int dev = -1;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) return set_error(B200Q_ERR_UNSUPPORTED, "minmax_static: device ordinal %d not supported", dev);
  if (!g_static_scratch_addr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_minmax_scratch);
    if (e != cudaSuccess) return cuda_error(e, "cudaGetSymbolAddress(g_static_minmax_scratch)", __FILE__, __LINE__);
    if (!p) return set_error(B200Q_ERR_CUDA, "minmax_static: the scratch symbol has no device address");
    g_static_scratch_addr[dev] = p;
  }
  *out = g_static_scratch_addr[dev];
  return B200Q_OK;
}

int minmax_static_launch(const float* x, long long n, long long samples, float* out, cudaStream_t s) {
  if (samples == 0) return B200Q_OK;
  if (samples > STATIC_MM_MAX_SAMPLES)
    return set_error(B200Q_ERR_UNSUPPORTED, "minmax_static: %lld samples exceed the fixed scratch (at most %d per call)",
                     samples, STATIC_MM_MAX_SAMPLES);
  int bps = minmax_blocks_per_sample(n, samples);
  if ((long long)bps * samples > STATIC_MM_MAX_PARTIALS) bps = (int)(STATIC_MM_MAX_PARTIALS / samples);
  if (bps < 1) bps = 1;
  void* base = nullptr;
  B200Q_TRY(static_scratch_for_current_device(&base));
  unsigned int* tickets = static_cast<unsigned int*>(base);
  float* partial = reinterpret_cast<float*>(static_cast<unsigned char*>(base) + STATIC_MM_TICKET_BYTES);
  // the array keeps whatever the previous call left: the ticket counters must start at zero
  CUDA_TRY(cudaMemsetAsync(tickets, 0, (size_t)samples * sizeof(unsigned int), s));
  dim3 grid(bps, (unsigned)samples);
  minmax_kernel<<<grid, MM_THREADS, 0, s>>>(x, n, out, partial, tickets);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int histogram_launch(const float* x, long long n, long long samples, const float* th, const int* nb, int* hist,
                     int max_bins, cudaStream_t s) {
  if (samples == 0 || n == 0) return B200Q_OK;
  if (samples > 65535) return set_error(B200Q_ERR_UNSUPPORTED, "histogram: at most 65535 samples per call");
  // shared-memory privatisation up to 48K bins (192 KB); sized by the largest bin count the caller announces
  int smem_bins = max_bins <= 49152 ? max_bins : 0;
  const size_t smem = (size_t)smem_bins * sizeof(int);
  if (smem > 48 * 1024) CUDA_TRY(cudaFuncSetAttribute(histogram_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  long long bps = (n + HIST_THREADS * 32 - 1) / (HIST_THREADS * 32);
  const long long cap = 148LL * 4 / samples > 0 ? 148LL * 4 / samples : 1;
  if (bps > cap) bps = cap;
  if (bps < 1) bps = 1;
  dim3 grid((unsigned)bps, (unsigned)samples);
  histogram_kernel<<<grid, HIST_THREADS, smem, s>>>(x, n, th, nb, hist, smem_bins);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int kl_raw_histogram_launch(const float* x, long long n, float width, int bins, int* hist, cudaStream_t s) {
  if (n == 0) return B200Q_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  kl_raw_histogram_kernel<<<(unsigned)blocks, 256, 0, s>>>(x, n, width, bins, hist);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int fold_launch(const int* in, long long n_in, int* out, long long n_out, cudaStream_t s) {
  if (n_out == 0) return B200Q_OK;
  fold_kernel<<<(unsigned)((n_out + 255) / 256), 256, 0, s>>>(in, n_in, out, n_out);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

int kld_launch(const int* hist_all, const long long* offsets_dev, const float* widths_dev, int tensors, int dst_bins,
               long long max_bins, float* thresholds_dev, float* kl_dev, cudaStream_t s) {
  if (tensors == 0) return B200Q_OK;
  if (dst_bins < 1 || max_bins / dst_bins > 1024)
    return set_error(B200Q_ERR_UNSUPPORTED, "kld: more than 1024 candidates (fold the histogram to at most %d bins first)", 1024 * dst_bins);
  int threads = (int)((max_bins / dst_bins + 31) / 32 * 32);
  if (threads < 32) threads = 32;
  kld_kernel<<<tensors, threads, 0, s>>>(hist_all, offsets_dev, widths_dev, dst_bins, thresholds_dev, kl_dev);
  CUDA_TRY(cudaGetLastError());
  return B200Q_OK;
}

}  // namespace b200q
