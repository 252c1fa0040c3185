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

#include <atomic>
#include <type_traits>

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
constexpr int HIST_THREADS = 1024;
constexpr int HIST_SMEM_BYTES = 208 * 1024;        // counters of one block (one block per SM)
constexpr long long HIST_FLUSH_ELEMS = 1998848;    // 488 * 4096 elements: the longest run a block counts without a merge
constexpr long long HIST_MERGE_EVERY = 2040;       // per-thread element budget between merges: 32 warps x 2040 < 2^16
constexpr uint32_t FLOOR_MAGIC = 0x4B000000u;      // bits of 2^23

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

// How a block keeps its counters in shared memory.
//   LANE16: every lane of a warp owns one bank.  Word (bin >> 1) * 32 + lane holds two 16-bit counters (bins 2j and
//           2j + 1) that only threads with this lane index touch: an update never meets a bank conflict nor another
//           lane's update of the same address, however the values pile up in a few bins.  A counter receives at most
//           32 warps x 2040 elements between two merges, so it cannot carry into its neighbour.
//   copies: 2^L 32-bit counters per bin, copy = lane mod 2^L (L = 0: one privatised copy); for bin counts whose
//           LANE16 form does not fit.  Bin counts that do not fit at all count straight into global memory.
struct HistGeom {
  int lane16;      // 1 = LANE16
  int copies_log2; // otherwise
  int cap_words;   // shared-memory words available
};

// Persistent: block b owns the flat element range [b * piece, (b + 1) * piece) of x[samples][n].  Sample s is
// histogrammed with its own (threshold th[s], bins nb[s]) and ADDED into the first nb[s] entries of hist; nb[s] == 0
// skips the sample.  Counters stay in shared memory across samples that share (threshold, bins) and are merged into
// hist when the geometry changes, before a 16-bit counter could overflow, and at the end.
template <bool LANE16>
__global__ void __launch_bounds__(HIST_THREADS, 1)
histogram_kernel(const float* __restrict__ x, long long n, long long samples, long long piece, const float* __restrict__ th,
                 const int* __restrict__ nbv, int* __restrict__ hist, int copies_log2, int cap_words, int zero_words) {
  extern __shared__ unsigned int sh[];
  const int tid = threadIdx.x, lane = tid & 31;
  const long long total = samples * n;
  const long long begin = (long long)blockIdx.x * piece;
  const long long end = begin + piece < total ? begin + piece : total;
  if (begin >= end) return;
  for (int i = tid; i < zero_words; i += HIST_THREADS) sh[i] = 0u;
  __syncthreads();

  int cur_bins = 0;            // geometry of the counters now in shared memory (0: none)
  uint32_t cur_th = 0;
  bool cur_shared = false;
  long long since_merge = 0;
  const int lcopy = lane & ((1 << copies_log2) - 1);

  auto merge = [&]() {
    if (cur_bins == 0 || !cur_shared) return;
    __syncthreads();
    // counters are indexed by k; numpy.histogram puts k into bin k or, by its float32 bin edges, into bin k + 1
    const float cur_binsf = (float)cur_bins;
    const double cur_step = (double)(cur_bins - 1) / (double)cur_bins;
    if (LANE16) {
      const int pairs = (cur_bins + 1) >> 1;
      for (int p = tid; p < pairs; p += HIST_THREADS) {
        unsigned lo = 0, hi = 0;
#pragma unroll 8
        for (int j = 0; j < 32; ++j) {
          const int w = p * 32 + ((j + lane) & 31);
          const unsigned v = sh[w];
          sh[w] = 0u;
          lo += v & 0xffffu;
          hi += v >> 16;
        }
        if (lo) atomicAdd(&hist[numpy_bin((float)(2 * p), cur_bins, cur_binsf, cur_step)], (int)lo);
        if (hi) atomicAdd(&hist[numpy_bin((float)(2 * p + 1), cur_bins, cur_binsf, cur_step)], (int)hi);
      }
    } else {
      const int R = 1 << copies_log2;
      for (int b = tid; b < cur_bins; b += HIST_THREADS) {
        unsigned c = 0;
        for (int j = 0; j < R; ++j) {
          const int w = (b << copies_log2) + ((j + lane) & (R - 1));
          c += sh[w];
          sh[w] = 0u;
        }
        if (c) atomicAdd(&hist[numpy_bin((float)b, cur_bins, cur_binsf, cur_step)], (int)c);
      }
    }
    __syncthreads();
    since_merge = 0;
  };

  long long pos = begin;
  while (pos < end) {
    const long long s = pos / n;
    long long seg_end = (s + 1) * n < end ? (s + 1) * n : end;
    const int bins = nbv[s];
    if (bins <= 0) {
      pos = seg_end;
      continue;
    }
    const float thv = th[s];
    if (bins != cur_bins || __float_as_uint(thv) != cur_th) {
      merge();
      cur_bins = bins;
      cur_th = __float_as_uint(thv);
      cur_shared = LANE16 ? (((bins + 1) >> 1) * 32 <= cap_words) : (((long long)bins << copies_log2) <= cap_words);
    }
    if (LANE16 && cur_shared) {
      // elements one thread can add to its lane's counters in this segment (float4 body + scalar head and tail)
      long long per_thread = (((seg_end - pos) >> 2) + HIST_THREADS - 1) / HIST_THREADS * 4 + 14;
      if (per_thread > HIST_MERGE_EVERY) {
        seg_end = pos + HIST_FLUSH_ELEMS;
        per_thread = ((HIST_FLUSH_ELEMS >> 2) + HIST_THREADS - 1) / HIST_THREADS * 4 + 14;
      }
      if (since_merge + per_thread > HIST_MERGE_EVERY) merge();
      since_merge += per_thread;
    }
    const bool shared_now = cur_shared;
    const float binsf = (float)bins;
    const uint32_t top = (uint32_t)(bins - 1);
    const float width = __fdiv_rn(thv, (float)(bins - 1));
    const double step = (double)(bins - 1) / (double)bins;
    // t / width, correctly rounded, without a division per element: with r = RN(1/width), q0 = RN(t*r),
    // rem = t - q0*width (exact in an FMA) and q = RN(q0 + rem*r) is the correctly rounded quotient (Markstein) unless
    // width's significand is all ones; that case, and widths whose reciprocal is not a normal number, divide.
    const float rw = __frcp_rn(width);
    const uint32_t wbits = __float_as_uint(width);
    const bool quick = (wbits & 0x007fffffu) != 0x007fffffu && width >= 1e-30f && width <= 1e30f;
    const uint32_t sh_base = static_cast<uint32_t>(__cvta_generic_to_shared(sh));
    // Per element, branch-free: quotient, k = floor(q + 0.5) as the low mantissa bits of a float, two comparisons,
    // one predicated shared-memory reduction.  FLOOR_MAGIC is folded into the comparison and into the address
    // (arithmetic modulo 2^32).  Shared counters are indexed by k itself; numpy's float32-edge rule, which sends
    // some k to bin k + 1, depends on k alone and is applied when the counters are merged.
    const uint32_t k_limit = FLOOR_MAGIC + top;   // largest valid bit pattern
    const uint32_t lane16_bias = sh_base + (uint32_t)lane * 4u - FLOOR_MAGIC * 64u;
    const uint32_t copies_bias = sh_base + (uint32_t)lcopy * 4u - ((FLOOR_MAGIC << copies_log2) << 2);
    const uint32_t copies_mul = 4u << copies_log2;
    auto run = [&](auto quick_tag, auto shared_tag) {
      constexpr bool QUICK = decltype(quick_tag)::value;
      constexpr bool SHARED = decltype(shared_tag)::value;
      auto one = [&](float v) {
        const float t = fabsf(v);
        float q;
        if (QUICK) {
          const float q0 = __fmul_rn(t, rw);
          q = __fmaf_rn(__fmaf_rn(-q0, width, t), rw, q0);
        } else {
          q = __fdiv_rn(t, width);
        }
        // k = floor(RN(q + 0.5)): adding 2^23 with rounding toward minus infinity leaves floor(y) in the low mantissa
        // bits for 0 <= y < 2^23; larger y (and infinity) give bit patterns above every valid bin and are dropped,
        // like values outside range=(0, bins-1) in numpy.histogram.  Zeros are excluded (cali_math.py:70); a NaN
        // fails t > 0 too.
        const uint32_t ub = __float_as_uint(__fadd_rd(__fadd_rn(q, 0.5f), 8388608.0f));
        if (!SHARED) {
          if (t > 0.f && ub <= k_limit) atomicAdd(&hist[numpy_bin((float)(ub - FLOOR_MAGIC), bins, binsf, step)], 1);
        } else {
          const uint32_t addr = LANE16 ? (ub & ~1u) * 64u + lane16_bias : ub * copies_mul + copies_bias;
          const uint32_t inc = LANE16 ? (ub & 1u) * 65535u + 1u : 1u;
          asm volatile(
              "{\n\t"
              ".reg .pred p, q;\n\t"
              "setp.gt.f32 q, %2, 0f00000000;\n\t"
              "setp.le.and.u32 p, %3, %4, q;\n\t"
              "@p red.shared.add.u32 [%0], %1;\n\t"
              "}\n" ::"r"(addr), "r"(inc), "f"(t), "r"(ub), "r"(k_limit)
              : "memory");
        }
      };
      // the segment [pos, seg_end) of the flat array: scalars up to a 16-byte boundary, float4 body, scalar tail
      const float* p = x + pos;
      const long long len = seg_end - pos;
      long long head = (long long)((16 - (reinterpret_cast<uintptr_t>(p) & 15)) & 15) >> 2;
      if (head > len) head = len;
      if (tid < head) one(p[tid]);
      const long long body4 = (len - head) >> 2;
      const float4* p4 = reinterpret_cast<const float4*>(p + head);
      // three float4 per thread per step, the next step's loads requested before this step's values are counted
      // (positions past the end read as zeros, which the histogram ignores)
      const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
      long long i = tid;
      float4 c0 = i < body4 ? __ldcs(p4 + i) : zero4;
      float4 c1 = i + HIST_THREADS < body4 ? __ldcs(p4 + i + HIST_THREADS) : zero4;
      float4 c2 = i + 2 * HIST_THREADS < body4 ? __ldcs(p4 + i + 2 * HIST_THREADS) : zero4;
      for (; i < body4; i += 3 * HIST_THREADS) {
        const long long j = i + 3 * HIST_THREADS;
        const float4 n0 = j < body4 ? __ldcs(p4 + j) : zero4;
        const float4 n1 = j + HIST_THREADS < body4 ? __ldcs(p4 + j + HIST_THREADS) : zero4;
        const float4 n2 = j + 2 * HIST_THREADS < body4 ? __ldcs(p4 + j + 2 * HIST_THREADS) : zero4;
        one(c0.x); one(c0.y); one(c0.z); one(c0.w);
        one(c1.x); one(c1.y); one(c1.z); one(c1.w);
        one(c2.x); one(c2.y); one(c2.z); one(c2.w);
        c0 = n0; c1 = n1; c2 = n2;
      }
      const long long done = head + body4 * 4;
      if (done + tid < len) one(p[done + tid]);
    };
    if (quick) {
      if (shared_now) run(std::true_type{}, std::true_type{});
      else run(std::true_type{}, std::false_type{});
    } else {
      if (shared_now) run(std::false_type{}, std::true_type{});
      else run(std::false_type{}, std::false_type{});
    }
    pos = seg_end;
  }
  merge();
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
static std::atomic<void*> g_static_scratch_addr[MAX_DEVICES];  // device address of the array, per device ordinal

// In host code the array's name is only a handle for the runtime, not a device address: the address a
// kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.
int static_scratch_for_current_device(void** out) {
  int dev = -1;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) return set_error(B200Q_ERR_UNSUPPORTED, "minmax_static: device ordinal %d not supported", dev);
  // Threads that make their first call on a device at the same time each ask the runtime and store the same
  // answer; the atomic makes that harmless.  (The cache does not survive a cudaDeviceReset of that device.)
  void* p = g_static_scratch_addr[dev].load(std::memory_order_acquire);
  if (!p) {
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_minmax_scratch);
    if (e != cudaSuccess) return cuda_error(e, "cudaGetSymbolAddress(g_static_minmax_scratch)", __FILE__, __LINE__);
    if (!p) return set_error(B200Q_ERR_CUDA, "minmax_static: the scratch symbol has no device address");
    g_static_scratch_addr[dev].store(p, std::memory_order_release);
  }
  *out = p;
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

static int g_hist_mode = -1;  // -1: chosen per launch; 0..4: 2^mode copies; 5: lane-owned 16-bit counters
void histogram_set_mode(int mode) { g_hist_mode = (mode >= 0 && mode <= 5) ? mode : -1; }

int histogram_launch(const float* x, long long n, long long samples, const float* th, const int* nb, int* hist,
                     int max_bins, cudaStream_t s) {
  if (samples == 0 || n == 0) return B200Q_OK;
  int dev = 0, sms = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const long long total = samples * n;
  // one block per SM; a block's piece is a multiple of one float4 per thread and at least 16 of them
  const long long quantum = 4LL * HIST_THREADS;
  long long blocks = (total + 16 * quantum - 1) / (16 * quantum);
  if (blocks > sms) blocks = sms;
  if (blocks < 1) blocks = 1;
  long long piece = (total + blocks - 1) / blocks;
  piece = (piece + quantum - 1) / quantum * quantum;
  blocks = (total + piece - 1) / piece;
  const int cap_words = HIST_SMEM_BYTES / 4;
  const long long lane16_words = (long long)((max_bins + 1) / 2) * 32;
  // Chosen layout: four copies per bin.  Measured on 64 x 802 816 normal values, 2048 bins: one copy 41.9 us, four
  // 42.2 us, sixteen 43.7 us, lane-owned 16-bit counters 46.3 us (two more instructions per element cost more than the
  // conflicts they avoid); on 64 x 100 352 values four copies are the fastest (20.0 us).  Copies also keep skewed data
  // (everything in a few bins) from serialising on one address.  Fewer copies when the bins do not fit, or when a
  // block would spend more than a quarter of its element count clearing and summing counters.
  int mode = g_hist_mode;
  if (mode < 0) {
    mode = 2;
    while (mode > 0 && (((long long)max_bins << mode) > cap_words || ((long long)max_bins << mode) * 4 > piece)) --mode;
  }
  if (mode == 5 && lane16_words > cap_words) mode = 0;
  while (mode > 0 && mode < 5 && ((long long)max_bins << mode) > cap_words) --mode;
  long long zero_words = mode == 5 ? lane16_words : ((long long)max_bins << mode);
  if (zero_words > cap_words) zero_words = 0;  // nothing fits: every sample counts into global memory
  const size_t smem = (size_t)(zero_words > 0 ? zero_words : 1) * 4;
  auto kfn = mode == 5 ? histogram_kernel<true> : histogram_kernel<false>;
  CUDA_TRY(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, HIST_SMEM_BYTES));
  kfn<<<(unsigned)blocks, HIST_THREADS, smem, s>>>(x, n, samples, piece, th, nb, hist, mode == 5 ? 0 : mode,
                                                   (int)zero_words, (int)zero_words);
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
