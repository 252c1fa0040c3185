// C ABI of the calibration math: a context that owns the scratch memory of the min/max, histogram and KLD
// kernels, plus the two entry points of the reference's calibration_math.so
// (bindings/kld/calibration_math.cpp:326-337) so that kld_calibrator.py:50-59 can load this library instead.
#include <cmath>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "calib.h"
#include "devbuf.h"
#include "internal.h"

namespace b200q {
namespace {

constexpr long long MAX_KLD_BINS = 64 * 2048;  // kld_calibrator.py:338

struct CalibCtx {
  DevBuf mm_scratch, params, work, work2, offsets, widths, thresholds, kl, stage, mm_out;
  size_t mm_scratch_zeroed = 0;
};

long long pad_to(long long n, long long m) { return (n + m - 1) / m * m; }

// pad + fold plan of find_threshold (kld_calibrator.py:329-342): final length and width
void fold_plan(long long nb, float width, long long dst_bins, long long* len_out, float* width_out, int* folds) {
  long long L = pad_to(nb, dst_bins);
  int f = 0;
  while (L > MAX_KLD_BINS) {
    L = pad_to(L / 2, dst_bins);
    width = width * 2.0f;
    ++f;
  }
  *len_out = L;
  *width_out = width;
  *folds = f;
}

int find_thresholds(CalibCtx* c, int tensors, const int32_t* const* hist_dev, const int64_t* n_bins,
                    const float* widths, long long dst_bins, float* thresholds_host, float* kl_host, cudaStream_t s) {
  if (tensors == 0) return B200Q_OK;
  if (dst_bins != 128 && dst_bins != 8) return set_error(B200Q_ERR_INVALID, "find_threshold: dst_bins must be 128 or 8 (asserted by the reference)");
  std::vector<long long> offs((size_t)tensors + 1, 0);
  std::vector<float> wfinal((size_t)tensors);
  std::vector<int> folds((size_t)tensors);
  long long max_len = 0, max_tmp = 0;
  for (int t = 0; t < tensors; ++t) {
    if (n_bins[t] < 1 || !hist_dev[t]) return set_error(B200Q_ERR_INVALID, "find_threshold: empty histogram %d", t);
    long long L;
    fold_plan(n_bins[t], widths[t], dst_bins, &L, &wfinal[(size_t)t], &folds[(size_t)t]);
    offs[(size_t)t + 1] = offs[(size_t)t] + L;
    if (L > max_len) max_len = L;
    if (folds[(size_t)t] > 1) {
      const long long tmp = pad_to(pad_to(n_bins[t], dst_bins) / 2, dst_bins);
      if (tmp > max_tmp) max_tmp = tmp;
    }
  }
  B200Q_TRY(c->work.ensure((size_t)offs[(size_t)tensors] * 4));
  if (max_tmp) {
    B200Q_TRY(c->work2.ensure((size_t)max_tmp * 4));
    B200Q_TRY(c->stage.ensure((size_t)max_tmp * 4));
  }
  int* work = c->work.as<int>();
  for (int t = 0; t < tensors; ++t) {
    int* dst = work + offs[(size_t)t];
    const long long L = offs[(size_t)t + 1] - offs[(size_t)t];
    if (folds[(size_t)t] == 0) {
      CUDA_TRY(cudaMemcpyAsync(dst, hist_dev[t], (size_t)n_bins[t] * 4, cudaMemcpyDeviceToDevice, s));
      if (L > n_bins[t]) CUDA_TRY(cudaMemsetAsync(dst + n_bins[t], 0, (size_t)(L - n_bins[t]) * 4, s));
    } else {
      // fold chain; intermediate results ping-pong between two scratch buffers, the last step lands in `dst`
      const int* src = hist_dev[t];
      long long n_in = n_bins[t], cur = pad_to(n_bins[t], dst_bins);
      int* bufs[2] = {c->work2.as<int>(), c->stage.as<int>()};
      for (int f = 0; f < folds[(size_t)t]; ++f) {
        const long long n_out = pad_to(cur / 2, dst_bins);
        int* out = (f == folds[(size_t)t] - 1) ? dst : bufs[f & 1];
        B200Q_TRY(fold_launch(src, n_in, out, n_out, s));
        src = out;
        n_in = n_out;
        cur = n_out;
      }
    }
  }
  B200Q_TRY(c->offsets.upload(offs.data(), offs.size() * sizeof(long long), s));
  B200Q_TRY(c->widths.upload(wfinal.data(), wfinal.size() * sizeof(float), s));
  B200Q_TRY(c->thresholds.ensure((size_t)tensors * 4));
  float* kl_dev = nullptr;
  if (kl_host) {
    B200Q_TRY(c->kl.ensure((size_t)tensors * 1024 * 4));
    kl_dev = c->kl.as<float>();
  }
  B200Q_TRY(kld_launch(work, c->offsets.as<long long>(), c->widths.as<float>(), tensors, (int)dst_bins, max_len,
                       c->thresholds.as<float>(), kl_dev, s));
  CUDA_TRY(cudaMemcpyAsync(thresholds_host, c->thresholds.p, (size_t)tensors * 4, cudaMemcpyDeviceToHost, s));
  if (kl_host) CUDA_TRY(cudaMemcpyAsync(kl_host, c->kl.p, (size_t)tensors * 1024 * 4, cudaMemcpyDeviceToHost, s));
  CUDA_TRY(cudaStreamSynchronize(s));
  return B200Q_OK;
}

CalibCtx* global_ctx() {
  static CalibCtx* ctx = new (std::nothrow) CalibCtx();
  return ctx;
}
std::mutex g_mutex;

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_calib_create(void** ctx) {
  if (!ctx) return set_error(B200Q_ERR_INVALID, "calib_create: null argument");
  auto* c = new (std::nothrow) CalibCtx();
  if (!c) return set_error(B200Q_ERR_NOMEM, "calib_create: out of host memory");
  *ctx = c;
  return B200Q_OK;
}

void b200q_calib_destroy(void** ctx) {
  if (ctx && *ctx) {
    delete static_cast<CalibCtx*>(*ctx);
    *ctx = nullptr;
  }
}

int b200q_calib_minmax(void* ctx, const float* x_dev, int64_t n_per_sample, int64_t samples, float* out_dev,
                       void* stream) {
  if (!ctx || !x_dev || !out_dev || n_per_sample < 1 || samples < 0) return set_error(B200Q_ERR_INVALID, "calib_minmax: bad argument");
  CalibCtx* c = static_cast<CalibCtx*>(ctx);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int bps = minmax_blocks_per_sample(n_per_sample, samples);
  const size_t need = minmax_scratch_bytes(samples, bps);
  if (need > c->mm_scratch.cap || c->mm_scratch_zeroed < need) {
    B200Q_TRY(c->mm_scratch.ensure(need));
    CUDA_TRY(cudaMemsetAsync(c->mm_scratch.p, 0, c->mm_scratch.cap, s));  // ticket counters start at zero
    c->mm_scratch_zeroed = c->mm_scratch.cap;
  } else {
    // the ticket area moves with (samples, bps): clear it (cheap) so that any layout starts from zero
    CUDA_TRY(cudaMemsetAsync(static_cast<char*>(c->mm_scratch.p) + (size_t)samples * bps * 8, 0, (size_t)samples * 4, s));
  }
  return minmax_launch(x_dev, n_per_sample, samples, out_dev, c->mm_scratch.p, bps, s);
}

int b200q_calib_minmax_noalloc(const float* x_dev, int64_t n_per_sample, int64_t samples, float* out_dev, void* stream) {
  if (!x_dev || !out_dev || n_per_sample < 1 || samples < 0) return set_error(B200Q_ERR_INVALID, "calib_minmax_noalloc: bad argument");
  return minmax_static_launch(x_dev, n_per_sample, samples, out_dev, static_cast<cudaStream_t>(stream));
}

int b200q_calib_histogram(void* ctx, const float* x_dev, int64_t n_per_sample, int64_t samples, const float* th_host,
                          const int32_t* nbins_host, int32_t* hist_dev, int64_t hist_len, void* stream) {
  if (!ctx || !x_dev || !th_host || !nbins_host || !hist_dev || n_per_sample < 1 || samples < 0)
    return set_error(B200Q_ERR_INVALID, "calib_histogram: bad argument");
  CalibCtx* c = static_cast<CalibCtx*>(ctx);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int max_bins = 0;
  for (int64_t i = 0; i < samples; ++i) {
    if (nbins_host[i] < 0 || nbins_host[i] > hist_len) return set_error(B200Q_ERR_INVALID, "calib_histogram: nbins[%lld] = %d exceeds the histogram length %lld", (long long)i, nbins_host[i], (long long)hist_len);
    if (nbins_host[i] == 1) return set_error(B200Q_ERR_INVALID, "calib_histogram: a histogram needs at least 2 bins");
    if (nbins_host[i] > max_bins) max_bins = nbins_host[i];
  }
  if (max_bins == 0) return B200Q_OK;
  // th | nbins packed in one upload
  std::vector<char> packed((size_t)samples * 8);
  memcpy(packed.data(), th_host, (size_t)samples * 4);
  memcpy(packed.data() + (size_t)samples * 4, nbins_host, (size_t)samples * 4);
  B200Q_TRY(c->params.upload(packed.data(), packed.size(), s));
  return histogram_launch(x_dev, n_per_sample, samples, c->params.as<float>(),
                          reinterpret_cast<const int*>(c->params.as<char>() + (size_t)samples * 4), hist_dev, max_bins, s);
}

void b200q_calib_set_histogram_layout(int32_t mode) { histogram_set_mode(mode); }

int b200q_calib_find_thresholds(void* ctx, int32_t tensors, const int32_t* const* hist_dev, const int64_t* n_bins,
                                const float* widths, int64_t dst_bins, float* thresholds_host, float* kl_host,
                                void* stream) {
  if (!ctx || tensors < 0 || (tensors > 0 && (!hist_dev || !n_bins || !widths || !thresholds_host)))
    return set_error(B200Q_ERR_INVALID, "calib_find_thresholds: bad argument");
  return find_thresholds(static_cast<CalibCtx*>(ctx), tensors, hist_dev, n_bins, widths, dst_bins, thresholds_host,
                         kl_host, static_cast<cudaStream_t>(stream));
}

// ---- the reference's calibration_math ABI (calibration_math.cpp:326-337); like the reference these report
// failure only by their return value, here NaN (message through b200q_last_error()).
float kl_diversity_hist(int* data, float width, long long num_bins, long long dst_bins) {
  std::lock_guard<std::mutex> lock(g_mutex);
  CalibCtx* c = global_ctx();
  if (!c || !data || num_bins < dst_bins || num_bins % dst_bins != 0) {
    set_error(B200Q_ERR_INVALID, "kl_diversity_hist: bad argument");
    return NAN;
  }
  cudaStream_t s = 0;
  if (c->stage.upload(data, (size_t)num_bins * 4, s) != B200Q_OK) return NAN;
  // the caller (find_threshold) has already padded and folded: run the search on the histogram as given
  if (num_bins / dst_bins > 1024) {
    set_error(B200Q_ERR_UNSUPPORTED, "kl_diversity_hist: more than 1024 candidates");
    return NAN;
  }
  const long long offs[2] = {0, num_bins};
  float th = NAN;
  if (c->offsets.upload(offs, sizeof(offs), s) != B200Q_OK || c->widths.upload(&width, 4, s) != B200Q_OK ||
      c->thresholds.ensure(4) != B200Q_OK)
    return NAN;
  if (kld_launch(c->stage.as<int>(), c->offsets.as<long long>(), c->widths.as<float>(), 1, (int)dst_bins, num_bins,
                 c->thresholds.as<float>(), nullptr, s) != B200Q_OK)
    return NAN;
  if (cudaMemcpyAsync(&th, c->thresholds.p, 4, cudaMemcpyDeviceToHost, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess) {
    cuda_error(cudaGetLastError(), "kl_diversity_hist", __FILE__, __LINE__);
    return NAN;
  }
  return th;
}

float kl_diversity(float* data, long long count, long long num_bins) {
  std::lock_guard<std::mutex> lock(g_mutex);
  CalibCtx* c = global_ctx();
  const long long BINS = 128;
  if (!c || !data || count < 1 || num_bins < BINS || num_bins % BINS != 0 || num_bins / BINS > 1024) {
    set_error(B200Q_ERR_INVALID, "kl_diversity: bad argument");
    return NAN;
  }
  cudaStream_t s = 0;
  // data_max = max |x| (calibration_math.cpp:60-68), width = data_max / (N - 1)
  if (c->work2.upload(data, (size_t)count * 4, s) != B200Q_OK || c->mm_out.ensure(8) != B200Q_OK) return NAN;
  const int bps = minmax_blocks_per_sample(count, 1);
  if (c->mm_scratch.ensure(minmax_scratch_bytes(1, bps)) != B200Q_OK) return NAN;
  cudaMemsetAsync(c->mm_scratch.p, 0, c->mm_scratch.cap, s);
  c->mm_scratch_zeroed = c->mm_scratch.cap;
  if (minmax_launch(c->work2.as<float>(), count, 1, c->mm_out.as<float>(), c->mm_scratch.p, bps, s) != B200Q_OK) return NAN;
  float mm[2];
  if (cudaMemcpyAsync(mm, c->mm_out.p, 8, cudaMemcpyDeviceToHost, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess) return NAN;
  const float data_max = fmaxf(fabsf(mm[0]), fabsf(mm[1]));
  const float width = data_max / (float)(num_bins - 1);
  if (c->stage.ensure((size_t)num_bins * 4) != B200Q_OK) return NAN;
  cudaMemsetAsync(c->stage.p, 0, (size_t)num_bins * 4, s);
  if (kl_raw_histogram_launch(c->work2.as<float>(), count, width, (int)num_bins, c->stage.as<int>(), s) != B200Q_OK) return NAN;
  const long long offs[2] = {0, num_bins};
  float th = NAN;
  if (c->offsets.upload(offs, sizeof(offs), s) != B200Q_OK || c->widths.upload(&width, 4, s) != B200Q_OK ||
      c->thresholds.ensure(4) != B200Q_OK)
    return NAN;
  if (kld_launch(c->stage.as<int>(), c->offsets.as<long long>(), c->widths.as<float>(), 1, (int)BINS, num_bins,
                 c->thresholds.as<float>(), nullptr, s) != B200Q_OK)
    return NAN;
  if (cudaMemcpyAsync(&th, c->thresholds.p, 4, cudaMemcpyDeviceToHost, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess) return NAN;
  return th;
}

}  // extern "C"
