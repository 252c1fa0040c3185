// Calibration kernel launchers (calib.cu).  All asynchronous on the given stream.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

namespace b200q {

int minmax_blocks_per_sample(long long n, long long samples);
size_t minmax_scratch_bytes(long long samples, int blocks_per_sample);
// out[s] = {min, max} of x[s*n .. (s+1)*n); scratch must be zero-initialised once and is left re-armed
int minmax_launch(const float* x, long long n, long long samples, float* out, void* scratch, int blocks_per_sample,
                  cudaStream_t s);
// Same result as minmax_launch with the scratch in a fixed device array of the library: no allocation.
int minmax_static_launch(const float* x, long long n, long long samples, float* out, cudaStream_t s);
// hist[0 .. nb[s]) += histogram of sample s with threshold th[s]; th / nb are DEVICE arrays
int histogram_launch(const float* x, long long n, long long samples, const float* th, const int* nb, int* hist,
                     int max_bins, cudaStream_t s);
// Counter layout of the histogram kernel: -1 = chosen per launch (default); 0..4 = 2^mode 32-bit copies per bin;
// 5 = lane-owned 16-bit counters.  A tuning control for measurements; every layout gives the same counts.
void histogram_set_mode(int mode);
int kl_raw_histogram_launch(const float* x, long long n, float width, int bins, int* hist, cudaStream_t s);
int fold_launch(const int* in, long long n_in, int* out, long long n_out, cudaStream_t s);
// thresholds[t] for histograms hist_all[offsets[t] .. offsets[t+1]); kl_dev (optional) gets 1024 floats per tensor
int kld_launch(const int* hist_all, const long long* offsets_dev, const float* widths_dev, int tensors, int dst_bins,
               long long max_bins, float* thresholds_dev, float* kl_dev, cudaStream_t s);

}  // namespace b200q
