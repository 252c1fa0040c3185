// Problem description of the INT8 (implicit) GEMM kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "requant.cuh"

namespace b200q {

enum { IGEMM_OUT_ROWMAJOR = 0, IGEMM_OUT_NCHW = 1, IGEMM_OUT_NHWC_BORDERED = 2, IGEMM_OUT_NHWC = 3 };  // NHWC: interior pixels only, [N][out_h][out_w][ldc]
enum { IGEMM_KIND_I8 = 0, IGEMM_KIND_BF16 = 1, IGEMM_KIND_F16 = 2 };  // operand type; BF16 / F16: fp32 accumulate, row-major output of the operand type

// What the host asks for.  A is [rows][k_per_tap] (row pitch a_pitch bytes): the GEMM's left matrix, or the
// pixels of a zero-bordered NHWC image flattened to rows.  B is [n][taps_h*taps_w*k_per_tap] (K-major weights).
struct IGemmProblem {
  const void* a;
  const void* b;
  int a_unsigned, b_unsigned;
  long long a_pitch, b_pitch;
  int rows, n, k_per_tap;
  int taps_h, taps_w, pad_top, pad_left;  // 1,1,0,0 for a plain GEMM
  int tap_step_w;                         // rows between horizontally adjacent taps (0 or 1: one pixel; 2: paired taps)
  int row_pitch;                          // Wp: rows per image line (convolution)
  int img_rows;                           // Hp*Wp: rows per image (convolution)
  int border_h, border_w;                 // zero border of the A image
  int out_h, out_w;                       // interior size = output H, W
  int out_mode;                           // IGEMM_OUT_*
  long long ldc;                          // elements per output row (ROWMAJOR / NHWC_BORDERED)
  void* out;
  int kind;                               // IGEMM_KIND_*; for BF16 k_per_tap and the pitches are in BYTES (2 per element)
  const float* bias_f32;                  // BF16 kind: optional per-column bias
  int dependent_launch;                   // launch as a programmatic dependent of the previous kernel in the stream
  // Fused residual Add (tpu.Add of this product's 8-bit output with another 8-bit tensor of the same shape and
  // layout, Add.cpp:177-207): out = clamp(((v*m_self + 2^(s_self-1)) >> s_self) + ((r*m_res + 2^(s_res-1)) >> s_res),
  // lo, hi) where v is the product's own requantised and saturated output, which is then not stored.  res == nullptr:
  // no fusion.  |m| < 2^23 and shifts in [1,31] (everything fits 32 bits).
  const void* res;
  int res_unsigned;
  int add_m_self, add_s_self, add_m_res, add_s_res, add_lo, add_hi;
  int per_row_params;                     // the epilogue's per-channel arrays index the GEMM's ROWS (transposed product);
                                          // 8-bit kinds with a fast dialect, n > 128
};

// Kernel argument block (device view of the same problem).
struct IGemmArgs {
  int rows, n, num_kb, kb_per_tap, taps_w, tap_step_w, tap_org_h, tap_org_w, row_pitch;
  int out_mode, img_rows, border_h, border_w, out_h, out_w;
  long long ldc;
  void* out;
  Epilogue epi;
  int* status;
  uint32_t idesc;
  int num_m_tiles, num_n_tiles;
  const float* bias_f32;
  int bf16;   // 16-bit float operands (kind::f16); with f16 set they and the output are IEEE half, else bf16
  int f16;
  int acc_small;
  int out_small;
  int floor_pre, sat_lo2, sat_hi, pack_sat, floor_needed;  // epilogue constants derived from epi (see the kernel)
  int dependent_launch;
  int acc_bound;  // |accumulator| <= this for every 8-bit operand pair (valid when acc_small)
  unsigned long long wait_budget_ns;  // every mbarrier wait of the kernel gives up after this long
  const uint8_t* res;                 // fused residual Add (see IGemmProblem); nullptr = none
  int res_unsigned, add_m_self, add_s_self, add_m_res, add_s_res, add_lo, add_hi;
  int band_m;                         // row tiles per band of the tile walk (<= 1: row-major over the column tiles)
  int expect_extra;                   // test aid: bytes added to what a stage's barrier expects (0 in normal use)
};

int make_tmap_u8(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                 const uint32_t* box);
int igemm_i8_tcgen05_supported(const IGemmProblem& p, const char** why);
int igemm_i8_tcgen05_launch(const IGemmProblem& p, const Epilogue& epi, int* status, cudaStream_t stream);
void igemm_set_wait_test(int extra_tx_bytes, long long budget_ns);
// Plain CUDA-core kernel for shapes the tensor-core path does not take (odd K, strides, groups, dilation).
struct ConvGeometry {
  int n, ic, ih, iw, oc, oh, ow, kh, kw, sh, sw, dh, dw, pht, pwl, groups, pad_value;
};
int conv2d_i8_direct_launch(const void* x_nchw, int x_unsigned, const int8_t* w_oihw, const ConvGeometry& g,
                            const Epilogue& epi, void* y_nchw, cudaStream_t stream);
int gemm_i8_direct_launch(const void* a, int a_unsigned, const void* b, int b_unsigned, int b_is_nk, int m, int n,
                          int k, int input_zp, int right_zp, const Epilogue& epi, void* out, cudaStream_t stream);

}  // namespace b200q
