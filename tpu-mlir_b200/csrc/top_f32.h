// fp32 Top-dialect forward kernels (top_f32.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200q {

struct TopConvPlan {
  int n, ic, ih, iw, oc, oh, ow, kh, kw, sh, sw, dh, dw, pht, pwl, groups;
  int icg, ocg;   // channels per group
  int K;          // icg * kh * kw
  int do_relu;
  float relu_limit;
  int splits;       // K splits (1 = none); set by the caller from top_conv_splits, needs the workspace
  int k_per_split;  // filled by top_conv_launch
};

// One-time: OIHW weight -> [groups][K][ocg], and the per-k gather table (K entries).
int top_conv_prepare(const TopConvPlan& p, const float* w_oihw, float* wt, int2* ktab, cudaStream_t s);
// y[n][oc][oh][ow] = relu(conv(x[n][ic][ih][iw]) + bias); wt / ktab from top_conv_prepare.  A matrix product
// y[M][N] = x[M][K] * w[K][N] is the case ih = iw = kh = kw = 1 with wt = w and ktab = null.
// p.splits > 1: `workspace` holds p.splits x (n * oc * oh * ow) floats; every split writes its partial sums there and a
// second kernel adds them in split order (deterministic) with the bias and the ReLU.
int top_conv_launch(const TopConvPlan& p, const float* x, const float* wt, const int2* ktab, const float* bias, float* y,
                    float* workspace, cudaStream_t s);
int top_conv_splits(const TopConvPlan& p, int sms);
int top_pool2d_launch(const float* x, float* y, long long nc, int ih, int iw, int oh, int ow, int kh, int kw, int sh, int sw,
                      int pht, int phb, int pwl, int pwr, bool is_max, bool count_include_pad, bool do_relu, float relu_limit,
                      cudaStream_t s);
// y = relu(a + b); b may be null (plain ReLU)
int top_add_launch(const float* a, const float* b, float* y, long long n, bool do_relu, float relu_limit, cudaStream_t s);

// elementwise float ops (same numbering as b200q_top_eltwise_op in the C header)
enum { TOP_ADD_CONST = 0, TOP_SUB_CONST, TOP_RSUB_CONST, TOP_MUL_CONST, TOP_MAX_CONST, TOP_MIN_CONST, TOP_MUL, TOP_SUB, TOP_RSUB,
       TOP_DIV, TOP_RDIV, TOP_SIGMOID, TOP_LOG_SIGMOID, TOP_SILU, TOP_GELU, TOP_FLOOR, TOP_ELTWISE_OPS };
int top_eltwise_launch(int op, const float* a, const float* b, double c, float* y, long long n, bool do_relu, float relu_limit,
                       cudaStream_t s);
// tpu::ActiveOp on float tensors; `mode` is the dialect's ActiveMode number, c0 / c1 its coeffs
int top_active_launch(int mode, const float* x, double c0, double c1, float* y, long long n, cudaStream_t s);
int top_scale_launch(const float* x, const float* scale, const float* bias, float* y, long long outer, int channels, long long inner,
                     bool do_relu, float relu_limit, cudaStream_t s);
enum { TOP_REDUCE_MEAN = 0, TOP_REDUCE_SUM, TOP_REDUCE_MAX, TOP_REDUCE_MIN, TOP_REDUCE_PROD, TOP_REDUCE_L2, TOP_REDUCE_L1, TOP_REDUCE_MEAN_RCP,
       TOP_REDUCE_MODES };
int top_reduce_launch(int mode, const float* x, float* y, long long outer, int axis, long long inner, cudaStream_t s);
// softmax over the middle dimension of [outer, channels, inner]; layer normalisation of rows of `inner` values
int top_softmax_launch(const float* x, float* y, long long outer, int channels, long long inner, bool log_form, cudaStream_t s);
int top_layernorm_launch(const float* x, const float* w, const float* b, float* y, long long outer, long long inner, float eps,
                         cudaStream_t s);
constexpr int TOP_REMAP_DIMS = 6;
struct TopRemap {   // layout-compatible with b200q_remap_desc
  long long dims[TOP_REMAP_DIMS], src_stride[TOP_REMAP_DIMS], mul[TOP_REMAP_DIMS], div[TOP_REMAP_DIMS], mod[TOP_REMAP_DIMS],
      off[TOP_REMAP_DIMS], extent[TOP_REMAP_DIMS], dst_stride[TOP_REMAP_DIMS];
  long long dst_offset;
};
int top_interp_launch(const float* x, float* y, long long nc, int ih, int iw, int oh, int ow, int mode, int coord_mode, int platform,
                      cudaStream_t s);
int top_grid_sampler_launch(const float* x, const float* grid, float* y, int N, int C, int IH, int IW, int OH, int OW, int mode, int padding,
                            bool align_corners, cudaStream_t s);
int top_arg_launch(const float* x, long long outer, int axis, long long inner, bool is_max, bool select_last, void* idx_out,
                   bool idx_is_float, float* val_out, cudaStream_t s);
int top_cast_launch(const float* x, long long n, int to_dt, int rmode, int out_dt, void* out, cudaStream_t s);
int top_gather_launch(const void* src, int elem_bytes, const void* indices, bool index_is_float, void* dst, long long outer,
                      long long axis_dim, long long num_indices, long long inner, cudaStream_t s);
int top_gather_elements_launch(const void* src, int elem_bytes, const void* indices, bool index_is_float, void* dst, int ndim,
                               const long long* src_shape, const long long* idx_shape, int axis, cudaStream_t s);
int top_remap_launch(const void* src, void* dst, int elem_bytes, const TopRemap& m, const void* pad_value, cudaStream_t s);

// y = clip(rint(x * 127 / threshold), -128, 127) * threshold / 127
int top_fake_quant_launch(const float* x, float* y, long long n, double threshold, cudaStream_t s);
// sums5 (device, accumulated into): sum (ref - x)^2, sum |ref|, sum x * ref, sum x^2, sum ref^2
int top_distance_launch(const float* x, const float* ref, long long n, double* sums5, cudaStream_t s);

}  // namespace b200q
