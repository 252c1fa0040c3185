// C ABI of the fp32 Top-dialect forward: the ops a calibration pass runs on the float graph.  A convolution handle
// keeps the transposed weight and the gather table; the other ops are stateless device calls.  The operator face of
// the convolution takes HOST float buffers like top::ConvOp::inference (lib/Dialect/Top/Interfaces/Conv.cpp:222-231).
#include <string.h>

#include <new>

#include "../../include/b200q.h"
#include "devbuf.h"
#include "internal.h"
#include "top_f32.h"

using namespace b200q;

namespace {

struct TopConvHandle {
  TopConvPlan plan{};
  DevBuf wt, ktab, bias, w_stage, x, y, ws;
  bool with_bias = false;
  const float* d_bias = nullptr;   // device face: the caller's
};

int make_plan(const b200q_top_conv_desc& d, TopConvPlan* out) {
  if (d.n < 0 || d.ic < 1 || d.ih < 1 || d.iw < 1 || d.oc < 1 || d.kh < 1 || d.kw < 1 || d.sh < 1 || d.sw < 1 || d.dh < 1 ||
      d.dw < 1 || d.groups < 1 || d.pht < 0 || d.phb < 0 || d.pwl < 0 || d.pwr < 0)
    return set_error(B200Q_ERR_INVALID, "top conv: bad attribute");
  if (d.ic % d.groups != 0 || d.oc % d.groups != 0) return set_error(B200Q_ERR_INVALID, "top conv: channels must divide into the groups");
  const int64_t oh = (d.ih + d.pht + d.phb - d.dh * (d.kh - 1) - 1) / d.sh + 1;
  const int64_t ow = (d.iw + d.pwl + d.pwr - d.dw * (d.kw - 1) - 1) / d.sw + 1;
  if (oh < 1 || ow < 1) return set_error(B200Q_ERR_INVALID, "top conv: empty output");
  const int64_t K = d.ic / d.groups * d.kh * d.kw;
  if (d.ic * d.ih * d.iw > 0x7fffffffLL || K > 0x7fffffffLL || d.oc > 0x7fffffffLL || d.n > 0x7fffffffLL || (d.kh - 1) * d.dh > 0x7fff ||
      (d.kw - 1) * d.dw > 0x7fff || d.groups > 65535)
    return set_error(B200Q_ERR_UNSUPPORTED, "top conv: shape out of the kernel's index range");
  TopConvPlan p{};
  p.n = (int)d.n; p.ic = (int)d.ic; p.ih = (int)d.ih; p.iw = (int)d.iw; p.oc = (int)d.oc; p.oh = (int)oh; p.ow = (int)ow;
  p.kh = (int)d.kh; p.kw = (int)d.kw; p.sh = (int)d.sh; p.sw = (int)d.sw; p.dh = (int)d.dh; p.dw = (int)d.dw;
  p.pht = (int)d.pht; p.pwl = (int)d.pwl; p.groups = (int)d.groups;
  p.icg = p.ic / p.groups; p.ocg = p.oc / p.groups; p.K = (int)K;
  p.do_relu = d.do_relu ? 1 : 0;
  p.relu_limit = d.relu_limit;
  p.splits = 1;
  *out = p;
  return B200Q_OK;
}

}  // namespace

extern "C" {

int b200q_top_conv2d_dev_create(const b200q_top_conv_desc* desc, const float* filter_oihw, const float* bias, void** handle) {
  if (!desc || !filter_oihw || !handle) return set_error(B200Q_ERR_INVALID, "top_conv2d_dev_create: null argument");
  if (desc->with_bias && !bias) return set_error(B200Q_ERR_INVALID, "top_conv2d_dev_create: with_bias but no bias");
  TopConvPlan p;
  B200Q_TRY(make_plan(*desc, &p));
  auto* h = new (std::nothrow) TopConvHandle();
  if (!h) return set_error(B200Q_ERR_NOMEM, "top_conv2d_dev_create: out of host memory");
  h->plan = p;
  h->with_bias = desc->with_bias != 0;
  h->d_bias = h->with_bias ? bias : nullptr;
  int rc = h->wt.ensure((size_t)p.oc * p.K * 4);
  if (rc == B200Q_OK) rc = h->ktab.ensure((size_t)p.K * sizeof(int2));
  if (rc == B200Q_OK) rc = top_conv_prepare(p, filter_oihw, h->wt.as<float>(), h->ktab.as<int2>(), 0);
  if (rc == B200Q_OK && cudaStreamSynchronize(0) != cudaSuccess) rc = cuda_error(cudaGetLastError(), "sync", __FILE__, __LINE__);
  if (rc != B200Q_OK) {
    delete h;
    return rc;
  }
  *handle = h;
  return B200Q_OK;
}

int b200q_top_conv2d_dev_run(void* handle, const float* x, float* y, int64_t batch, void* stream) {
  if (!handle || !x || !y || batch < 0 || batch > 0x7fffffffLL) return set_error(B200Q_ERR_INVALID, "top_conv2d_dev_run: bad argument");
  TopConvHandle* h = static_cast<TopConvHandle*>(handle);
  TopConvPlan p = h->plan;
  p.n = (int)batch;
  int dev = 0, sms = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  p.splits = top_conv_splits(p, sms);
  if (p.splits > 1) B200Q_TRY(h->ws.ensure((size_t)p.splits * p.n * p.oc * p.oh * p.ow * 4));   // grows on the first call of a batch size
  return top_conv_launch(p, x, h->wt.as<float>(), h->ktab.as<int2>(), h->d_bias, y, h->ws.as<float>(), static_cast<cudaStream_t>(stream));
}

void b200q_top_conv2d_dev_output_shape(void* handle, int64_t* oh, int64_t* ow) {
  if (!handle) return;
  TopConvHandle* h = static_cast<TopConvHandle*>(handle);
  if (oh) *oh = h->plan.oh;
  if (ow) *ow = h->plan.ow;
}

void b200q_top_conv2d_dev_destroy(void** handle) {
  if (!handle || !*handle) return;
  delete static_cast<TopConvHandle*>(*handle);
  *handle = nullptr;
}

int b200q_top_conv2d_inference(const b200q_top_conv_desc* desc, float* const* inputs, int n_inputs, float* const* outputs,
                               int n_outputs) {
  if (!desc || !inputs || !outputs || n_inputs < 2 || n_outputs < 1 || !inputs[0] || !inputs[1] || !outputs[0])
    return set_error(B200Q_ERR_INVALID, "top_conv2d_inference: null argument");
  const float* bias_h = (desc->with_bias && n_inputs > 2) ? inputs[2] : nullptr;
  if (desc->with_bias && !bias_h) return set_error(B200Q_ERR_INVALID, "top_conv2d_inference: with_bias but inputs[2] is null");
  TopConvPlan p;
  B200Q_TRY(make_plan(*desc, &p));
  TopConvHandle h;
  cudaStream_t s = 0;
  const size_t w_bytes = (size_t)p.oc * p.K * 4, x_bytes = (size_t)p.n * p.ic * p.ih * p.iw * 4,
               y_bytes = (size_t)p.n * p.oc * p.oh * p.ow * 4;
  int rc = B200Q_OK;
  do {
    if ((rc = h.w_stage.upload(inputs[1], w_bytes, s))) break;
    if (bias_h && (rc = h.bias.upload(bias_h, (size_t)p.oc * 4, s))) break;
    if ((rc = h.wt.ensure(w_bytes))) break;
    if ((rc = h.ktab.ensure((size_t)p.K * sizeof(int2)))) break;
    if ((rc = top_conv_prepare(p, h.w_stage.as<float>(), h.wt.as<float>(), h.ktab.as<int2>(), s))) break;
    if (x_bytes == 0 || y_bytes == 0) break;
    if ((rc = h.x.upload(inputs[0], x_bytes, s))) break;
    if ((rc = h.y.ensure(y_bytes))) break;
    if ((rc = top_conv_launch(p, h.x.as<float>(), h.wt.as<float>(), h.ktab.as<int2>(), bias_h ? h.bias.as<float>() : nullptr,
                              h.y.as<float>(), nullptr, s))) break;
    if (cudaMemcpyAsync(outputs[0], h.y.p, y_bytes, cudaMemcpyDeviceToHost, s) != cudaSuccess) { rc = cuda_error(cudaGetLastError(), "D2H output", __FILE__, __LINE__); break; }
    if (cudaStreamSynchronize(s) != cudaSuccess) { rc = cuda_error(cudaGetLastError(), "sync", __FILE__, __LINE__); break; }
  } while (0);
  if (rc != B200Q_OK) cudaStreamSynchronize(s);
  return rc;
}

int b200q_top_matmul_f32_dev(const float* x, const float* w_kn, const float* bias, float* y, int64_t M, int64_t K, int64_t N,
                             int32_t do_relu, float relu_limit, void* stream) {
  if (!x || !w_kn || !y) return set_error(B200Q_ERR_INVALID, "top_matmul_f32_dev: null argument");
  if (M < 0 || K < 1 || N < 1 || M > 0x7fffffffLL || K > 0x7fffffffLL || N > 0x7fffffffLL) return set_error(B200Q_ERR_INVALID, "top_matmul_f32_dev: bad shape");
  // x[M][K] * w[K][N]: a 1x1 convolution over M one-pixel images; without a table the gather offset of k is k itself
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TopConvPlan p{};
  p.n = (int)M; p.ic = (int)K; p.ih = p.iw = p.oh = p.ow = 1; p.oc = (int)N; p.kh = p.kw = p.sh = p.sw = p.dh = p.dw = 1;
  p.groups = 1; p.icg = (int)K; p.ocg = (int)N; p.K = (int)K; p.do_relu = do_relu ? 1 : 0; p.relu_limit = relu_limit;
  return top_conv_launch(p, x, w_kn, nullptr, bias, y, nullptr, s);
}

int b200q_top_pool2d_f32_dev(const float* x, float* y, int64_t nc, int32_t ih, int32_t iw, int32_t kh, int32_t kw, int32_t sh,
                             int32_t sw, int32_t pht, int32_t phb, int32_t pwl, int32_t pwr, int32_t is_max,
                             int32_t count_include_pad, int32_t do_relu, float relu_limit, void* stream) {
  if (!x || !y) return set_error(B200Q_ERR_INVALID, "top_pool2d_f32_dev: null argument");
  if (nc < 0 || ih < 1 || iw < 1 || kh < 1 || kw < 1 || sh < 1 || sw < 1 || pht < 0 || phb < 0 || pwl < 0 || pwr < 0)
    return set_error(B200Q_ERR_INVALID, "top_pool2d_f32_dev: bad attribute");
  const int oh = (ih + pht + phb - kh) / sh + 1, ow = (iw + pwl + pwr - kw) / sw + 1;
  if (oh < 1 || ow < 1) return set_error(B200Q_ERR_INVALID, "top_pool2d_f32_dev: empty output");
  return top_pool2d_launch(x, y, nc, ih, iw, oh, ow, kh, kw, sh, sw, pht, phb, pwl, pwr, is_max != 0, count_include_pad != 0,
                           do_relu != 0, relu_limit, static_cast<cudaStream_t>(stream));
}

int b200q_top_add_f32_dev(const float* a, const float* b, float* y, int64_t count, int32_t do_relu, float relu_limit, void* stream) {
  if (!a || !b || !y || count < 0) return set_error(B200Q_ERR_INVALID, "top_add_f32_dev: bad argument");
  return top_add_launch(a, b, y, count, do_relu != 0, relu_limit, static_cast<cudaStream_t>(stream));
}

int b200q_top_relu_f32_dev(const float* x, float* y, int64_t count, float relu_limit, void* stream) {
  if (!x || !y || count < 0) return set_error(B200Q_ERR_INVALID, "top_relu_f32_dev: bad argument");
  return top_add_launch(x, nullptr, y, count, true, relu_limit, static_cast<cudaStream_t>(stream));
}

int b200q_top_eltwise_f32_dev(int32_t op, const float* a, const float* b, double const_val, float* y, int64_t count, int32_t do_relu,
                              float relu_limit, void* stream) {
  if (!a || !y || count < 0) return set_error(B200Q_ERR_INVALID, "top_eltwise_f32_dev: bad argument");
  return top_eltwise_launch(op, a, b, const_val, y, count, do_relu != 0, relu_limit, static_cast<cudaStream_t>(stream));
}

int b200q_active_f32_dev(int32_t mode, const float* x, double coeff0, double coeff1, float* y, int64_t count, void* stream) {
  if (!x || !y || count < 0) return set_error(B200Q_ERR_INVALID, "active_f32_dev: bad argument");
  return top_active_launch(mode, x, coeff0, coeff1, y, count, static_cast<cudaStream_t>(stream));
}

int b200q_top_scale_f32_dev(const float* x, const float* scale, const float* bias, float* y, int64_t outer, int32_t channels,
                            int64_t inner, int32_t do_relu, float relu_limit, void* stream) {
  if (!x || !scale || !y || outer < 0 || channels < 1 || inner < 1) return set_error(B200Q_ERR_INVALID, "top_scale_f32_dev: bad argument");
  return top_scale_launch(x, scale, bias, y, outer, channels, inner, do_relu != 0, relu_limit, static_cast<cudaStream_t>(stream));
}

int b200q_top_reduce_f32_dev(int32_t mode, const float* x, float* y, int64_t outer, int32_t axis, int64_t inner, void* stream) {
  if (!x || !y || outer < 0 || inner < 0) return set_error(B200Q_ERR_INVALID, "top_reduce_f32_dev: bad argument");
  return top_reduce_launch(mode, x, y, outer, axis, inner, static_cast<cudaStream_t>(stream));
}

int b200q_top_softmax_f32_dev(const float* x, float* y, int64_t outer, int32_t channels, int64_t inner, int32_t log_form, void* stream) {
  if (!x || !y || outer < 0 || channels < 0 || inner < 1) return set_error(B200Q_ERR_INVALID, "top_softmax_f32_dev: bad argument");
  return top_softmax_launch(x, y, outer, channels, inner, log_form != 0, static_cast<cudaStream_t>(stream));
}

int b200q_top_layernorm_f32_dev(const float* x, const float* weight, const float* bias, float* y, int64_t outer, int64_t inner, float eps,
                                void* stream) {
  if (!x || !y || outer < 0 || inner < 0) return set_error(B200Q_ERR_INVALID, "top_layernorm_f32_dev: bad argument");
  return top_layernorm_launch(x, weight, bias, y, outer, inner, eps, static_cast<cudaStream_t>(stream));
}

int b200q_interp_f32_dev(const float* x, float* y, int64_t nc, int32_t ih, int32_t iw, int32_t oh, int32_t ow, int32_t mode, int32_t coord_mode,
                         int32_t platform, void* stream) {
  if (!x || !y || nc < 0 || ih < 1 || iw < 1 || oh < 0 || ow < 0) return set_error(B200Q_ERR_INVALID, "interp_f32_dev: bad argument");
  return top_interp_launch(x, y, nc, ih, iw, oh, ow, mode, coord_mode, platform, static_cast<cudaStream_t>(stream));
}

int b200q_grid_sampler_f32_dev(const float* x, const float* grid, float* y, int32_t n, int32_t c, int32_t ih, int32_t iw, int32_t oh, int32_t ow,
                               int32_t mode, int32_t padding_mode, int32_t align_corners, void* stream) {
  if (!x || !grid || !y || n < 0 || c < 0 || ih < 1 || iw < 1 || oh < 0 || ow < 0) return set_error(B200Q_ERR_INVALID, "grid_sampler_f32_dev: bad argument");
  return top_grid_sampler_launch(x, grid, y, n, c, ih, iw, oh, ow, mode, padding_mode, align_corners != 0, static_cast<cudaStream_t>(stream));
}

int b200q_arg_f32_dev(const float* x, int64_t outer, int32_t axis, int64_t inner, int32_t is_max, int32_t select_last_index, void* indices,
                      int32_t index_is_float, float* values, void* stream) {
  if (!x || !indices || outer < 0 || axis < 1 || inner < 1) return set_error(B200Q_ERR_INVALID, "arg_f32_dev: bad argument");
  return top_arg_launch(x, outer, axis, inner, is_max != 0, select_last_index != 0, indices, index_is_float != 0, values,
                        static_cast<cudaStream_t>(stream));
}

int b200q_top_cast_f32_dev(const float* x, int64_t count, int32_t to_dtype, int32_t round_mode, int32_t out_dtype, void* out, void* stream) {
  if (!x || !out || count < 0) return set_error(B200Q_ERR_INVALID, "top_cast_f32_dev: bad argument");
  if (to_dtype < B200Q_DT_I8 || to_dtype > B200Q_DT_F32 || (out_dtype != B200Q_DT_F32 && out_dtype != to_dtype))
    return set_error(B200Q_ERR_INVALID, "top_cast_f32_dev: the output is stored as float or in the target type");
  return top_cast_launch(x, count, to_dtype, round_mode, out_dtype, out, static_cast<cudaStream_t>(stream));
}

int b200q_gather_dev(const void* src, int32_t elem_bytes, const void* indices, int32_t index_is_float, void* dst, int64_t outer,
                     int64_t axis_dim, int64_t num_indices, int64_t inner, void* stream) {
  if (!src || !indices || !dst || outer < 0 || axis_dim < 1 || num_indices < 0 || inner < 0)
    return set_error(B200Q_ERR_INVALID, "gather_dev: bad argument");
  return top_gather_launch(src, elem_bytes, indices, index_is_float != 0, dst, outer, axis_dim, num_indices, inner,
                           static_cast<cudaStream_t>(stream));
}

int b200q_gather_elements_dev(const void* src, int32_t elem_bytes, const void* indices, int32_t index_is_float, void* dst, int32_t ndim,
                              const int64_t* src_shape, const int64_t* indices_shape, int32_t axis, void* stream) {
  if (!src || !indices || !dst || !src_shape || !indices_shape) return set_error(B200Q_ERR_INVALID, "gather_elements_dev: bad argument");
  long long ss[8], is[8];
  if (ndim < 1 || ndim > 8) return set_error(B200Q_ERR_INVALID, "gather_elements_dev: rank %d", ndim);
  for (int i = 0; i < ndim; ++i) {
    ss[i] = src_shape[i];
    is[i] = indices_shape[i];
    if (ss[i] < 1 || is[i] < 0) return set_error(B200Q_ERR_INVALID, "gather_elements_dev: bad shape");
  }
  return top_gather_elements_launch(src, elem_bytes, indices, index_is_float != 0, dst, ndim, ss, is, axis, static_cast<cudaStream_t>(stream));
}

int b200q_remap_dev(const void* src, void* dst, int32_t elem_bytes, const b200q_remap_desc* desc, const void* pad_value, void* stream) {
  if (!src || !dst || !desc) return set_error(B200Q_ERR_INVALID, "remap_dev: null argument");
  static_assert(sizeof(b200q_remap_desc) == sizeof(TopRemap), "the two descriptors must stay layout-compatible");
  TopRemap m;
  memcpy(&m, desc, sizeof(m));
  return top_remap_launch(src, dst, elem_bytes, m, pad_value, static_cast<cudaStream_t>(stream));
}

int b200q_top_fake_quant_f32_dev(const float* x, float* y, int64_t count, double threshold, void* stream) {
  if (!x || !y || count < 0) return set_error(B200Q_ERR_INVALID, "top_fake_quant_f32_dev: bad argument");
  return top_fake_quant_launch(x, y, count, threshold, static_cast<cudaStream_t>(stream));
}

int b200q_top_distance_f32_dev(const float* x, const float* ref, int64_t count, double* sums5, void* stream) {
  if (!x || !ref || !sums5 || count < 0) return set_error(B200Q_ERR_INVALID, "top_distance_f32_dev: bad argument");
  return top_distance_launch(x, ref, count, sums5, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
