// C ABI for tpu.MatMul and tpu.Conv2D (INT8): the operator face over host float buffers and the device
// face over native device tensors.  The host side here mirrors what tpu::MatMulOp / tpu::Conv2DOp do around
// their oneDNN calls: resolve the op attributes to one requantisation form, keep the weights resident, pick
// the kernel, and convert between the interpreter's float storage and native integers.
#include <cmath>
#include <cstring>
#include <new>
#include <vector>

#include "devbuf.h"
#include "eltwise.h"
#include "igemm.h"
#include "internal.h"
#include "layout.h"
#include "top_f32.h"

namespace b200q {
namespace {

inline bool is_q8(int dt) { return dt == B200Q_DT_I8 || dt == B200Q_DT_U8; }
inline size_t dtype_size(int dt) {
  switch (dt) {
    case B200Q_DT_I8:
    case B200Q_DT_U8: return 1;
    case B200Q_DT_I16:
    case B200Q_DT_U16:
    case B200Q_DT_BF16:
    case B200Q_DT_F16: return 2;
    default: return 4;
  }
}

int check_int32(const int64_t* v, int n, const char* what) {
  for (int i = 0; i < n; ++i)
    if (v[i] > 2147483647ll || v[i] < -2147483648ll)
      return set_error(B200Q_ERR_UNSUPPORTED, "%s[%d] = %lld does not fit int32", what, i, (long long)v[i]);
  return B200Q_OK;
}

// Host description of a resolved requantisation; uploaded into an Epilogue with device arrays.
struct ResolvedRequant {
  int dialect = B200Q_RQ_NONE, round_mode = B200Q_ROUND_HALF_UP, per_channel = 0, out_zp = 0, relu = B200Q_RELU_NONE;
  int out_dtype = B200Q_DT_I8;
  float scale = 0.f;
  std::vector<int32_t> multiplier, shift;
};

int make_epilogue(const ResolvedRequant& r, const int32_t* d_bias, DevBuf& d_mult, DevBuf& d_shift, cudaStream_t s,
                  Epilogue* e) {
  e->dialect = r.dialect;
  e->round_mode = r.round_mode;
  e->per_channel = r.per_channel;
  e->out_zp = r.out_zp;
  e->relu = r.relu;
  e->out_dtype = r.out_dtype;
  e->scale = r.scale;
  e->bias = d_bias;
  e->multiplier = nullptr;
  e->shift = nullptr;
  if (!r.multiplier.empty()) {
    B200Q_TRY(d_mult.upload(r.multiplier.data(), r.multiplier.size() * 4, s));
    e->multiplier = d_mult.as<int32_t>();
  }
  if (!r.shift.empty()) {
    B200Q_TRY(d_shift.upload(r.shift.data(), r.shift.size() * 4, s));
    e->shift = d_shift.as<int32_t>();
  }
  return B200Q_OK;
}

int read_status(DevBuf& d_status, cudaStream_t s, const char* what) {
  int h = 0;
  CUDA_TRY(cudaMemcpyAsync(&h, d_status.p, 4, cudaMemcpyDeviceToHost, s));
  CUDA_TRY(cudaStreamSynchronize(s));
  if (h != 0) {
    cudaMemsetAsync(d_status.p, 0, 4, s);
    return set_error(B200Q_ERR_TIMEOUT, "%s: a bounded wait inside the kernel ran out (wait site %d)", what, h);
  }
  return B200Q_OK;
}

// ---------------------------------------------------------------------------------------------- MatMul
// Which requantisation a tpu.MatMul resolves to: MatMul.cpp:636-728 (one entry per batch on CV18xx).
int resolve_matmul(const b200q_matmul_desc& d, const float* multi_operand, int batch_index, ResolvedRequant* r) {
  r->out_dtype = d.out_dtype;
  r->relu = d.do_relu ? B200Q_RELU_BEFORE_REQUANT : B200Q_RELU_NONE;
  if (d.out_dtype == B200Q_DT_I32 && d.n_quant == 0) {
    r->dialect = B200Q_RQ_NONE;
    return B200Q_OK;
  }
  if (d.out_dtype >= B200Q_DT_F32) return set_error(B200Q_ERR_UNSUPPORTED, "matmul: float output types are not handled by the INT8 path");
  const int qm = d.quant_mode;
  if (qm == B200Q_QM_ONLY_SCALE && !d.is_cv18xx) {
    if (d.fuse_rq) return set_error(B200Q_ERR_UNSUPPORTED, "matmul: OnlyScale with fuse_rq (asserted off in the reference)");
    r->dialect = B200Q_RQ_ONLY_SCALE;
    r->scale = (float)d.out_scale;
    r->out_zp = d.out_zp;
    return B200Q_OK;
  }
  if (d.n_quant < 1 || !d.multipliers || !d.rshifts) return set_error(B200Q_ERR_INVALID, "matmul: multipliers/rshifts missing");
  B200Q_TRY(check_int32(d.multipliers, d.n_quant, "multipliers"));
  B200Q_TRY(check_int32(d.rshifts, d.n_quant, "rshifts"));
  if (d.is_cv18xx) {  // :638-664, applyMultiplierAndRShift(.., qmode, HALF_AWAY) with isCV18xx()
    const int bi = batch_index < d.n_quant ? batch_index : 0;
    r->round_mode = B200Q_ROUND_HALF_AWAY_FROM_ZERO;
    r->out_zp = 0;
    r->multiplier.assign(1, (int32_t)d.multipliers[bi]);
    const int32_t rs = (int32_t)d.rshifts[bi];
    switch (qm) {
      case B200Q_QM_MULTIPLIER_SHIFT:
        if (rs < 0 || rs > 30) return set_error(B200Q_ERR_INVALID, "matmul: cv18xx rshift %d outside [0,30]", rs);
        r->dialect = B200Q_RQ_MULTIPLIER_SHIFT_F32;
        r->shift.assign(1, rs);
        break;
      case B200Q_QM_ONLY_SHIFT: r->dialect = B200Q_RQ_ONLY_SHIFT; r->shift.assign(1, rs); break;
      case B200Q_QM_QDM:
      case B200Q_QM_TFLITE:
      case B200Q_QM_TFLITE_LSHIFT: r->dialect = B200Q_RQ_QDM; r->shift.assign(1, -rs); break;
      default: return set_error(B200Q_ERR_UNSUPPORTED, "matmul: quant_mode %d on cv18xx", qm);
    }
    return B200Q_OK;
  }
  r->out_zp = d.out_zp;
  if (qm == B200Q_QM_TFLITE || qm == B200Q_QM_TFLITE_LSHIFT) {  // :696-707
    r->dialect = B200Q_RQ_QDM;
    r->round_mode = B200Q_ROUND_HALF_AWAY_FROM_ZERO;
    r->multiplier.assign(1, (int32_t)d.multipliers[0]);
    r->shift.assign(1, -(int32_t)d.rshifts[0]);
    return B200Q_OK;
  }
  if (qm == B200Q_QM_MULTIPLIER_SHIFT) {  // :708-726
    r->dialect = B200Q_RQ_MULTIPLIER_SHIFT;
    r->round_mode = B200Q_ROUND_HALF_UP;
    if (d.fuse_rq) {
      if (!multi_operand) return set_error(B200Q_ERR_INVALID, "matmul: fuse_rq needs the multi operand (inputs[3])");
      r->per_channel = 1;
      r->multiplier.resize((size_t)d.N);
      r->shift.assign((size_t)d.N, (int32_t)d.rshifts[0]);
      for (int64_t n = 0; n < d.N; ++n) {
        const int64_t m = (int64_t)multi_operand[n];  // the interpreter reads the float operand back as int64
        if (m > 2147483647ll || m < -2147483648ll) return set_error(B200Q_ERR_UNSUPPORTED, "matmul: multi[%lld] does not fit int32", (long long)n);
        r->multiplier[(size_t)n] = (int32_t)m;
      }
    } else {
      r->multiplier.assign(1, (int32_t)d.multipliers[0]);
      r->shift.assign(1, (int32_t)d.rshifts[0]);
    }
    return B200Q_OK;
  }
  return set_error(B200Q_ERR_UNSUPPORTED, "matmul: quant_mode %d leaves the output un-requantised in the reference", qm);
}

int validate_matmul(const b200q_matmul_desc& d) {
  if (d.batch < 1 || d.M < 0 || d.K < 1 || d.N < 1) return set_error(B200Q_ERR_INVALID, "matmul: bad shape");
  if (d.M * d.batch > 0x7fffffffLL || d.N > 0x7fffffffLL || d.K > 0x7fffffffLL) return set_error(B200Q_ERR_UNSUPPORTED, "matmul: dimension exceeds int32");
  if (d.hdim_is_batch) {
    if (d.batch_low < 0 || d.M * d.batch * (d.batch_low ? d.batch_low : 1) > 0x7fffffffLL) return set_error(B200Q_ERR_INVALID, "matmul: bad batch_low");
    if (!d.right_batched) return set_error(B200Q_ERR_INVALID, "matmul: hdim_is_batch goes with a batched right operand");
    if (d.is_cv18xx) return set_error(B200Q_ERR_UNSUPPORTED, "matmul: hdim_is_batch in the CV18xx form is not implemented");
  }
  if (!is_q8(d.input_dtype) || !is_q8(d.right_dtype)) return set_error(B200Q_ERR_INVALID, "matmul: operands must be int8/uint8");
  return B200Q_OK;
}

// Launch out = epilogue(A * B^T) on the best kernel.  b is [N,K].
int gemm_dispatch(const void* a, int a_dt, const void* b_nk, int b_dt, int64_t M, int64_t N, int64_t K, int input_zp,
                  int right_zp, const Epilogue& e, void* out, int* status, int algo, cudaStream_t s) {
  if (M == 0) return B200Q_OK;
  IGemmProblem p{};
  p.a = a;
  p.b = b_nk;
  p.a_unsigned = a_dt == B200Q_DT_U8;
  p.b_unsigned = b_dt == B200Q_DT_U8;
  p.a_pitch = K;
  p.b_pitch = K;
  p.rows = (int)M;
  p.n = (int)N;
  p.k_per_tap = (int)K;
  p.taps_h = p.taps_w = 1;
  p.out_mode = IGEMM_OUT_ROWMAJOR;
  p.ldc = N;
  p.out = out;
  const char* why = nullptr;
  const bool tc_ok = igemm_i8_tcgen05_supported(p, &why) && input_zp == 0 && right_zp == 0;
  if (algo == 1 && !tc_ok)
    return set_error(B200Q_ERR_UNSUPPORTED, "gemm: tensor-core path unavailable: %s", why ? why : "non-zero zero point");
  if (tc_ok && algo != 2) return igemm_i8_tcgen05_launch(p, e, status, s);
  return gemm_i8_direct_launch(a, p.a_unsigned, b_nk, p.b_unsigned, 1, (int)M, (int)N, (int)K, input_zp, right_zp, e, out, s);
}

struct MatMulHandle {
  DevBuf stage_f32, a_q8, b_f32, b_nk, bias, mult, shift, out_q, out_f32, status, perm;
  bool weights_ready = false;
  int weight_version = -1;
  const float* weight_ptr = nullptr;
};

// ---------------------------------------------------------------------------------------------- Conv2D
int resolve_conv(const b200q_conv2d_desc& d, ResolvedRequant* r) {  // Conv2D.cpp:295-341
  r->out_dtype = d.out_dtype;
  r->relu = d.do_relu ? B200Q_RELU_AFTER_REQUANT : B200Q_RELU_NONE;
  r->out_zp = d.out_zp;
  if (d.out_dtype >= B200Q_DT_F32) return set_error(B200Q_ERR_UNSUPPORTED, "conv2d: float output types are not handled by the INT8 path");
  if (d.n_quant < 1 || !d.rshifts) return set_error(B200Q_ERR_INVALID, "conv2d: rshift attribute missing");
  if (d.n_quant != 1 && d.n_quant != d.oc) return set_error(B200Q_ERR_INVALID, "conv2d: n_quant must be 1 or oc");
  const int qm = d.quant_mode;
  r->per_channel = (d.n_quant == d.oc) ? 1 : 0;
  B200Q_TRY(check_int32(d.rshifts, d.n_quant, "rshift"));
  r->shift.resize((size_t)d.n_quant);
  r->multiplier.assign((size_t)d.n_quant, 1);
  if (qm != B200Q_QM_ONLY_SHIFT) {
    if (!d.multipliers) return set_error(B200Q_ERR_INVALID, "conv2d: multiplier attribute missing");
    B200Q_TRY(check_int32(d.multipliers, d.n_quant, "multiplier"));
    for (int i = 0; i < d.n_quant; ++i) r->multiplier[(size_t)i] = (int32_t)d.multipliers[i];
  }
  const bool is_tf = qm == B200Q_QM_QDM || qm == B200Q_QM_TFLITE || qm == B200Q_QM_TFLITE_LSHIFT;
  r->round_mode = is_tf ? B200Q_ROUND_HALF_AWAY_FROM_ZERO : B200Q_ROUND_HALF_UP;  // :312-315
  for (int i = 0; i < d.n_quant; ++i) {
    const int32_t rs = (int32_t)d.rshifts[i];
    if (qm == B200Q_QM_MULTIPLIER_SHIFT && d.is_cv18xx && (rs < 0 || rs > 30))
      return set_error(B200Q_ERR_INVALID, "conv2d: cv18xx rshift %d outside [0,30]", rs);
    r->shift[(size_t)i] = is_tf ? (d.is_cv18xx ? -rs : rs) : rs;  // MathUtils.cpp:549-556
  }
  switch (qm) {
    case B200Q_QM_MULTIPLIER_SHIFT: r->dialect = d.is_cv18xx ? B200Q_RQ_MULTIPLIER_SHIFT_F32 : B200Q_RQ_MULTIPLIER_SHIFT; break;
    case B200Q_QM_ONLY_SHIFT: r->dialect = B200Q_RQ_ONLY_SHIFT; break;
    case B200Q_QM_QDM:
    case B200Q_QM_TFLITE:
    case B200Q_QM_TFLITE_LSHIFT: r->dialect = B200Q_RQ_QDM; break;
    default: return set_error(B200Q_ERR_UNSUPPORTED, "conv2d: quant_mode %d (unreachable in the reference)", qm);
  }
  return B200Q_OK;
}

struct ConvHandle {
  b200q_conv2d_desc d{};
  ConvGeometry g{};
  bool use_tc = false;      // tensor cores on the zero-bordered image directly (stride 1, IC fits the K blocking)
  bool pair_taps = false;   // use_tc with 64 channels: adjacent taps paired into 128-byte K blocks
  bool use_im2col = false;  // tensor cores on an im2col matrix (strides, dilation, any IC)
  bool few_channels = false;  // use_im2col with the (fy, c, fx8) row order gathered straight from NCHW (a network's stem)
  int kpad = 0;             // im2col row length (KH*KW*IC rounded up to 16)
  int bh = 0, bw = 0, Hp = 0, Wp = 0;
  Epilogue epi{};
  DevBuf w_oihw, w_packed, bias, mult, shift, x_bordered, a_cols, status;
  // operator-face staging
  DevBuf x_f32, x_q8, y_q, y_f32, w_f32, bias_f32;
  // operator face: which host filter the device copy was made from (b200q_conv2d_desc::weight_version)
  int weight_version = -1;
  const float* weight_ptr = nullptr;
  // optional per-kernel timing of the device face: one event triple per run since profiling was switched on
  bool profiling = false;
  std::vector<cudaEvent_t> events;  // 3 per run: before the layout kernel, between, after the conv kernel
  size_t runs_recorded = 0;
  cudaEvent_t* ev = nullptr;        // the triple of the run being recorded
  int next_triple() {
    if (events.size() < (runs_recorded + 1) * 3) {
      for (int i = 0; i < 3; ++i) {
        cudaEvent_t e;
        CUDA_TRY(cudaEventCreate(&e));
        events.push_back(e);
      }
    }
    ev = &events[runs_recorded * 3];
    ++runs_recorded;
    return B200Q_OK;
  }
  // operator face: host copies pipelined over pieces of the batch (copy-in, compute, copy-out streams)
  cudaStream_t pipe[3] = {nullptr, nullptr, nullptr};
  std::vector<cudaEvent_t> pipe_ev;
  int ensure_pipe(int pieces) {
    for (int i = 0; i < 3; ++i)
      if (!pipe[i]) CUDA_TRY(cudaStreamCreateWithFlags(&pipe[i], cudaStreamNonBlocking));
    while ((int)pipe_ev.size() < 2 * pieces) {
      cudaEvent_t e;
      CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
      pipe_ev.push_back(e);
    }
    return B200Q_OK;
  }
  ~ConvHandle() {
    for (auto& e : events) cudaEventDestroy(e);
    for (auto& e : pipe_ev) cudaEventDestroy(e);
    for (auto& st : pipe)
      if (st) cudaStreamDestroy(st);
  }
};

int conv_out_dims(const b200q_conv2d_desc& d, int64_t* oh, int64_t* ow) {
  if (d.n < 0 || d.ic < 1 || d.ih < 1 || d.iw < 1 || d.oc < 1 || d.kh < 1 || d.kw < 1 || d.sh < 1 || d.sw < 1 ||
      d.dh < 1 || d.dw < 1 || d.groups < 1 || d.ic % d.groups || d.oc % d.groups || d.pht < 0 || d.phb < 0 ||
      d.pwl < 0 || d.pwr < 0)
    return set_error(B200Q_ERR_INVALID, "conv2d: bad geometry");
  *oh = (d.ih + d.pht + d.phb - d.dh * (d.kh - 1) - 1) / d.sh + 1;
  *ow = (d.iw + d.pwl + d.pwr - d.dw * (d.kw - 1) - 1) / d.sw + 1;
  if (*oh < 1 || *ow < 1) return set_error(B200Q_ERR_INVALID, "conv2d: empty output");
  if (!is_q8(d.input_dtype)) return set_error(B200Q_ERR_INVALID, "conv2d: input must be int8/uint8");
  return B200Q_OK;
}

// filter / bias already on the device in native types
int conv_setup(ConvHandle* h, const b200q_conv2d_desc& d, const void* w_dev, int w_is_f32, const void* bias_dev,
               int bias_is_f32, cudaStream_t s) {
  int64_t oh = 0, ow = 0;
  B200Q_TRY(conv_out_dims(d, &oh, &ow));
  h->d = d;
  h->d.multipliers = nullptr;
  h->d.rshifts = nullptr;
  ConvGeometry& g = h->g;
  g = ConvGeometry{(int)d.n, (int)d.ic, (int)d.ih, (int)d.iw, (int)d.oc, (int)oh, (int)ow, (int)d.kh, (int)d.kw,
                   (int)d.sh, (int)d.sw, (int)d.dh, (int)d.dw, (int)d.pht, (int)d.pwl, (int)d.groups, d.pad_value};
  ResolvedRequant r;
  B200Q_TRY(resolve_conv(d, &r));
  // bias -> int32 on the device
  const int32_t* d_bias = nullptr;
  if (d.with_bias) {
    if (!bias_dev) return set_error(B200Q_ERR_INVALID, "conv2d: with_bias but no bias operand");
    B200Q_TRY(h->bias.ensure((size_t)d.oc * 4));
    if (bias_is_f32) B200Q_TRY(f32_to_i32((const float*)bias_dev, h->bias.as<int32_t>(), d.oc, s));
    else CUDA_TRY(cudaMemcpyAsync(h->bias.p, bias_dev, (size_t)d.oc * 4, cudaMemcpyDeviceToDevice, s));
    d_bias = h->bias.as<int32_t>();
  }
  B200Q_TRY(make_epilogue(r, d_bias, h->mult, h->shift, s, &h->epi));
  B200Q_TRY(h->status.ensure(4));
  CUDA_TRY(cudaMemsetAsync(h->status.p, 0, 4, s));

  // tensor-core path: stride 1, no dilation, no groups, zero padding value, channels fit the K blocking
  const bool geometry_ok = d.sh == 1 && d.sw == 1 && d.dh == 1 && d.dw == 1 && d.groups == 1 && d.pad_value == 0;
  // 64 input channels and a filter wider than one tap: two horizontally adjacent taps form one 128-byte K block
  // (the bordered NHWC image holds pixel p+1's 64 channels right behind pixel p's), an odd last tap pairs with zeros
  h->pair_taps = d.ic == 64 && d.kw >= 2;
  const bool k_ok = (d.kh * d.kw == 1) ? (d.ic % 16 == 0) : (d.ic % 128 == 0 || h->pair_taps);
  h->bh = (int)(d.pht > d.phb ? d.pht : d.phb);
  h->bw = (int)(d.pwl > d.pwr ? d.pwl : d.pwr);
  h->Hp = (int)d.ih + 2 * h->bh;
  h->Wp = (int)d.iw + 2 * h->bw;
  const long long rows = (long long)d.n * h->Hp * h->Wp;
  h->use_tc = geometry_ok && k_ok && rows < 0x7fffffffLL && d.algo != 2;
  const long long out_rows = (long long)d.n * oh * ow;
  h->kpad = (int)((d.kh * d.kw * d.ic + 15) / 16 * 16);
  h->use_im2col = !h->use_tc && d.groups == 1 && d.pad_value == 0 && d.algo != 2 && out_rows < 0x7fffffffLL &&
                  (long long)d.kh * d.kw * d.ic < 0x7fffffffLL;
  h->few_channels = h->use_im2col && im2col_few_channels_ok((int)d.ic, (int)d.ih, (int)d.iw, (int)d.kh, (int)d.kw, (int)d.sh,
                                                            (int)d.sw, (int)d.dh, (int)d.dw, (int)d.pwl, (int)ow);
  if (h->few_channels) h->kpad = (int)((d.kh * d.ic * 8 + 63) / 64 * 64);  // rows start on 64-byte boundaries: whole sectors per TMA row
  if (d.algo == 1 && !h->use_tc && !h->use_im2col)
    return set_error(B200Q_ERR_UNSUPPORTED, "conv2d: the tensor-core paths need groups = 1 and a zero padding value");
  const size_t wbytes = (size_t)d.oc * (d.ic / d.groups) * d.kh * d.kw;
  if (h->use_tc && h->pair_taps) {
    const size_t pbytes = (size_t)d.oc * d.kh * ((d.kw + 1) / 2) * 128;
    B200Q_TRY(h->w_packed.ensure(pbytes));
    B200Q_TRY(repack_weight_pairs64(w_dev, w_is_f32, h->w_packed.p, (int)d.oc, (int)d.kh, (int)d.kw, s));
    // one extra (zero) pixel behind the image: the zero-weight partner of an odd last tap may read one pixel further
    B200Q_TRY(h->x_bordered.ensure((size_t)rows * d.ic + 64));
    CUDA_TRY(cudaMemsetAsync(h->x_bordered.p, 0, (size_t)rows * d.ic + 64, s));
  } else if (h->use_tc) {
    B200Q_TRY(h->w_packed.ensure(wbytes));
    B200Q_TRY(repack_weight_oihw(w_dev, w_is_f32, h->w_packed.p, (int)d.oc, (int)d.ic, (int)d.kh, (int)d.kw, s));
    B200Q_TRY(h->x_bordered.ensure((size_t)rows * d.ic));
    CUDA_TRY(cudaMemsetAsync(h->x_bordered.p, 0, (size_t)rows * d.ic, s));  // the border stays zero for every run
  } else if (h->use_im2col && h->few_channels) {
    B200Q_TRY(h->w_packed.ensure((size_t)d.oc * h->kpad));
    B200Q_TRY(repack_weight_fy_c_fx8(w_dev, w_is_f32, h->w_packed.p, (int)d.oc, (int)d.ic, (int)d.kh, (int)d.kw, h->kpad, s));
    B200Q_TRY(h->a_cols.ensure((size_t)out_rows * h->kpad));
  } else if (h->use_im2col) {
    const size_t kk = (size_t)d.kh * d.kw * d.ic;
    // weights [OC][kk] -> pitch kpad (zero padded)
    B200Q_TRY(h->w_oihw.ensure(wbytes));
    B200Q_TRY(repack_weight_oihw(w_dev, w_is_f32, h->w_oihw.p, (int)d.oc, (int)d.ic, (int)d.kh, (int)d.kw, s));
    B200Q_TRY(h->w_packed.ensure((size_t)d.oc * h->kpad));
    CUDA_TRY(cudaMemsetAsync(h->w_packed.p, 0, (size_t)d.oc * h->kpad, s));
    CUDA_TRY(cudaMemcpy2DAsync(h->w_packed.p, (size_t)h->kpad, h->w_oihw.p, kk, kk, (size_t)d.oc, cudaMemcpyDeviceToDevice, s));
    B200Q_TRY(h->x_bordered.ensure((size_t)rows * d.ic));
    CUDA_TRY(cudaMemsetAsync(h->x_bordered.p, 0, (size_t)rows * d.ic, s));
    B200Q_TRY(h->a_cols.ensure((size_t)out_rows * h->kpad));
    CUDA_TRY(cudaMemsetAsync(h->a_cols.p, 0, (size_t)out_rows * h->kpad, s));  // the pad columns stay zero
  } else {
    B200Q_TRY(h->w_oihw.ensure(wbytes));
    if (w_is_f32) B200Q_TRY(f32_to_q8((const float*)w_dev, h->w_oihw.p, (long long)wbytes, s));
    else CUDA_TRY(cudaMemcpyAsync(h->w_oihw.p, w_dev, wbytes, cudaMemcpyDeviceToDevice, s));
  }
  return B200Q_OK;
}

// x: device NCHW (bytes, or float holding integers); y: device NCHW native out dtype
// `images` < 0: the whole batch of the descriptor; otherwise the first `images` images of x / y (the operator face
// pipelines its host copies over pieces of the batch)
// The transposed product for a channels-last output: the GEMM's rows are the output channels (left operand = the
// filter [OC][K]), its columns the pixels (right operand = the activation rows [pixels][K]); element (oc, pixel)
// goes to out[pixel * OC + oc].  Every epilogue thread then owns one channel and keeps its requantisation constants
// in registers, which is what a short-K product (epilogue-bound) needs.  Expressed through the NCHW output mode:
// one "image" of OC x 1 "pixels" whose "channels" are the GEMM's columns.
bool transposed_product_ok(const Epilogue& e, int oc, long long pixels) {
  const bool fast = (e.dialect == B200Q_RQ_MULTIPLIER_SHIFT && e.round_mode == B200Q_ROUND_HALF_UP) ||
                    (e.dialect == B200Q_RQ_QDM && e.round_mode == B200Q_ROUND_HALF_AWAY_FROM_ZERO);
  static const bool on = [] {
    const char* v = getenv("B200Q_CONV_TRANSPOSED");  // =0 keeps the pixel-major product (for A/B timing)
    return !(v && v[0] == '0');
  }();
  return on && fast && oc % 128 == 0 && pixels > 128 && pixels < 0x7fffffffLL;
}

void make_transposed(IGemmProblem* p, int oc) {
  IGemmProblem q = *p;
  q.a = p->b;
  q.b = p->a;
  q.a_unsigned = p->b_unsigned;
  q.b_unsigned = p->a_unsigned;
  q.a_pitch = p->b_pitch;
  q.b_pitch = p->a_pitch;
  q.rows = oc;
  q.n = p->rows;
  q.row_pitch = 1;
  q.img_rows = 0x7fffffff;
  q.border_h = q.border_w = 0;
  q.out_h = oc;
  q.out_w = 1;
  q.out_mode = IGEMM_OUT_NCHW;
  q.ldc = 0;
  q.per_row_params = 1;
  *p = q;
}

// x_nhwc / y_nhwc: the tensor is [N][H][W][C] bytes instead of NCHW (the tensor-core routes only; a channels-last
// graph keeps its activations in that form between ops, so no transposing kernel runs and outputs are stored as
// whole 16-byte channel runs)
// `add`: fuse a tpu.Add of the output with add->residual (same shape and layout as y) into the epilogue; y then
// receives the Add's result and the convolution's own output is not stored (tensor-core routes only)
int conv_run(ConvHandle* h, const void* x, int x_is_f32, void* y, cudaStream_t s, long long images = -1, bool x_nhwc = false,
             bool y_nhwc = false, const b200q_fused_add* add = nullptr) {
  auto set_add = [&](IGemmProblem* p) {
    if (!add) return;
    p->res = add->residual;
    p->res_unsigned = add->residual_dtype == B200Q_DT_U8;
    p->add_m_self = add->conv_multiplier;
    p->add_s_self = add->conv_rshift;
    p->add_m_res = add->residual_multiplier;
    p->add_s_res = add->residual_rshift;
    const int lo = add->out_dtype == B200Q_DT_U8 ? 0 : -128, hi = add->out_dtype == B200Q_DT_U8 ? 255 : 127;
    p->add_lo = add->do_relu && lo < 0 ? 0 : lo;
    p->add_hi = hi;
  };
  if (add) {
    const bool t8 = (add->residual_dtype == B200Q_DT_I8 || add->residual_dtype == B200Q_DT_U8) &&
                    (add->out_dtype == B200Q_DT_I8 || add->out_dtype == B200Q_DT_U8);
    if (!add->residual || !t8) return set_error(B200Q_ERR_INVALID, "conv2d: fused Add needs an 8-bit residual tensor and output type");
    if (!(h->use_tc || h->use_im2col)) return set_error(B200Q_ERR_UNSUPPORTED, "conv2d: fused Add needs one of the tensor-core routes");
  }
  const b200q_conv2d_desc& d = h->d;
  const long long nb = images < 0 ? (long long)d.n : images;
  if (nb == 0) return B200Q_OK;
  if ((x_nhwc || y_nhwc) && !(h->use_tc || h->use_im2col))
    return set_error(B200Q_ERR_UNSUPPORTED, "conv2d: channels-last tensors need one of the tensor-core routes");
  if (x_nhwc && (x_is_f32 || d.ic % 16 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0))
    return set_error(B200Q_ERR_UNSUPPORTED, "conv2d: a channels-last input is 16-byte aligned bytes with channels %% 16 == 0");
  if (h->profiling && (h->use_tc || h->use_im2col)) B200Q_TRY(h->next_triple());
  if (h->use_tc) {
    if (h->profiling) CUDA_TRY(cudaEventRecord(h->ev[0], s));
    // a channels-last input without a border is the GEMM's left operand as it lies
    const bool direct = x_nhwc && h->bh == 0 && h->bw == 0 && !h->pair_taps;
    if (direct) {
    } else if (x_nhwc) {
      B200Q_TRY(nhwc_to_bordered_launch(x, h->x_bordered.p, nb, (int)d.ic, (int)d.ih, (int)d.iw, h->bh, h->bw, s));
    } else {
      B200Q_TRY(nchw_to_bordered_nhwc(x, x_is_f32, h->x_bordered.p, (int)nb, (int)d.ic, (int)d.ih, (int)d.iw, h->bh, h->bw, s));
    }
    if (h->profiling) CUDA_TRY(cudaEventRecord(h->ev[1], s));
    IGemmProblem p{};
    p.a = direct ? x : h->x_bordered.p;
    p.b = h->w_packed.p;
    p.a_unsigned = d.input_dtype == B200Q_DT_U8;
    p.b_unsigned = 0;
    p.a_pitch = d.ic;
    p.b_pitch = d.ic * d.kh * d.kw;
    p.rows = (int)(nb * h->Hp * h->Wp);
    p.n = (int)d.oc;
    p.k_per_tap = (int)d.ic;
    p.taps_h = (int)d.kh;
    p.taps_w = (int)d.kw;
    p.pad_top = (int)d.pht;
    p.pad_left = (int)d.pwl;
    p.row_pitch = h->Wp;
    p.img_rows = h->Hp * h->Wp;
    // GEMM row (hp, wp) reads bordered positions (hp + fy - pht, wp + fx - pwl), i.e. it is output pixel
    // (hp - bh, wp - bw); rows outside [0, oh) x [0, ow) are discarded by the epilogue.
    p.border_h = h->bh;
    p.border_w = h->bw;
    p.out_h = h->g.oh;
    p.out_w = h->g.ow;
    p.out_mode = y_nhwc ? IGEMM_OUT_NHWC : IGEMM_OUT_NCHW;
    p.ldc = y_nhwc ? (long long)d.oc : 0;
    p.out = y;
    // Programmatic dependent launch: behind a kernel of this library (layout, im2col, add, pool, another convolution)
    // the grid sets itself up while that kernel drains; behind any other kernel the attribute changes nothing.
    p.dependent_launch = h->profiling ? 0 : 1;
    if (h->pair_taps) {
      p.k_per_tap = 128;                    // two pixels' channels
      p.taps_w = (int)((d.kw + 1) / 2);
      p.tap_step_w = 2;
      p.b_pitch = (long long)d.kh * p.taps_w * 128;
    }
    // a 1x1 filter without a border is a plain GEMM whose rows are exactly the output pixels
    if (y_nhwc && d.kh * d.kw == 1 && h->bh == 0 && h->bw == 0 && transposed_product_ok(h->epi, (int)d.oc, p.rows))
      make_transposed(&p, (int)d.oc);
    set_add(&p);
    B200Q_TRY(igemm_i8_tcgen05_launch(p, h->epi, h->status.as<int>(), s));
    if (h->profiling) CUDA_TRY(cudaEventRecord(h->ev[2], s));
    return B200Q_OK;
  }
  if (h->use_im2col) {
    if (h->profiling) CUDA_TRY(cudaEventRecord(h->ev[0], s));
    if (x_nhwc) {
      // rows gathered straight from the channels-last input; taps that fall into the padding read zeros
      B200Q_TRY(im2col_nhwc_launch(x, h->a_cols.p, nb, (int)d.ic, (int)d.ih, (int)d.iw, h->g.oh, h->g.ow, (int)d.kh, (int)d.kw,
                                   (int)d.sh, (int)d.sw, (int)d.dh, (int)d.dw, -(int)d.pht, -(int)d.pwl, h->kpad, s));
    } else if (h->few_channels) {
      // few input channels (a network's stem): rows are built from 8-byte runs of the NCHW input
      B200Q_TRY(im2col_few_channels_launch(x, x_is_f32, h->a_cols.p, nb, (int)d.ic, (int)d.ih, (int)d.iw, h->g.oh, h->g.ow,
                                           (int)d.kh, (int)d.sh, (int)d.sw, (int)d.pht, (int)d.pwl, h->kpad, s));
    } else if (d.ic <= 4) {
      // few input channels, other geometry: rows are gathered byte by byte straight from the NCHW input
      B200Q_TRY(im2col_nchw_small_c_launch(x, x_is_f32, h->a_cols.p, nb, (int)d.ic, (int)d.ih, (int)d.iw, h->g.oh, h->g.ow,
                                           (int)d.kh, (int)d.kw, (int)d.sh, (int)d.sw, (int)d.dh, (int)d.dw, (int)d.pht,
                                           (int)d.pwl, h->kpad, s));
    } else {
      B200Q_TRY(nchw_to_bordered_nhwc(x, x_is_f32, h->x_bordered.p, (int)nb, (int)d.ic, (int)d.ih, (int)d.iw, h->bh, h->bw, s));
      B200Q_TRY(im2col_nhwc_launch(h->x_bordered.p, h->a_cols.p, nb, (int)d.ic, h->Hp, h->Wp, h->g.oh, h->g.ow, (int)d.kh,
                                   (int)d.kw, (int)d.sh, (int)d.sw, (int)d.dh, (int)d.dw, h->bh - (int)d.pht,
                                   h->bw - (int)d.pwl, h->kpad, s));
    }
    if (h->profiling) CUDA_TRY(cudaEventRecord(h->ev[1], s));
    IGemmProblem p{};
    p.a = h->a_cols.p;
    p.b = h->w_packed.p;
    p.a_unsigned = d.input_dtype == B200Q_DT_U8;
    p.a_pitch = p.b_pitch = h->kpad;
    p.rows = (int)(nb * h->g.oh * h->g.ow);
    p.n = (int)d.oc;
    p.k_per_tap = h->kpad;
    p.taps_h = p.taps_w = 1;
    p.row_pitch = h->g.ow;
    p.img_rows = h->g.oh * h->g.ow;
    p.out_h = h->g.oh;
    p.out_w = h->g.ow;
    p.out_mode = y_nhwc ? IGEMM_OUT_ROWMAJOR : IGEMM_OUT_NCHW;  // the rows are the output pixels in NHW order
    p.ldc = y_nhwc ? (long long)d.oc : 0;
    p.out = y;
    p.dependent_launch = h->profiling ? 0 : 1;
    if (y_nhwc && transposed_product_ok(h->epi, (int)d.oc, p.rows)) make_transposed(&p, (int)d.oc);
    set_add(&p);
    B200Q_TRY(igemm_i8_tcgen05_launch(p, h->epi, h->status.as<int>(), s));
    if (h->profiling) CUDA_TRY(cudaEventRecord(h->ev[2], s));
    return B200Q_OK;
  }
  const void* xin = x;
  if (x_is_f32) {
    const long long n = nb * d.ic * d.ih * d.iw;
    B200Q_TRY(h->x_q8.ensure((size_t)n));
    B200Q_TRY(f32_to_q8((const float*)x, h->x_q8.p, n, s));
    xin = h->x_q8.p;
  }
  ConvGeometry g = h->g;
  g.n = (int)nb;
  return conv2d_i8_direct_launch(xin, d.input_dtype == B200Q_DT_U8, h->w_oihw.as<int8_t>(), g, h->epi, y, s);
}

// tensor_hc_transpose (include/tpu_mlir/Support/MathUtils.h:213-228): src [n][c][h][w] -> dst [n][h][c][w]
int hc_transpose_f32(const float* src, float* dst, long long n, long long c, long long h, long long w, cudaStream_t s) {
  TopRemap m{};
  const long long dims[6] = {1, 1, n, h, c, w}, sstr[6] = {0, 0, c * h * w, w, h * w, 1}, dstr[6] = {0, 0, c * h * w, c * w, w, 1};
  for (int i = 0; i < 6; ++i) {
    m.dims[i] = dims[i];
    m.src_stride[i] = sstr[i];
    m.dst_stride[i] = dstr[i];
    m.mul[i] = m.div[i] = 1;
    m.mod[i] = m.off[i] = 0;
    m.extent[i] = dims[i];
  }
  m.dst_offset = 0;
  return top_remap_launch(src, dst, 4, m, nullptr, s);
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" {

// ------------------------------------------------------------------------------------------------ MatMul
int b200q_matmul_init(const b200q_matmul_desc* desc, void** handle) {
  if (!desc || !handle) return set_error(B200Q_ERR_INVALID, "matmul_init: null argument");
  B200Q_TRY(validate_matmul(*desc));
  auto* h = new (std::nothrow) MatMulHandle();
  if (!h) return set_error(B200Q_ERR_NOMEM, "matmul_init: out of host memory");
  *handle = h;
  return B200Q_OK;
}

void b200q_matmul_deinit(void** handle) {
  if (handle && *handle) {
    delete static_cast<MatMulHandle*>(*handle);
    *handle = nullptr;
  }
}

int b200q_matmul_inference(const b200q_matmul_desc* desc, float* const* inputs, int n_inputs, float* const* outputs,
                           int n_outputs, void** handle) {
  if (!desc || !inputs || !outputs || !handle || n_inputs < 2 || n_outputs < 1 || !inputs[0] || !inputs[1] || !outputs[0])
    return set_error(B200Q_ERR_INVALID, "matmul_inference: null argument");
  const b200q_matmul_desc& d = *desc;
  B200Q_TRY(validate_matmul(d));
  const bool own = (*handle == nullptr);
  if (own) B200Q_TRY(b200q_matmul_init(desc, handle));
  MatMulHandle* h = static_cast<MatMulHandle*>(*handle);
  cudaStream_t s = 0;
  int rc = B200Q_OK;
  do {
    const float* bias_f = (d.with_bias && n_inputs > 2) ? inputs[2] : nullptr;
    const float* multi_f = (n_inputs > 3) ? inputs[3] : nullptr;
    if (d.with_bias && !bias_f) { rc = set_error(B200Q_ERR_INVALID, "matmul: with_bias but inputs[2] is null"); break; }
    // hdim_is_batch: batch x batch_low independent products; a transposed operand / output carries batch_low between its
    // matrix dimensions and is brought to batch-major order by tensor_hc_transpose first (lib/Support/Dnnl/MatMul.cpp:172-241)
    const bool hdim = d.hdim_is_batch != 0;
    const int64_t blow = hdim && d.batch_low > 0 ? d.batch_low : 1;
    const int64_t B = d.batch * blow;
    const bool right_t = d.right_transpose && !hdim, left_t = d.left_transpose && !hdim, out_t = d.output_transpose && !hdim;
    const int64_t nb = d.right_batched ? B : 1;
    const int64_t rows = d.right_batched ? d.M : B * d.M;  // a shared right operand folds the batch into M
    const size_t a_elems = (size_t)(B * d.M * d.K), b_elems = (size_t)(nb * d.K * d.N), o_elems = (size_t)(B * d.M * d.N);
    // right operand: [N,K] bytes per batch
    const bool cached = d.right_is_weight && h->weights_ready && h->weight_version == d.weight_version && h->weight_ptr == inputs[1];
    if (!cached) {
      if ((rc = h->b_f32.ensure(b_elems * 4))) break;
      if ((rc = h->b_nk.ensure(b_elems))) break;
      if (cudaMemcpyAsync(h->b_f32.p, inputs[1], b_elems * 4, cudaMemcpyHostToDevice, s) != cudaSuccess) { rc = cuda_error(cudaGetLastError(), "H2D right", __FILE__, __LINE__); break; }
      const float* right_f = h->b_f32.as<float>();
      if (hdim && d.right_transpose) {   // [batch][K][batch_low][N] -> [batch][batch_low][K][N]
        if ((rc = h->perm.ensure(b_elems * 4))) break;
        if ((rc = hc_transpose_f32(right_f, h->perm.as<float>(), d.batch, d.K, blow, d.N, s))) break;
        right_f = h->perm.as<float>();
      }
      for (int64_t b = 0; b < nb && rc == B200Q_OK; ++b) {
        const float* src = right_f + b * d.K * d.N;
        uint8_t* dst = h->b_nk.as<uint8_t>() + b * d.K * d.N;
        rc = right_t ? f32_to_q8(src, dst, d.K * d.N, s) : transpose_to_u8(src, 1, dst, (int)d.K, (int)d.N, s);
      }
      if (rc) break;
      if (bias_f) {
        if ((rc = h->stage_f32.ensure((size_t)d.N * 4))) break;
        if ((rc = h->bias.ensure((size_t)d.N * 4))) break;
        if (cudaMemcpyAsync(h->stage_f32.p, bias_f, (size_t)d.N * 4, cudaMemcpyHostToDevice, s) != cudaSuccess) { rc = cuda_error(cudaGetLastError(), "H2D bias", __FILE__, __LINE__); break; }
        if ((rc = f32_to_i32(h->stage_f32.as<float>(), h->bias.as<int32_t>(), d.N, s))) break;
        // the staging buffer is reused for A below; stream order keeps this safe
      }
      h->weights_ready = true;
      h->weight_version = d.weight_version;
      h->weight_ptr = inputs[1];
    }
    if ((rc = h->status.ensure(4))) break;
    if (cudaMemsetAsync(h->status.p, 0, 4, s) != cudaSuccess) { rc = cuda_error(cudaGetLastError(), "memset", __FILE__, __LINE__); break; }
    if (a_elems == 0) break;
    if ((rc = h->stage_f32.ensure(a_elems * 4 > (size_t)d.N * 4 ? a_elems * 4 : (size_t)d.N * 4))) break;
    if ((rc = h->a_q8.ensure(a_elems))) break;
    if ((rc = h->out_q.ensure(o_elems * dtype_size(d.out_dtype)))) break;
    if ((rc = h->out_f32.ensure(o_elems * 4))) break;
    if (cudaMemcpyAsync(h->stage_f32.p, inputs[0], a_elems * 4, cudaMemcpyHostToDevice, s) != cudaSuccess) { rc = cuda_error(cudaGetLastError(), "H2D input", __FILE__, __LINE__); break; }
    if (hdim && d.left_transpose) {   // [batch][M][batch_low][K] -> [batch][batch_low][M][K]
      if ((rc = h->perm.ensure(a_elems * 4))) break;
      if ((rc = hc_transpose_f32(h->stage_f32.as<float>(), h->perm.as<float>(), d.batch, d.M, blow, d.K, s))) break;
      if ((rc = f32_to_q8(h->perm.as<float>(), h->a_q8.p, (long long)a_elems, s))) break;
    } else if (left_t) {
      // the input is stored [batch][K][M] (MatMul.cpp:24-135 reads M from the last dimension; lib/Support/Dnnl/MatMul.cpp:
      // 182-186 transposes every batch entry before the product)
      for (int64_t b = 0; b < d.batch && rc == B200Q_OK; ++b)
        rc = transpose_to_u8(h->stage_f32.as<float>() + b * d.K * d.M, 1, h->a_q8.as<uint8_t>() + b * d.M * d.K, (int)d.K, (int)d.M, s);
      if (rc) break;
    } else if ((rc = f32_to_q8(h->stage_f32.as<float>(), h->a_q8.p, (long long)a_elems, s))) {
      break;
    }
    const int n_launch = (d.right_batched || d.is_cv18xx) ? (int)B : 1;
    const int64_t rows_per = (n_launch == 1) ? rows : d.M;
    for (int b = 0; b < n_launch && rc == B200Q_OK; ++b) {
      ResolvedRequant r;
      if ((rc = resolve_matmul(d, multi_f, b, &r))) break;
      Epilogue e;
      // per-launch multiplier/shift arrays: small, re-uploaded (stream ordered) for each batch entry
      if ((rc = make_epilogue(r, bias_f ? h->bias.as<int32_t>() : nullptr, h->mult, h->shift, s, &e))) break;
      const uint8_t* a = h->a_q8.as<uint8_t>() + (size_t)b * d.M * d.K;
      const uint8_t* bm = h->b_nk.as<uint8_t>() + (d.right_batched ? (size_t)b * d.K * d.N : 0);
      uint8_t* o = h->out_q.as<uint8_t>() + (size_t)b * d.M * d.N * dtype_size(d.out_dtype);
      rc = gemm_dispatch(a, d.input_dtype, bm, d.right_dtype, rows_per, d.N, d.K, d.input_zp, d.right_zp, e, o,
                         h->status.as<int>(), d.algo, s);
      if (n_launch > 1 && rc == B200Q_OK && cudaStreamSynchronize(s) != cudaSuccess) rc = cuda_error(cudaGetLastError(), "sync", __FILE__, __LINE__);
    }
    if (rc) break;
    if ((rc = q_to_f32(h->out_q.p, d.out_dtype, h->out_f32.as<float>(), (long long)o_elems, s))) break;
    const float* result = h->out_f32.as<float>();
    if (hdim && d.output_transpose) {   // [batch][batch_low][M][N] -> [batch][M][batch_low][N]
      if ((rc = h->stage_f32.ensure(o_elems * 4))) break;
      if ((rc = hc_transpose_f32(h->out_f32.as<float>(), h->stage_f32.as<float>(), d.batch, blow, d.M, d.N, s))) break;
      result = h->stage_f32.as<float>();
    } else if (out_t) {
      // the output is stored [batch][N][M] (lib/Support/Dnnl/MatMul.cpp:229-238)
      if ((rc = h->stage_f32.ensure(o_elems * 4))) break;
      for (int64_t b = 0; b < d.batch && rc == B200Q_OK; ++b)
        rc = transpose_f32(h->out_f32.as<float>() + b * d.M * d.N, h->stage_f32.as<float>() + b * d.M * d.N, (int)d.M, (int)d.N, s);
      if (rc) break;
      result = h->stage_f32.as<float>();
    }
    if (cudaMemcpyAsync(outputs[0], result, o_elems * 4, cudaMemcpyDeviceToHost, s) != cudaSuccess) { rc = cuda_error(cudaGetLastError(), "D2H output", __FILE__, __LINE__); break; }
    rc = read_status(h->status, s, "matmul");
  } while (0);
  if (rc != B200Q_OK) cudaStreamSynchronize(s);
  if (own) b200q_matmul_deinit(handle);
  return rc;
}

int b200q_gemm_i8_dev(const void* a, int a_dtype, const void* b_nk, int b_dtype, int64_t M, int64_t N, int64_t K,
                      const b200q_epilogue* epilogue, void* out, int32_t* status, int algo, void* stream) {
  if (!a || !b_nk || !epilogue || !out) return set_error(B200Q_ERR_INVALID, "gemm_i8_dev: null argument");
  if (!is_q8(a_dtype) || !is_q8(b_dtype)) return set_error(B200Q_ERR_INVALID, "gemm_i8_dev: operands must be int8/uint8");
  if (M < 0 || N < 1 || K < 1 || M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return set_error(B200Q_ERR_INVALID, "gemm_i8_dev: bad shape");
  Epilogue e;
  static_assert(sizeof(Epilogue) == sizeof(b200q_epilogue), "public and internal epilogue structs must match");
  std::memcpy(&e, epilogue, sizeof(e));
  return gemm_dispatch(a, a_dtype, b_nk, b_dtype, M, N, K, 0, 0, e, out, status, algo, static_cast<cudaStream_t>(stream));
}

int b200q_gemm_i8_zp_dev(const void* a, int a_dtype, const void* b_nk, int b_dtype, int64_t M, int64_t N, int64_t K,
                         int32_t input_zp, int32_t right_zp, const b200q_epilogue* epilogue, void* out, int32_t* status,
                         int algo, void* stream) {
  if (!a || !b_nk || !epilogue || !out) return set_error(B200Q_ERR_INVALID, "gemm_i8_zp_dev: null argument");
  if (!is_q8(a_dtype) || !is_q8(b_dtype)) return set_error(B200Q_ERR_INVALID, "gemm_i8_zp_dev: operands must be int8/uint8");
  if (M < 0 || N < 1 || K < 1 || M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return set_error(B200Q_ERR_INVALID, "gemm_i8_zp_dev: bad shape");
  Epilogue e;
  std::memcpy(&e, epilogue, sizeof(e));
  return gemm_dispatch(a, a_dtype, b_nk, b_dtype, M, N, K, input_zp, right_zp, e, out, status, algo, static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------------------------------------ Conv2D
// Operator face: filter and bias from the host float buffers into the handle (upload, conversion, repacking).
static int conv_upload_weights(ConvHandle* h, const b200q_conv2d_desc& d, float* const* inputs, int n_inputs, cudaStream_t s) {
  const size_t w_elems = (size_t)d.oc * (d.ic / d.groups) * d.kh * d.kw;
  B200Q_TRY(h->w_f32.ensure(w_elems * 4));
  CUDA_TRY(cudaMemcpyAsync(h->w_f32.p, inputs[1], w_elems * 4, cudaMemcpyHostToDevice, s));
  const float* bias_f = (d.with_bias && n_inputs > 2) ? inputs[2] : nullptr;
  if (d.with_bias && !bias_f) return set_error(B200Q_ERR_INVALID, "conv2d: with_bias but inputs[2] is null");
  if (bias_f) {
    B200Q_TRY(h->bias_f32.ensure((size_t)d.oc * 4));
    CUDA_TRY(cudaMemcpyAsync(h->bias_f32.p, bias_f, (size_t)d.oc * 4, cudaMemcpyHostToDevice, s));
  }
  B200Q_TRY(conv_setup(h, d, h->w_f32.p, 1, bias_f ? h->bias_f32.p : nullptr, 1, s));
  CUDA_TRY(cudaStreamSynchronize(s));
  h->weight_version = d.weight_version;
  h->weight_ptr = inputs[1];
  return B200Q_OK;
}

int b200q_conv2d_init(const b200q_conv2d_desc* desc, float* const* inputs, int n_inputs, void** handle) {
  if (!desc || !inputs || !handle || n_inputs < 2 || !inputs[1]) return set_error(B200Q_ERR_INVALID, "conv2d_init: null argument");
  const b200q_conv2d_desc& d = *desc;
  int64_t oh, ow;
  B200Q_TRY(conv_out_dims(d, &oh, &ow));
  auto* h = new (std::nothrow) ConvHandle();
  if (!h) return set_error(B200Q_ERR_NOMEM, "conv2d_init: out of host memory");
  cudaStream_t s = 0;
  const int rc = conv_upload_weights(h, d, inputs, n_inputs, s);
  if (rc != B200Q_OK) {
    cudaStreamSynchronize(s);
    delete h;
    return rc;
  }
  *handle = h;
  return B200Q_OK;
}

void b200q_conv2d_deinit(void** handle) {
  if (handle && *handle) {
    delete static_cast<ConvHandle*>(*handle);
    *handle = nullptr;
  }
}

int b200q_conv2d_inference(const b200q_conv2d_desc* desc, float* const* inputs, int n_inputs, float* const* outputs,
                           int n_outputs, void** handle) {
  if (!handle || !*handle) return set_error(B200Q_ERR_INVALID, "conv2d_inference: no handle (call b200q_conv2d_init first)");
  if (!inputs || !outputs || n_inputs < 1 || n_outputs < 1 || !inputs[0] || !outputs[0]) return set_error(B200Q_ERR_INVALID, "conv2d_inference: null argument");
  ConvHandle* h = static_cast<ConvHandle*>(*handle);
  cudaStream_t s = 0;
  // The interpreter may rewrite a filter in place (setTensor, fake_quant_weight: ModuleInterpreter.cpp:583-612); the
  // caller says so by bumping weight_version (or by handing in another buffer), and the device copy is remade.
  if (desc && n_inputs >= 2 && inputs[1] && (desc->weight_version != h->weight_version || inputs[1] != h->weight_ptr)) {
    if (desc->n != h->d.n || desc->ic != h->d.ic || desc->ih != h->d.ih || desc->iw != h->d.iw || desc->oc != h->d.oc ||
        desc->kh != h->d.kh || desc->kw != h->d.kw || desc->groups != h->d.groups)
      return set_error(B200Q_ERR_INVALID, "conv2d_inference: the descriptor's shape differs from the one the handle was made for");
    B200Q_TRY(conv_upload_weights(h, *desc, inputs, n_inputs, s));
  }
  const b200q_conv2d_desc& d = h->d;
  const size_t x_elems = (size_t)d.n * d.ic * d.ih * d.iw;
  const size_t y_elems = (size_t)d.n * d.oc * h->g.oh * h->g.ow;
  if (x_elems == 0) return B200Q_OK;
  B200Q_TRY(h->x_f32.ensure(x_elems * 4));
  B200Q_TRY(h->y_q.ensure(y_elems * dtype_size(d.out_dtype)));
  B200Q_TRY(h->y_f32.ensure(y_elems * 4));
  // The float ABI makes this call a PCIe transfer with a convolution in the middle: the batch is cut into pieces so
  // that the upload of piece i+1, the kernels of piece i and the download of piece i-1 overlap (both directions of
  // the link at once; the host buffers should be pinned for that).
  const size_t xi = (size_t)d.ic * d.ih * d.iw, yi = (size_t)d.oc * h->g.oh * h->g.ow;  // elements per image
  // The first upload and the last download overlap with nothing, which favours many pieces; every piece costs
  // launches and stream hand-offs, which favours few.  Measured on config 1 (103 MB each way): 8 pieces 2.59 ms,
  // 16 pieces 2.76 ms, 32 pieces 3.32 ms.  Pieces are >= 2 MB, at most 8 (B200Q_CONV_PIECES overrides the count).
  static const int max_pieces = [] {
    const char* v = getenv("B200Q_CONV_PIECES");
    const int n = v ? atoi(v) : 0;
    return n >= 1 && n <= 1024 ? n : 8;
  }();
  const long long min_imgs = (long long)((((size_t)2 << 20) + xi * 4 - 1) / (xi * 4));
  const long long even = (d.n + max_pieces - 1) / max_pieces;
  long long per = even > min_imgs ? even : min_imgs;
  if (per > d.n) per = d.n;
  const int pieces = (int)((d.n + per - 1) / per);
  int rc = B200Q_OK;
  if (pieces <= 1) {
    CUDA_TRY(cudaMemcpyAsync(h->x_f32.p, inputs[0], x_elems * 4, cudaMemcpyHostToDevice, s));
    rc = conv_run(h, h->x_f32.p, 1, h->y_q.p, s);
    if (rc == B200Q_OK) rc = q_to_f32(h->y_q.p, d.out_dtype, h->y_f32.as<float>(), (long long)y_elems, s);
    if (rc == B200Q_OK && cudaMemcpyAsync(outputs[0], h->y_f32.p, y_elems * 4, cudaMemcpyDeviceToHost, s) != cudaSuccess)
      rc = cuda_error(cudaGetLastError(), "D2H output", __FILE__, __LINE__);
    if (rc == B200Q_OK) rc = read_status(h->status, s, "conv2d");
    else cudaStreamSynchronize(s);
    return rc;
  }
  CUDA_TRY(cudaStreamSynchronize(s));  // whatever the caller queued on the default stream comes first
  B200Q_TRY(h->ensure_pipe(pieces));
  cudaStream_t s_in = h->pipe[0], s_cmp = h->pipe[1], s_out = h->pipe[2];
  const size_t ysz = dtype_size(d.out_dtype);
  for (int c = 0; c < pieces && rc == B200Q_OK; ++c) {
    const long long i0 = (long long)c * per, cnt = (i0 + per <= d.n) ? per : d.n - i0;
    float* xd = h->x_f32.as<float>() + (size_t)i0 * xi;
    uint8_t* yq = h->y_q.as<uint8_t>() + (size_t)i0 * yi * ysz;
    float* yd = h->y_f32.as<float>() + (size_t)i0 * yi;
    CUDA_TRY(cudaMemcpyAsync(xd, inputs[0] + (size_t)i0 * xi, (size_t)cnt * xi * 4, cudaMemcpyHostToDevice, s_in));
    CUDA_TRY(cudaEventRecord(h->pipe_ev[2 * c], s_in));
    CUDA_TRY(cudaStreamWaitEvent(s_cmp, h->pipe_ev[2 * c], 0));
    rc = conv_run(h, xd, 1, yq, s_cmp, cnt);
    if (rc == B200Q_OK) rc = q_to_f32(yq, d.out_dtype, yd, (long long)((size_t)cnt * yi), s_cmp);
    if (rc != B200Q_OK) break;
    CUDA_TRY(cudaEventRecord(h->pipe_ev[2 * c + 1], s_cmp));
    CUDA_TRY(cudaStreamWaitEvent(s_out, h->pipe_ev[2 * c + 1], 0));
    CUDA_TRY(cudaMemcpyAsync(outputs[0] + (size_t)i0 * yi, yd, (size_t)cnt * yi * 4, cudaMemcpyDeviceToHost, s_out));
  }
  if (rc == B200Q_OK) {
    CUDA_TRY(cudaStreamSynchronize(s_out));
    rc = read_status(h->status, s_cmp, "conv2d");
  } else {
    for (auto& st : h->pipe) cudaStreamSynchronize(st);
  }
  return rc;
}

int b200q_conv2d_dev_create(const b200q_conv2d_desc* desc, const void* filter_oihw_s8, const int32_t* bias_s32, void** handle) {
  if (!desc || !filter_oihw_s8 || !handle) return set_error(B200Q_ERR_INVALID, "conv2d_dev_create: null argument");
  auto* h = new (std::nothrow) ConvHandle();
  if (!h) return set_error(B200Q_ERR_NOMEM, "conv2d_dev_create: out of host memory");
  cudaStream_t s = 0;
  int rc = conv_setup(h, *desc, filter_oihw_s8, 0, bias_s32, 0, s);
  if (rc == B200Q_OK && cudaStreamSynchronize(s) != cudaSuccess) rc = cuda_error(cudaGetLastError(), "sync", __FILE__, __LINE__);
  if (rc != B200Q_OK) {
    delete h;
    return rc;
  }
  *handle = h;
  return B200Q_OK;
}

int b200q_conv2d_dev_run(void* handle, const void* x_nchw, void* y_nchw, void* stream) {
  if (!handle || !x_nchw || !y_nchw) return set_error(B200Q_ERR_INVALID, "conv2d_dev_run: null argument");
  return conv_run(static_cast<ConvHandle*>(handle), x_nchw, 0, y_nchw, static_cast<cudaStream_t>(stream));
}

int b200q_conv2d_dev_run_layout(void* handle, const void* x, int32_t x_layout, void* y, int32_t y_layout, void* stream) {
  if (!handle || !x || !y) return set_error(B200Q_ERR_INVALID, "conv2d_dev_run_layout: null argument");
  if ((x_layout != B200Q_LAYOUT_NCHW && x_layout != B200Q_LAYOUT_NHWC) || (y_layout != B200Q_LAYOUT_NCHW && y_layout != B200Q_LAYOUT_NHWC))
    return set_error(B200Q_ERR_INVALID, "conv2d_dev_run_layout: unknown layout");
  return conv_run(static_cast<ConvHandle*>(handle), x, 0, y, static_cast<cudaStream_t>(stream), -1, x_layout == B200Q_LAYOUT_NHWC,
                  y_layout == B200Q_LAYOUT_NHWC);
}

int b200q_conv2d_dev_run_add(void* handle, const void* x, int32_t x_layout, void* y, int32_t y_layout, const b200q_fused_add* add,
                             void* stream) {
  if (!handle || !x || !y || !add) return set_error(B200Q_ERR_INVALID, "conv2d_dev_run_add: null argument");
  if ((x_layout != B200Q_LAYOUT_NCHW && x_layout != B200Q_LAYOUT_NHWC) || (y_layout != B200Q_LAYOUT_NCHW && y_layout != B200Q_LAYOUT_NHWC))
    return set_error(B200Q_ERR_INVALID, "conv2d_dev_run_add: unknown layout");
  return conv_run(static_cast<ConvHandle*>(handle), x, 0, y, static_cast<cudaStream_t>(stream), -1, x_layout == B200Q_LAYOUT_NHWC,
                  y_layout == B200Q_LAYOUT_NHWC, add);
}

int b200q_conv2d_dev_route(void* handle) {
  if (!handle) return set_error(B200Q_ERR_INVALID, "conv2d_dev_route: null handle");
  ConvHandle* h = static_cast<ConvHandle*>(handle);
  return h->use_tc ? 1 : (h->use_im2col ? 2 : 0);
}

int b200q_conv2d_dev_status(void* handle, void* stream) {
  if (!handle) return set_error(B200Q_ERR_INVALID, "conv2d_dev_status: null handle");
  return read_status(static_cast<ConvHandle*>(handle)->status, static_cast<cudaStream_t>(stream), "conv2d");
}

void b200q_conv2d_dev_destroy(void** handle) { b200q_conv2d_deinit(handle); }

int b200q_conv2d_dev_set_profiling(void* handle, int enable) {
  if (!handle) return set_error(B200Q_ERR_INVALID, "conv2d_dev_set_profiling: null handle");
  ConvHandle* h = static_cast<ConvHandle*>(handle);
  h->profiling = enable != 0;
  h->runs_recorded = 0;  // a new measurement starts
  return B200Q_OK;
}

int b200q_conv2d_dev_profile(void* handle, int64_t* runs, double* layout_ms_total, double* kernel_ms_total) {
  if (!handle || !runs || !layout_ms_total || !kernel_ms_total) return set_error(B200Q_ERR_INVALID, "conv2d_dev_profile: null argument");
  ConvHandle* h = static_cast<ConvHandle*>(handle);
  *runs = (int64_t)h->runs_recorded;
  *layout_ms_total = 0.0;
  *kernel_ms_total = 0.0;
  for (size_t r = 0; r < h->runs_recorded; ++r) {
    cudaEvent_t* e = &h->events[r * 3];
    float a = 0.f, b = 0.f;
    CUDA_TRY(cudaEventSynchronize(e[2]));
    CUDA_TRY(cudaEventElapsedTime(&a, e[0], e[1]));
    CUDA_TRY(cudaEventElapsedTime(&b, e[1], e[2]));
    *layout_ms_total += a;
    *kernel_ms_total += b;
  }
  return B200Q_OK;
}

// ------------------------------------------------------------------------------------------------ glue ops (device face)
int b200q_requant_int_axis_dev(const int32_t* x, int64_t outer, int64_t C, int64_t inner, const int32_t* multiplier,
                               const int32_t* shift, const int32_t* zero_point, int32_t dialect, int32_t round_mode,
                               int32_t in_zp, int32_t out_dtype, void* out, void* stream) {
  if (!x || !out || outer < 0 || C < 1 || inner < 1 || C > 0x7fffffffLL) return set_error(B200Q_ERR_INVALID, "requant_int_axis_dev: bad argument");
  Epilogue e{};
  e.dialect = dialect;
  e.round_mode = round_mode;
  e.out_dtype = out_dtype;
  return requant_axis_launch(x, outer, (int)C, inner, multiplier, shift, zero_point, 1, in_zp, e, out, static_cast<cudaStream_t>(stream));
}

int b200q_add_i8_dev(const void* a, int32_t a_dtype, const void* b, int32_t b_dtype, int64_t count, int32_t m0, int32_t s0,
                     int32_t m1, int32_t s1, int32_t do_relu, int32_t out_dtype, void* out, void* stream) {
  if (!a || !b || !out || count < 0) return set_error(B200Q_ERR_INVALID, "add_i8_dev: bad argument");
  return add_i8_launch(a, a_dtype, b, b_dtype, count, m0, s0, m1, s1, do_relu, out_dtype, out, static_cast<cudaStream_t>(stream));
}

int b200q_constop_i8_dev(int32_t form, const void* x, int32_t dtype, int64_t count, int32_t multiplier, double const_val, int32_t rshift,
                         int32_t in_zp, int32_t do_relu, float relu_limit, int32_t out_dtype, void* out, void* stream) {
  if (!x || !out || count < 0 || form < 0 || form > 3 || !is_q8(dtype) || rshift < 0 || rshift > 62)
    return set_error(B200Q_ERR_INVALID, "constop_i8_dev: bad argument");
  if (form >= 2 && in_zp != 0) return set_error(B200Q_ERR_INVALID, "constop_i8_dev: tpu.SubConst takes no input zero point");
  return constop_i8_launch(form, x, dtype, count, multiplier, const_val, rshift, in_zp, do_relu, relu_limit, out_dtype, out,
                           static_cast<cudaStream_t>(stream));
}

int b200q_sub_i8_dev(const void* a, int32_t a_dtype, const void* b, int32_t b_dtype, int64_t count, int32_t m0, int32_t s0,
                     int32_t m1, int32_t s1, int32_t do_relu, int32_t out_dtype, void* out, void* stream) {
  if (!a || !b || !out || count < 0 || !is_q8(a_dtype) || !is_q8(b_dtype)) return set_error(B200Q_ERR_INVALID, "sub_i8_dev: bad argument");
  return sub_i8_launch(a, a_dtype, b, b_dtype, count, m0, s0, m1, s1, do_relu, out_dtype, out, static_cast<cudaStream_t>(stream));
}

int b200q_lut_dev(const void* x, int64_t count, const void* table, int32_t table_dtype, void* out, void* stream) {
  if (!x || !table || !out || count < 0) return set_error(B200Q_ERR_INVALID, "lut_dev: bad argument");
  return lut_launch(x, count, table, (int)dtype_size(table_dtype), out, static_cast<cudaStream_t>(stream));
}

int b200q_mulshift_i8_dev(const void* x, int32_t dtype, int64_t count, int32_t multiplier, int32_t rshift, int32_t in_zp,
                          int32_t out_zp, int32_t out_dtype, void* out, void* stream) {
  if (!x || !out || count < 0 || !is_q8(dtype) || rshift < 0 || rshift > 62)
    return set_error(B200Q_ERR_INVALID, "mulshift_i8_dev: bad argument");
  return mulshift_i8_launch(x, dtype, count, multiplier, rshift, in_zp, out_zp, out_dtype, out, static_cast<cudaStream_t>(stream));
}

int b200q_addconst_i8_dev(const void* x, int32_t dtype, int64_t count, int32_t multiplier, double const_val, int32_t rshift, int32_t in_zp,
                          int32_t do_relu, int32_t out_dtype, void* out, void* stream) {
  if (!x || !out || count < 0 || !is_q8(dtype) || rshift < 0 || rshift > 62)
    return set_error(B200Q_ERR_INVALID, "addconst_i8_dev: bad argument");
  return addconst_i8_launch(x, dtype, count, multiplier, const_val, rshift, in_zp, do_relu, out_dtype, out, static_cast<cudaStream_t>(stream));
}

int b200q_requant_fp_dev(const void* x, int32_t dtype, int64_t count, double scale, double offset, int32_t out_zp, int32_t quant_mode,
                         int32_t round_mode, int32_t out_dtype, void* out, void* stream) {
  if (!x || !out || count < 0 || (dtype != B200Q_DT_I32 && dtype != B200Q_DT_F32) || out_dtype >= B200Q_DT_F32)
    return set_error(B200Q_ERR_INVALID, "requant_fp_dev: bad argument");
  const bool tflite = quant_mode == B200Q_QM_TFLITE || quant_mode == B200Q_QM_TFLITE_LSHIFT;
  if (!tflite && quant_mode != B200Q_QM_MULTIPLIER_SHIFT)
    return set_error(B200Q_ERR_UNSUPPORTED, "requant_fp_dev: quant mode %d (the 8-bit float outputs of OnlyScale are not implemented)", quant_mode);
  return requant_fp_launch(x, dtype == B200Q_DT_I32, count, (float)scale, (float)offset, out_zp, tflite, round_mode, out_dtype, out,
                           static_cast<cudaStream_t>(stream));
}

int b200q_prelu_dev(const void* x, int32_t dtype, const void* slope, int64_t count, int64_t inner, int32_t num_slope, int32_t rshift,
                    int32_t out_dtype, void* out, void* stream) {
  if (!x || !slope || !out || count < 0 || inner < 1 || num_slope < 1 || rshift < 0 || rshift > 62)
    return set_error(B200Q_ERR_INVALID, "prelu_dev: bad argument");
  if (dtype == B200Q_DT_F32 && out_dtype == B200Q_DT_F32)
    return prelu_f32_launch(static_cast<const float*>(x), static_cast<const float*>(slope), count, inner, num_slope, static_cast<float*>(out),
                            static_cast<cudaStream_t>(stream));
  if (!is_q8(dtype) || !is_q8(out_dtype)) return set_error(B200Q_ERR_UNSUPPORTED, "prelu_dev: f32 -> f32 or 8-bit -> 8-bit");
  return prelu_i8_launch(x, dtype, slope, count, inner, num_slope, rshift, out_dtype, out, static_cast<cudaStream_t>(stream));
}

int b200q_mul_i8_dev(const void* a, int32_t a_dtype, const void* b, int32_t b_dtype, int64_t count, int32_t multiplier,
                     int32_t rshift, int32_t do_relu, int32_t out_dtype, void* out, void* stream) {
  if (!a || !b || !out || count < 0 || !is_q8(a_dtype) || !is_q8(b_dtype) || rshift < 0 || rshift > 62)
    return set_error(B200Q_ERR_INVALID, "mul_i8_dev: bad argument");
  return mul_i8_launch(a, a_dtype, b, b_dtype, count, multiplier, rshift, do_relu, out_dtype, out, static_cast<cudaStream_t>(stream));
}

int b200q_pool2d_i8_nhwc_dev(const void* x, int32_t dtype, int64_t n, int32_t c, int32_t ih, int32_t iw, int32_t kh, int32_t kw,
                             int32_t sh, int32_t sw, int32_t pht, int32_t phb, int32_t pwl, int32_t pwr, int32_t is_avg,
                             int32_t multiplier, int32_t rshift, int32_t do_relu, int32_t out_dtype, void* out, void* stream) {
  if (!x || !out || n < 0 || n > 0x7fffffffLL || c < 1 || ih < 1 || iw < 1 || kh < 1 || kw < 1 || sh < 1 || sw < 1)
    return set_error(B200Q_ERR_INVALID, "pool2d_i8_nhwc_dev: bad argument");
  return pool2d_i8_nhwc_launch(x, dtype, n, c, ih, iw, kh, kw, sh, sw, pht, phb, pwl, pwr, is_avg ? 1 : 0, multiplier, rshift,
                               do_relu, out_dtype, out, static_cast<cudaStream_t>(stream));
}

int b200q_pool2d_i8_dev(const void* x, int32_t dtype, int64_t nc, int32_t ih, int32_t iw, int32_t kh, int32_t kw, int32_t sh,
                        int32_t sw, int32_t pht, int32_t phb, int32_t pwl, int32_t pwr, int32_t is_avg, int32_t multiplier,
                        int32_t rshift, int32_t do_relu, int32_t out_dtype, void* out, void* stream) {
  if (!x || !out || nc < 0 || nc > 0x7fffffffLL || ih < 1 || iw < 1 || kh < 1 || kw < 1 || sh < 1 || sw < 1)
    return set_error(B200Q_ERR_INVALID, "pool2d_i8_dev: bad argument");
  return pool2d_i8_launch(x, dtype, (int)nc, ih, iw, kh, kw, sh, sw, pht, phb, pwl, pwr, is_avg ? 1 : 0, multiplier, rshift,
                          do_relu, out_dtype, out, static_cast<cudaStream_t>(stream));
}

int b200q_cast_f32_to_q8_dev(const float* x, int64_t count, double scale, int32_t zero_point, int32_t round_mode,
                             int32_t out_dtype, void* out, void* stream) {
  if (!x || !out || count < 0 || !(scale > 0)) return set_error(B200Q_ERR_INVALID, "cast_f32_to_q8_dev: bad argument");
  return cast_f32_q8_launch(x, count, scale, zero_point, round_mode, out_dtype, out, static_cast<cudaStream_t>(stream));
}

int b200q_cast_q8_to_f32_dev(const void* x, int32_t dtype, int64_t count, double scale, int32_t zero_point, float* out,
                             void* stream) {
  if (!x || !out || count < 0) return set_error(B200Q_ERR_INVALID, "cast_q8_to_f32_dev: bad argument");
  return cast_q8_f32_launch(x, dtype, count, scale, zero_point, out, static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------------------------------------ RequantInt(Axis), operator face
// Stateless: uploads, runs, downloads (these ops carry no weights worth keeping resident).
int b200q_requant_int_axis_inference(const b200q_requant_desc* desc, float* const* inputs, int n_inputs,
                                     float* const* outputs, int n_outputs) {
  if (!desc || !inputs || !outputs || n_inputs < 1 || n_outputs < 1 || !inputs[0] || !outputs[0])
    return set_error(B200Q_ERR_INVALID, "requant_int_axis_inference: null argument");
  const b200q_requant_desc& d = *desc;
  if (d.outer < 0 || d.channels < 1 || d.inner < 1) return set_error(B200Q_ERR_INVALID, "requant: bad shape");
  const long long total = d.outer * d.channels * d.inner;
  const int C = (int)d.channels;
  std::vector<int32_t> m((size_t)C), sh((size_t)C), zp((size_t)C);
  int dialect, rmode = d.round_mode;
  const bool tf = d.quant_mode == B200Q_QM_TFLITE || d.quant_mode == B200Q_QM_TFLITE_LSHIFT;
  if (!tf && d.quant_mode != B200Q_QM_MULTIPLIER_SHIFT) return set_error(B200Q_ERR_UNSUPPORTED, "requant: quant_mode %d does nothing in the reference", d.quant_mode);
  dialect = tf ? B200Q_RQ_QDM : B200Q_RQ_MULTIPLIER_SHIFT;
  if (d.per_axis) {
    if (n_inputs < 2 || !inputs[1]) return set_error(B200Q_ERR_INVALID, "requant_int_axis: quant operand missing");
    if (d.quant_words != 0 && d.quant_words != 2 && d.quant_words != 3) return set_error(B200Q_ERR_INVALID, "requant_int_axis: quant_words must be 2 or 3");
    for (int c = 0; c < C; ++c) {
      long long mm, ss, zz;
      if (d.quant_words == 2) {
        // every chip but BM1684X: {multiplier, packed word}, shift = the low byte as a signed char, zero point = the
        // high half-word as a signed short (RequantIntAxis.cpp:49-54), both read back from floats
        mm = (long long)inputs[1][c * 2];
        const uint32_t tmp = (uint32_t)inputs[1][c * 2 + 1];
        ss = (long long)(signed char)(tmp & 0xffu);
        zz = (long long)(short)((tmp & 0xffff0000u) >> 16);
      } else {  // BM1684X: {multiplier, shift, zero point} (RequantIntAxis.cpp:45-48)
        mm = (long long)inputs[1][c * 3];
        ss = (long long)inputs[1][c * 3 + 1];
        zz = (long long)inputs[1][c * 3 + 2];
      }
      if (mm > 2147483647ll || mm < -2147483648ll) return set_error(B200Q_ERR_UNSUPPORTED, "requant: multiplier does not fit int32");
      m[(size_t)c] = (int32_t)mm;
      zp[(size_t)c] = (int32_t)zz;
      // TFLite: MultiplyByQuantizedMultiplier(x, m, shift); MultiplierShift: rshift = shift word when fuse_rq_axis, else -shift
      sh[(size_t)c] = tf ? (int32_t)ss : (d.fuse_rq_axis ? (int32_t)ss : (int32_t)(-ss));
    }
  } else {  // tpu.RequantInt: one multiplier / rshift attribute (RequantInt.cpp:33-36)
    for (int c = 0; c < C; ++c) {
      m[(size_t)c] = (int32_t)d.multiplier;
      zp[(size_t)c] = d.out_zp;
      sh[(size_t)c] = tf ? (int32_t)(-d.rshift) : (int32_t)d.rshift;
    }
  }
  cudaStream_t s = 0;
  DevBuf xf, xi, q, of, dm, ds, dz;
  B200Q_TRY(xf.upload(inputs[0], (size_t)total * 4, s));
  B200Q_TRY(xi.ensure((size_t)total * 4));
  B200Q_TRY(f32_to_i32(xf.as<float>(), xi.as<int32_t>(), total, s));
  B200Q_TRY(dm.upload(m.data(), (size_t)C * 4, s));
  B200Q_TRY(ds.upload(sh.data(), (size_t)C * 4, s));
  B200Q_TRY(dz.upload(zp.data(), (size_t)C * 4, s));
  B200Q_TRY(q.ensure((size_t)total * dtype_size(d.out_dtype)));
  Epilogue e{};
  e.dialect = dialect;
  e.round_mode = rmode;
  e.out_dtype = d.out_dtype;
  B200Q_TRY(requant_axis_launch(xi.as<int32_t>(), d.outer, C, d.inner, dm.as<int32_t>(), ds.as<int32_t>(), dz.as<int32_t>(), 1,
                                tf ? 0 : d.in_zp, e, q.p, s));
  B200Q_TRY(q_to_f32(q.p, d.out_dtype, xf.as<float>(), total, s));
  CUDA_TRY(cudaMemcpyAsync(outputs[0], xf.p, (size_t)total * 4, cudaMemcpyDeviceToHost, s));
  CUDA_TRY(cudaStreamSynchronize(s));
  return B200Q_OK;
}

}  // extern "C"

// Test aid (no counterpart in the reference): the tensor-core GEMM/convolution launches that follow expect
// `extra_tx_bytes` more per stage than their loads deliver and give every wait `budget_ns`; (0, 0) restores normal use.
extern "C" void b200q_debug_set_wait_fault(int32_t extra_tx_bytes, int64_t budget_ns) {
  b200q::igemm_set_wait_test(extra_tx_bytes, budget_ns);
}
