// Test infrastructure only: compiles the reference's OWN code of some ops of the wider op set, for the tests' numpy
// restatements of those ops to be checked against.
//
// The build recipe (Makefile target ref_moreops) cuts these line ranges out of the reference checkout into generated include
// files under _ref/ (never committed; each range is checked against the text its first line must contain):
//   include/tpu_mlir/Backend/BM168x/Param.h:197-206                PLATFORM_SUPPORT
//   lib/Dialect/Top/Interfaces/Interp.cpp:14-15,:27-175            MIN / MAX, calc_resize_scale, backward_map, interp_core
//   third_party/nntoolchain/include/bmcpu_common.h:469-477         grid sampler enums
//   include/tpu_mlir/Support/GenericCpuFunc.h:58-62,:635-659       tensor_list_t, GridSamplerParam, class GridSamplerFunc
//   lib/Support/GenericCpuFunc.cpp:25-33,:3325-3579                the mish helper; GridSamplerFunc (constructor ... invoke)
//   lib/Support/ActiveUtils.cpp:16-149                             the activation helpers and getActivateFunc(mode, coeffs)
//   lib/Support/MathUtils.cpp:673-705,:1539-1564                   pad_tensor_for_deconv, swap_dim_data
//   include/tpu_mlir/Support/MathUtils.h:213-228                   tensor_hc_transpose
//   lib/Dialect/Top/Interfaces/Pad.cpp:121-213                     the reflect / edge loops of top.Pad
// This file supplies what those bodies expect from the rest of the reference (the ActiveMode enumeration with the
// dialect's numbering, two typedefs, llvm_unreachable) and plain C entry points.
#include <algorithm>
#include <cassert>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <memory>
#include <numeric>
#include <string>
#include <vector>
#include <linux/limits.h>   // XATTR_LIST_MAX, which the reference's sign() tests
#undef ARG_MAX               // (that header's macro; Arg.cpp has an enumerator of this name)

#define llvm_unreachable(msg) abort()
#define omp_schedule(n) 1

namespace tpu {
// Tpu_ActiveMode, include/tpu_mlir/Dialect/Tpu/IR/TpuOps.td:284-321 (same numbering)
enum class ActiveMode {
  TANH = 0, SIGMOID, RELU, EXP, ELU, SQRT, SQUARE, RSQRT, ABSVAL, LN, ROUND, CEIL, FLOOR, SIN, COS, IS_FINITE, MISH, SWISH, HSWISH, SILU,
  ARCSIN, ARCCOS, ARCSINH, ARCCOSH, ARCTANH, SINH, COSH, TAN, SIGN, GELU, ERF, HSIGMOID, LOG_SIGMOID, SOFT_PLUS, SOFT_SIGN, LOG2, TGELU, QGELU
};
}  // namespace tpu
typedef std::shared_ptr<std::vector<double>> f64_array_t;
using activate_f = std::function<double(double)>;

#include "_ref/platform_support.inc"
#include "_ref/interp_macros.inc"
#include "_ref/interp_core.inc"

#include "_ref/grid_enums.inc"
#include "_ref/tensor_list.inc"
#include "_ref/grid_class.inc"
#include "_ref/mish.inc"
#include "_ref/grid_func.inc"

#include "_ref/active_utils.inc"

#include "_ref/pad_for_deconv.inc"
#include "_ref/swap_dim.inc"
#include "_ref/hc_transpose.inc"

extern "C" {

// interp_core<float> on one plane (Interp.cpp:105-175); platform_sp is a PLATFORM_SUPPORT value
void ref_interp_plane(const float* in, float* out, int ih, int iw, int oh, int ow, int align_corners, int half_pixel, int platform_sp) {
  interp_core<float>(in, out, ih, iw, oh, ow, 0, 0, align_corners != 0, half_pixel != 0, (PLATFORM_SUPPORT)platform_sp);
}

// GridSamplerFunc::invoke with a 4-D grid, called the way GridSampler.cpp:36-62 fills the parameter
void ref_grid_sampler(float* x, float* grid, float* y, int n, int c, int ih, int iw, int oh, int ow, int mode, int padding_mode,
                      int align_corners) {
  GridSamplerParam p;
  tensor_list_t in, g, out;
  in.ptr = x;
  in.shape = {n, c, ih, iw};
  in.size = (size_t)n * c * ih * iw;
  g.ptr = grid;
  g.shape = {n, oh, ow, 2};
  g.size = (size_t)n * oh * ow * 2;
  out.ptr = y;
  out.shape = {n, c, oh, ow};
  out.size = (size_t)n * c * oh * ow;
  p.inputs = {in, g};
  p.output = out;
  p.mode = mode;
  p.padding_mode = padding_mode;
  p.align_corners = align_corners != 0;
  GridSamplerFunc f(p);
  f.invoke();
}

// tpu::ActiveOp's loop (Active.cpp:20-25) over the function getActivateFunc returns
void ref_active(int mode, int n_coeffs, double c0, double c1, const float* x, float* y, long long n) {
  f64_array_t coeffs;
  if (n_coeffs > 0) {
    coeffs = std::make_shared<std::vector<double>>();
    coeffs->push_back(c0);
    if (n_coeffs > 1) coeffs->push_back(c1);
  }
  activate_f f = getActivateFunc((tpu::ActiveMode)mode, coeffs);
  for (long long i = 0; i < n; ++i) y[i] = f(x[i]);
}

// top::SwapDimInnerOp::inference (SwapDimInner.cpp:17-46): swap_dim_data once per axis with an offset, ping-ponging buffers
void ref_swap_dim_inner(const float* x, float* y, int rank, const int64_t* shape, const int64_t* offsets) {
  std::vector<int64_t> ishape(shape, shape + rank), offs(offsets, offsets + rank);
  long long total = 1;
  for (int i = 0; i < rank; ++i) total *= shape[i];
  std::vector<float> a(x, x + total), b((size_t)total);
  for (int i = 0; i < rank; ++i)
    if (offsets[i] != 0) {
      swap_dim_data(a.data(), b.data(), ishape, offs);   // takes the first axis whose offset is not zero, and zeroes it
      a.swap(b);
    }
  memcpy(y, a.data(), (size_t)total * sizeof(float));
}

void ref_pad_tensor_for_deconv(float* dst, float* src, int n, int c, int h, int w, int kh, int kw, int dh, int dw, int sh, int sw, int pht,
                               int phb, int pwl, int pwr, int oph, int opw, float pad_value) {
  pad_tensor_for_deconv(dst, src, n, c, 1, h, w, 1, kh, kw, 1, dh, dw, 1, sh, sw, 0, 0, pht, phb, pwl, pwr, 0, oph, opw, pad_value);
}

void ref_tensor_hc_transpose(float* dst, float* src, long long n, long long c, long long h, long long w) {
  tensor_hc_transpose<float>(dst, src, n, c, h, w);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------------------
// Whole inference bodies of top::Depth2SpaceOp (Depth2Space.cpp:19-104), top::GatherOp (Gather.cpp:17-82), top::ArgOp
// (Arg.cpp:17-97 with its comparison helper) and gather_dim8 (GatherElements.cpp:20-80), compiled as members of stand-in
// operator classes that answer the attribute accessors from plain fields.
struct LogicalResult {};
static inline LogicalResult success() { return {}; }
struct InferenceParameter {
  std::vector<float*> inputs, outputs;
};
#define ASSERT_THIS(x) assert(x)
struct FakeValue {
  std::vector<int64_t> shape;
  bool none = false;
};
struct FakeStr {
  std::string s;
  std::string str() const { return s; }
};
namespace module {
static inline void getNCHW(const FakeValue& v, int64_t& n, int64_t& c, int64_t& h, int64_t& w, bool) {
  n = v.shape[0];
  c = v.shape[1];
  h = v.shape[2];
  w = v.shape[3];
}
static inline std::vector<int64_t> getShape(const FakeValue& v) { return v.shape; }
static inline int64_t getNumElements(const FakeValue& v) {
  int64_t n = 1;
  for (auto d : v.shape) n *= d;
  return n;
}
static inline bool isNone(const FakeValue& v) { return v.none; }
static std::vector<int64_t> g_last_shape;
static inline void setShape(const FakeValue&, const std::vector<int64_t>& s) { g_last_shape = s; }
}  // namespace module

namespace top {
struct Depth2SpaceOp {
  FakeValue in_, out_;
  bool in_nchw, out_nchw, crd, inv, swap;
  int64_t bh, bw;
  FakeValue getInput() { return in_; }
  FakeValue getOutput() { return out_; }
  bool getInIs_NCHW() { return in_nchw; }
  bool getOutIs_NCHW() { return out_nchw; }
  bool getIs_CRD() { return crd; }
  bool getIsInversed() { return inv; }
  bool getSwapCr() { return swap; }
  int64_t getBlockH() { return bh; }
  int64_t getBlockW() { return bw; }
  LogicalResult inference(InferenceParameter& p);
};
struct GatherOp {
  FakeValue in_, idx_, out_;
  int64_t axis;
  bool keepdims;
  FakeValue getInput() { return in_; }
  FakeValue getIndices() { return idx_; }
  FakeValue getOutput() { return out_; }
  int64_t getAxis() { return axis; }
  bool getKeepdims() { return keepdims; }
  LogicalResult inference(InferenceParameter& p);
};
struct ArgOp {
  FakeValue in_, idx_, val_;
  int64_t axis;
  bool keepdims, select_last;
  FakeStr mode;
  FakeValue getInput() { return in_; }
  FakeValue getIndices() { return idx_; }
  FakeValue getValues() { return val_; }
  int64_t getAxis() { return axis; }
  void setAxis(int64_t a) { axis = a; }
  bool getKeepdims() { return keepdims; }
  bool getSelectLastIndex() { return select_last; }
  FakeStr getMode() { return mode; }
  LogicalResult inference(InferenceParameter& p);
};
}  // namespace top

#include "_ref/depth2space.inc"
#include "_ref/gather.inc"
#include "_ref/arg.inc"
#include "_ref/gather_dim8.inc"

extern "C" {

void ref_depth2space(float* x, float* y, const int64_t* in_shape, const int64_t* out_shape, int bh, int bw, int crd, int inversed, int in_nchw,
                     int out_nchw, int swap_cr) {
  top::Depth2SpaceOp op;
  op.in_.shape.assign(in_shape, in_shape + 4);
  op.out_.shape.assign(out_shape, out_shape + 4);
  op.bh = bh;
  op.bw = bw;
  op.crd = crd;
  op.inv = inversed;
  op.in_nchw = in_nchw;
  op.out_nchw = out_nchw;
  op.swap = swap_cr;
  InferenceParameter p;
  p.inputs = {x};
  p.outputs = {y};
  op.inference(p);
}

void ref_gather(float* x, float* indices, float* y, int rank, const int64_t* shape, int idx_rank, const int64_t* idx_shape, int axis) {
  top::GatherOp op;
  op.in_.shape.assign(shape, shape + rank);
  op.idx_.shape.assign(idx_shape, idx_shape + idx_rank);
  op.axis = axis;
  op.keepdims = true;
  InferenceParameter p;
  p.inputs = {x, indices};
  p.outputs = {y};
  op.inference(p);
}

void ref_arg(float* x, float* indices, float* values, int rank, const int64_t* shape, int axis, int is_max, int select_last) {
  top::ArgOp op;
  op.in_.shape.assign(shape, shape + rank);
  op.val_.none = values == nullptr;
  op.axis = axis;
  op.keepdims = true;
  op.select_last = select_last;
  op.mode.s = is_max ? "ArgMax" : "ArgMin";
  InferenceParameter p;
  p.inputs = {x};
  p.outputs = {indices, values};
  op.inference(p);
}

void ref_gather_elements(float* dst, const float* src, const float* indices, const int* indices_shape, int* src_shape, int rank, int axis) {
  gather_dim8(dst, src, indices, indices_shape, src_shape, rank, axis, rank);
}

// top::PadOp::inference, modes "reflect" and "edge" (Pad.cpp:121-213) on a 4-D tensor padded in its last two dimensions
void ref_pad_mode(const float* src, float* dst, int n_, int c_, int h_, int w_, int pt, int pl, int pb, int pr, const char* mode) {
  const int64_t in = n_, ic = c_, ih = h_, iw = w_;
  std::vector<int> pads = {0, 0, pt, pl, 0, 0, pb, pr};
  const int64_t oc = ic, oh = pt + pb + ih, ow = pl + pr + iw;
  const std::string pad_mode = mode;
#define UNREACHABLE_THIS(msg) abort()
#include "_ref/pad_modes.inc"
#undef UNREACHABLE_THIS
}

}  // extern "C"
