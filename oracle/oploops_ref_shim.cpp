// Test infrastructure only: compiles the reference's OWN operator loops for the oracle to be checked against.
//
// The interpreter cannot be built here (it needs MLIR, oneDNN and flatbuffers), but the loops that turn an fp32
// accumulator into a quantised output are plain C++ whose only ties to MLIR are a handful of accessors.  The build
// recipe (Makefile target ref_oploops) cuts these line ranges out of the reference checkout into generated include
// files under _ref/ (never committed; each range is checked against the line it must start with):
//   include/tpu_mlir/Support/MathUtils.h:172-181                   declarations (default arguments) of the rounding helpers
//   lib/Support/MathUtils.cpp:849-872                              saturate
//   lib/Dialect/Tpu/Interfaces/Common/Conv2D.cpp:311-340           requantisation of tpu.Conv2D
//   lib/Dialect/Tpu/Interfaces/Common/MatMul.cpp:637-728           requantisation of tpu.MatMul (all dialects, cv18xx)
//   lib/Dialect/Tpu/Interfaces/Common/Add.cpp:180-206              tpu.Add, symmetric int8, BM168x
//   lib/Dialect/Tpu/Interfaces/Common/Pool2D.cpp:179-198           tpu.Pool2D average, symmetric int8
//   lib/Dialect/Tpu/Interfaces/Common/A16MatMul.cpp:190-197        4-bit group dequantisation of tpu.A16MatMul
//   lib/Dialect/Tpu/Interfaces/Common/RequantIntAxis.cpp:18-120    tpu.RequantIntAxis::inference, whole body
//   lib/Dialect/Tpu/Interfaces/Common/RequantInt.cpp:18-71         tpu.RequantInt::inference, whole body
//   lib/Support/CastUtils.cpp:15-47                                requant / dequant of tpu.Cast
//   lib/Dialect/Tpu/Interfaces/Common/RequantFp.cpp:19-67          tpu.RequantFp::inference, whole body
//   lib/Dialect/Tpu/Interfaces/Common/MaxConst.cpp:36-45, MinConst.cpp:36-45   the uniform-quantized loops
//   lib/Dialect/Tpu/Interfaces/Common/PRelu.cpp:73-96              the symmetric 8-bit loop of tpu.PRelu
//   lib/Dialect/Tpu/Interfaces/Common/SubConst.cpp:19-111          tpu.SubConst::inference, whole body
//   lib/Dialect/Tpu/Interfaces/Common/Sub.cpp:160-185              tpu.Sub, symmetric int8, BM168x
//   lib/Dialect/Tpu/Interfaces/Common/Reduce.cpp:206-213           the requantisation tail of tpu.Reduce
//   include/tpu_mlir/Support/MathUtils.h:311-337, lib/Dialect/Top/Interfaces/Cast.cpp:18-64   to_int8 ... to_uint16; top.Cast::inference, whole body
// This file supplies only what those bodies expect from the rest of the reference: the operator's attribute
// accessors (answered from a context the C entry points fill), the shapes, a stand-in for mlir::Type that knows a
// width and a signedness, and the element-wise fp32 add (+ ReLU) that the reference obtains from oneDNN's binary
// primitive (lib/Support/Dnnl/Binary.cpp; oneDNN is a third-party dependency that is not in the checkout).
#include <algorithm>
#include <cassert>
#include <climits>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <optional>
#include <string>
#include <vector>

#include "_ref/mathutils_enum.inc"

namespace tpu {
enum class RequantMode { TFLite_LShift = 0, TFLite = 1, MultiplierShift = 2, OnlyShift = 3, QDM = 4, OnlyScale = 5 };
}

// ---------------------------------------------------------------------------------------------- stand-ins
namespace mlir {
struct IntegerType {
  int width = 0;
  bool uns = false, valid = false;
  explicit operator bool() const { return valid; }
  int getWidth() const { return width; }
  bool isUnsigned() const { return uns; }
};
struct FloatType {};
struct Type {
  int width = 8;
  bool uns = false, is_int = true;
  void dump() const {}
  bool isInteger(int w) const { return is_int && width == w; }
  bool isFloat8E4M3FN() const { return false; }
  bool isFloat8E5M2() const { return false; }
  bool isBF16() const { return false; }
  bool isF16() const { return false; }
  template <typename T>
  bool isa() const;
};
template <>
bool Type::isa<FloatType>() const { return !is_int; }
template <>
bool Type::isa<IntegerType>() const { return is_int; }
}  // namespace mlir
template <typename T>
static T dyn_cast(const mlir::Type& t);
template <>
mlir::IntegerType dyn_cast<mlir::IntegerType>(const mlir::Type& t) {
  mlir::IntegerType i;
  i.width = t.width;
  i.uns = t.uns;
  i.valid = t.is_int;
  return i;
}
namespace llvm {
static int64_t maxUIntN(int n) { return (int64_t)((n >= 64) ? ~0ull : ((1ull << n) - 1)); }
static int64_t maxIntN(int n) { return (int64_t)((1ull << (n - 1)) - 1); }
static int64_t minIntN(int n) { return -(int64_t)(1ull << (n - 1)); }
}  // namespace llvm
#define llvm_unreachable(msg) abort()
static int omp_schedule(int count) { return count > 64 ? count / 64 : 1; }  // only a loop chunk size

// what the cut bodies ask the operator and the module for
struct QType {
  int64_t zp = 0;
  double scale = 1.0;
  int expressed = 0;  // 0 f32, 1 f16, 2 bf16
  int64_t getZeroPoint() const { return zp; }
  double getScale() const { return scale; }
  struct Expressed {
    int e;
    bool isF32() const { return e == 0; }
    bool isF16() const { return e == 1; }
    bool isBF16() const { return e == 2; }
  };
  Expressed getExpressedType() const { return Expressed{expressed}; }
  void dump() const {}
};
struct Ctx {
  bool cv18xx = false, bm1684x = true;
  tpu::RequantMode qmode = tpu::RequantMode::MultiplierShift;
  int round_mode = 0;
  bool fuse_rq = false, fuse_rq_axis = false, do_relu = false, right_is_weight = true;
  std::optional<std::vector<int64_t>> rshifts, multipliers;
  std::optional<std::vector<double>> out_scales;
  std::vector<int64_t> out_shape;
  mlir::Type out_type;
  QType out_q, in_q;
  bool in_quantized = false;
  int64_t rshift = 0, multiplier = 1;                       // RequantInt attributes
  std::optional<int64_t> pool_multiplier, pool_rshift;      // Pool2D attributes
  int64_t batch = 1, batch_low = 1, M = 0, N = 0;           // MatMul parseParam
};
static Ctx g;

namespace module {
static bool isCV18xx() { return g.cv18xx; }
static bool isBM1684X() { return g.bm1684x; }
struct Value { int which; };
static const std::vector<int64_t>& getShape(Value) { return g.out_shape; }
static int64_t getNumElements(Value) {
  int64_t n = 1;
  for (auto d : g.out_shape) n *= d;
  return n;
}
static mlir::Type getStorageType(Value) { return g.out_type; }
static bool isUniformQuantized(Value v) { return v.which == 0 ? true : g.in_quantized; }
static QType getUniformQuantizedType(Value v) { return v.which == 0 ? g.out_q : g.in_q; }
static bool isWeight(Value) { return g.right_is_weight; }
static bool g_module_asym = false;
static bool isAsymmetric() { return g_module_asym; }
static void setShape(Value, const std::vector<int64_t>&) {}
typedef std::shared_ptr<std::vector<int64_t>> i64_array_t;
typedef std::shared_ptr<std::vector<double>> f64_array_t;
// Module.cpp:570-578: the attribute's values when present (their count is asserted), else num_elem defaults
static i64_array_t getI64Array(const std::optional<std::vector<int64_t>>& a, int64_t num_elem, int64_t default_value) {
  if (a.has_value()) {
    assert((int64_t)a->size() == num_elem);
    return std::make_shared<std::vector<int64_t>>(*a);
  }
  return std::make_shared<std::vector<int64_t>>(num_elem, default_value);
}
static i64_array_t getI64Array(const std::optional<std::vector<int64_t>>& a) { return std::make_shared<std::vector<int64_t>>(*a); }
static f64_array_t getF64Array(const std::vector<double>& a) { return std::make_shared<std::vector<double>>(a); }
}  // namespace module
using module::f64_array_t;
using module::i64_array_t;

template <typename T>
int64_t to_int(T v, RoundingMode round_mode);
#include "_ref/mathutils_decl.inc"   // MathUtils.h:172-181: the declarations, with the reference's default arguments
#include "_ref/mathutils_body.inc"   // to_int, RightShiftRound, MultiplyByQuantizedMultiplier, applyMultiplierAndRShift

template <typename T>
int64_t saturate(T v, mlir::Type type, RoundingMode round_mode = ROUNDING_HALF_AWAY_FROM_ZERO);
#include "_ref/saturate.inc"

struct InferenceParameter {
  std::vector<float*> inputs, outputs;
  void* handle = nullptr;
};
static module::Value getOutput() { return module::Value{0}; }
static module::Value getInput() { return module::Value{1}; }
static module::Value getRight() { return module::Value{2}; }
static tpu::RequantMode getQuantMode() { return g.qmode; }
static int getRoundMode() { return g.round_mode; }
static RoundingMode round_mode_convert(int m) { return (RoundingMode)m; }  // the attribute already carries the enum value
static bool getFuseRq() { return g.fuse_rq; }
static bool getFuseRqAxis() { return g.fuse_rq_axis; }
static bool getDoRelu() { return g.do_relu; }
static const std::optional<std::vector<int64_t>>& getRshifts() { return g.rshifts; }
static const std::optional<std::vector<int64_t>>& getMultipliers() { return g.multipliers; }
static const std::optional<std::vector<double>>& getOutScales() { return g.out_scales; }
static int success() { return 0; }
#define ASSERT_THIS(x) assert(x)

// ---------------------------------------------------------------------------------------------- tpu.Conv2D
static void conv2d_requant(InferenceParameter& p, int64_t n, int64_t c, int64_t h, int64_t w, bool use_winograd,
                           const std::vector<int64_t>& rshift, const std::vector<int64_t>& mult,
                           const std::vector<int32_t>& bias, bool do_relu) {
  auto rshift_v = std::make_shared<std::vector<int64_t>>(rshift);
  auto multiplier_v = std::make_shared<std::vector<int64_t>>(mult);
  auto bias_i32 = std::make_shared<std::vector<int32_t>>(bias);
  bool per_axis = (int64_t)rshift_v->size() == c;   // Conv2D.cpp:302
  auto o_qtype = g.out_q;
  auto out_type = g.out_type;
#include "_ref/conv2d_requant.inc"
}

// ---------------------------------------------------------------------------------------------- tpu.MatMul
struct matmul_attr_t {
  int64_t batch, batch_low, M, N;
};
static matmul_attr_t parseParam() { return matmul_attr_t{g.batch, g.batch_low, g.M, g.N}; }
static void matmul_requant(InferenceParameter& p) {
  auto out_type = g.out_type;
  bool is_cv18xx = g.cv18xx;
  {
#include "_ref/matmul_requant.inc"
  }
}

// ---------------------------------------------------------------------------------------------- tpu.Add
// element-wise fp32 add with optional ReLU: what the reference's Binary (oneDNN binary_add + eltwise_relu post-op,
// lib/Support/Dnnl/Binary.cpp) computes for equal shapes
struct Binary {
  const float *l = nullptr, *r = nullptr;
  float* dst = nullptr;
  int64_t count = 0;
  bool relu = false, sub = false;
  Binary& lhs(const float* p, const std::vector<int64_t>&) {
    l = p;
    return *this;
  }
  Binary& rhs(const float* p, const std::vector<int64_t>&) {
    r = p;
    return *this;
  }
  void run() {
    for (int64_t i = 0; i < count; ++i) {
      float v = sub ? l[i] - r[i] : l[i] + r[i];
      dst[i] = relu && v < 0.f ? 0.f : v;
    }
  }
};
static std::vector<module::Value> getInputs() { return {module::Value{1}, module::Value{1}}; }
static void add_int8(InferenceParameter& p, int64_t num_elem) {
  auto out_type = g.out_type;
  {
#include "_ref/add_int8.inc"
  }
}

// ---------------------------------------------------------------------------------------------- tpu.Pool2D (average)
struct Pooling {
  int kh, kw;
};
static void avgpool_int8(InferenceParameter& p, Pooling* pooling, int64_t num_elem) {
  auto out_type = g.out_type;
  auto getMultiplier = [] { return g.pool_multiplier; };
  auto getRshift = [] { return g.pool_rshift; };
  {
#include "_ref/avgpool_int8.inc"
  }
}

// ---------------------------------------------------------------------------------------------- tpu.A16MatMul (4-bit)
static void a16_dequant(const float* weight, const float* scale, const float* zp, int K, int N, int q_group_size,
                        std::vector<float>& new_weight) {
  // K, N as A16MatMul.cpp:173 leaves them: N already doubled (two weights per byte)
#include "_ref/a16_dequant.inc"
}

// ---------------------------------------------------------------------------------------------- RequantIntAxis / RequantInt
static int requant_int_axis(InferenceParameter& p) {
#include "_ref/requant_int_axis.inc"
}
static int requant_int(InferenceParameter& p) {
  auto getRshift = [] { return g.rshift; };
  auto getMultiplier = [] { return g.multiplier; };
#include "_ref/requant_int.inc"
}

// ---------------------------------------------------------------------------------------------- tpu.Cast helpers
namespace quant {
typedef ::QType UniformQuantizedType;
}
namespace tpu_mlir {
float F16(float src);               // lib/Support/Float16.cpp, compiled from the checkout into this library
float BF16(float src, bool is_tpu = true);
#include "_ref/castutils.inc"
}  // namespace tpu_mlir

// ---------------------------------------------------------------------------------------------- RequantFp, Max/MinConst, PRelu
struct FpAttr {
  double v;
  double convertToDouble() const { return v; }
};
static double g_fp_scale = 1.0, g_fp_offset = 0.0;
static void F8E4M3(float*, float*, int64_t, double, bool) { abort(); }   // 8-bit float outputs are not exercised
static void F8E5M2(float*, float*, int64_t, double, bool) { abort(); }
static int requant_fp(InferenceParameter& p) {
  using tpu::RequantMode;   // the body sits inside namespace tpu in the reference
  auto getScale = [] { return FpAttr{g_fp_scale}; };
  auto getOffset = [] { return FpAttr{g_fp_offset}; };
#include "_ref/requant_fp.inc"
}
static void maxconst_q(InferenceParameter& p, int64_t num_elem, double izp, float const_val) {
  auto out_type = g.out_type;
  auto getMultiplier = [] { return g.multiplier; };
  auto getRshift = [] { return g.rshift; };
#include "_ref/maxconst_q.inc"
}
static void minconst_q(InferenceParameter& p, int64_t num_elem, double izp, float const_val) {
  auto out_type = g.out_type;
  auto getMultiplier = [] { return g.multiplier; };
  auto getRshift = [] { return g.rshift; };
#include "_ref/minconst_q.inc"
}
static void prelu_q(InferenceParameter& p, int64_t num_outer, int64_t num_inner, int64_t num_slope, int64_t shift) {
  auto out_type = g.out_type;
  const bool is_cv18xx = false;
  int64_t shift_pos = 0, multiplier_pos = 0;
#include "_ref/prelu_q.inc"
}

// ---------------------------------------------------------------------------------------------- tpu.SubConst, top.Cast
namespace tpu_mlir {
void F16(float* p_src, float* p_dst, int num);                      // lib/Support/Float16.cpp (compiled in)
void BF16(float* p_src, float* p_dst, int num, bool is_tpu = true);
}  // namespace tpu_mlir
static double g_const_val = 0.0, g_relu_limit = -1.0;
static bool g_is_reverse = false;
struct LimitAttr {
  double v;
  double getValueAsDouble() const { return v; }
};
static int subconst(InferenceParameter& p) {
  using mlir::FloatType;
  using tpu_mlir::BF16;
  using tpu_mlir::F16;
  auto getConstVal = [] { return FpAttr{g_const_val}; };
  auto getF8Scale = [] { return FpAttr{1.0}; };
  auto getIsReverse = [] { return g_is_reverse; };
  auto getMultiplier = [] { return g.multiplier; };
  auto getRshift = [] { return g.rshift; };
  auto getReluLimitAttr = [] { return LimitAttr{g_relu_limit}; };
#include "_ref/subconst.inc"
}
#include "_ref/to_intn.inc"
#define UNREACHABLE_THIS(msg) abort()
static int failure() { return 1; }
static std::string g_cast_to;
static int top_cast(InferenceParameter& p) {
  struct RmStr {
    std::string str() const { return ""; }
  };
  auto getRoundMode = [] { return RmStr{}; };
  auto round_mode_convert = [](const std::string&) { return (RoundingMode)g.round_mode; };
  auto getTo = [] { return g_cast_to; };
#include "_ref/top_cast.inc"
}

// ---------------------------------------------------------------------------------------------- tpu.Sub (int8), tpu.Reduce tail
static void sub_int8(InferenceParameter& p, int64_t num_elem) {
  auto out_type = g.out_type;
  {
#include "_ref/sub_int8.inc"
  }
}
struct OptArr {
  std::optional<std::vector<int64_t>> a;
  const std::optional<std::vector<int64_t>>& value() const { return a; }
};
static void reduce_tail(float* output_v, size_t num_elem, int64_t multiplier, int64_t rshift) {
  auto getRshift = [&] { return OptArr{std::vector<int64_t>{rshift}}; };
  auto getMultiplier = [&] { return OptArr{std::vector<int64_t>{multiplier}}; };
  {
#include "_ref/reduce_tail.inc"
  }
}

// ---------------------------------------------------------------------------------------------- C entry points
static void set_out_type(int width, int is_unsigned) {
  g.out_type.width = width;
  g.out_type.uns = is_unsigned != 0;
  g.out_type.is_int = true;
}

extern "C" {

long long ref_saturate_i64(long long v, int width, int is_unsigned) {
  set_out_type(width, is_unsigned);
  return saturate<long>((long)v, g.out_type);
}
long long ref_saturate_f32(float v, int width, int is_unsigned, int rmode) {
  set_out_type(width, is_unsigned);
  return saturate<float>(v, g.out_type, (RoundingMode)rmode);
}

// acc: fp32 accumulators [n][c][h*w], overwritten with the quantised values (as floats), like p.outputs[0]
void ref_conv2d_requant(float* acc, long long n, long long c, long long hw, const long long* rshift, int n_shift,
                        const long long* mult, int n_mult, const int* bias, int qmode, int do_relu, long long zp,
                        int out_width, int out_unsigned, int cv18xx) {
  g = Ctx();
  g.cv18xx = cv18xx != 0;
  g.qmode = (tpu::RequantMode)qmode;
  g.out_q.zp = zp;
  set_out_type(out_width, out_unsigned);
  InferenceParameter p;
  p.outputs.push_back(acc);
  std::vector<int64_t> rs(rshift, rshift + n_shift), mu(mult, mult + n_mult);
  // Conv2D.cpp:300-301: getI64Array(getMultiplier(), rshift_v->size(), 1)
  if (mu.empty()) mu.assign(rs.size(), 1);
  std::vector<int32_t> b(bias, bias + c);
  conv2d_requant(p, n, c, hw, 1, false, rs, mu, b, do_relu != 0);
}

// out: fp32 GEMM result (+bias, +relu) [batch*batch_low][M][N], overwritten; multi_operand: p.inputs[3] (fuse_rq) or null
void ref_matmul_requant(float* out, long long full_batch, long long M, long long N, const long long* rshifts, int n_rshifts,
                        const long long* multipliers, int n_multipliers, const float* multi_operand, int qmode,
                        int fuse_rq, double out_scale, long long zp, int out_width, int out_unsigned, int cv18xx,
                        int right_is_weight) {
  g = Ctx();
  g.cv18xx = cv18xx != 0;
  g.qmode = (tpu::RequantMode)qmode;
  g.fuse_rq = fuse_rq != 0;
  g.out_q.zp = zp;
  g.right_is_weight = right_is_weight != 0;
  g.batch = full_batch;
  g.batch_low = 1;
  g.M = M;
  g.N = N;
  g.out_shape = {full_batch, M, N};
  if (n_rshifts > 0) g.rshifts = std::vector<int64_t>(rshifts, rshifts + n_rshifts);
  if (n_multipliers > 0) g.multipliers = std::vector<int64_t>(multipliers, multipliers + n_multipliers);
  g.out_scales = std::vector<double>{out_scale};
  set_out_type(out_width, out_unsigned);
  InferenceParameter p;
  p.outputs.push_back(out);
  p.inputs.assign(5, nullptr);
  p.inputs[3] = const_cast<float*>(multi_operand);
  matmul_requant(p);
}

void ref_add_int8(const float* a, const float* b, float* out, long long count, long long m0, long long s0, long long m1,
                  long long s1, int do_relu, int out_width, int out_unsigned) {
  g = Ctx();
  g.multipliers = std::vector<int64_t>{m0, m1};
  g.rshifts = std::vector<int64_t>{s0, s1};
  g.out_shape = {count};
  set_out_type(out_width, out_unsigned);
  Binary bin;
  bin.dst = out;
  bin.count = count;
  bin.relu = do_relu != 0;
  InferenceParameter p;
  p.inputs = {const_cast<float*>(a), const_cast<float*>(b)};
  p.outputs = {out};
  p.handle = &bin;
  add_int8(p, count);
}

// avg: fp32 window averages (what the pooling primitive leaves in p.outputs[0]), overwritten
void ref_avgpool_int8(float* avg, long long count, int kh, int kw, int has_multiplier, long long multiplier, int has_rshift,
                      long long rshift, int do_relu, int out_width, int out_unsigned, int cv18xx) {
  g = Ctx();
  g.cv18xx = cv18xx != 0;
  g.do_relu = do_relu != 0;
  if (has_multiplier) g.pool_multiplier = multiplier;
  if (has_rshift) g.pool_rshift = rshift;
  set_out_type(out_width, out_unsigned);
  Pooling pool{kh, kw};
  InferenceParameter p;
  p.outputs = {avg};
  avgpool_int8(p, &pool, count);
}

// weight: N_out * K/2 float-stored bytes; scale / zp: float-stored, one per group; out: N_out * K floats
void ref_a16_dequant_w4(const float* weight, const float* scale, const float* zp, long long rows, long long k,
                        int q_group_size, float* out) {
  // the reference names the stored weight shape [K][N/2] before its swap for w_transpose (A16MatMul.cpp:172-173,:203)
  std::vector<float> nw((size_t)(rows * k), 0.f);
  a16_dequant(weight, scale, zp, (int)rows, (int)k, q_group_size, nw);
  memcpy(out, nw.data(), nw.size() * sizeof(float));
}

void ref_requant_int_axis(const float* x, const float* quant, float* out, const long long* shape, int rank, int qmode,
                          int round_mode, int fuse_rq_axis, int bm1684x, int in_quantized, long long in_zp, int out_width,
                          int out_unsigned) {
  g = Ctx();
  g.qmode = (tpu::RequantMode)qmode;
  g.round_mode = round_mode;
  g.fuse_rq_axis = fuse_rq_axis != 0;
  g.bm1684x = bm1684x != 0;
  g.in_quantized = in_quantized != 0;
  g.in_q.zp = in_zp;
  g.out_shape.assign(shape, shape + rank);
  set_out_type(out_width, out_unsigned);
  InferenceParameter p;
  p.inputs = {const_cast<float*>(x), const_cast<float*>(quant)};
  p.outputs = {out};
  requant_int_axis(p);
}

void ref_requant_int(const float* x, float* out, const long long* shape, int rank, long long multiplier, long long rshift,
                     int qmode, int round_mode, int in_quantized, long long in_zp, long long out_zp, int out_width,
                     int out_unsigned) {
  g = Ctx();
  g.qmode = (tpu::RequantMode)qmode;
  g.round_mode = round_mode;
  g.multiplier = multiplier;
  g.rshift = rshift;
  g.in_quantized = in_quantized != 0;
  g.in_q.zp = in_zp;
  g.out_q.zp = out_zp;
  g.out_shape.assign(shape, shape + rank);
  set_out_type(out_width, out_unsigned);
  InferenceParameter p;
  p.inputs = {const_cast<float*>(x)};
  p.outputs = {out};
  requant_int(p);
}

float ref_cast_requant(float v, double scale, long long zp, int expressed) {
  QType q;
  q.scale = scale;
  q.zp = zp;
  q.expressed = expressed;
  return tpu_mlir::requant(v, q);
}
float ref_cast_dequant(float v, double scale, long long zp, int expressed) {
  QType q;
  q.scale = scale;
  q.zp = zp;
  q.expressed = expressed;
  return tpu_mlir::dequant(v, q);
}

void ref_requant_fp(float* x, float* y, long long n, double scale, double offset, int qmode, int round_mode, int width, int is_unsigned,
                    long long out_zp) {
  set_out_type(width, is_unsigned);
  g.out_shape = {(int64_t)n};
  g.out_q.zp = out_zp;
  g.qmode = (tpu::RequantMode)qmode;
  g.round_mode = round_mode;
  g_fp_scale = scale;
  g_fp_offset = offset;
  InferenceParameter p;
  p.inputs = {x};
  p.outputs = {y};
  requant_fp(p);
}

void ref_maxmin_const(int is_max, float* x, float* y, long long n, double izp, float const_val, long long multiplier, long long rshift,
                      int do_relu, int width, int is_unsigned) {
  set_out_type(width, is_unsigned);
  g.multiplier = multiplier;
  g.rshift = rshift;
  g.do_relu = do_relu != 0;
  InferenceParameter p;
  p.inputs = {x};
  p.outputs = {y};
  if (is_max) maxconst_q(p, n, izp, const_val);
  else minconst_q(p, n, izp, const_val);
}

void ref_prelu_int8(float* x, float* slope, float* y, long long num_outer, long long num_inner, long long num_slope, long long shift, int width,
                    int is_unsigned) {
  set_out_type(width, is_unsigned);
  InferenceParameter p;
  p.inputs = {x, slope};
  p.outputs = {y};
  prelu_q(p, num_outer, num_inner, num_slope, shift);
}

void ref_subconst(float* x, float* y, long long n, double const_val, int is_reverse, long long multiplier, long long rshift, int do_relu,
                  double relu_limit, int width, int is_unsigned) {
  set_out_type(width, is_unsigned);
  g.out_shape = {(int64_t)n};
  g.multiplier = multiplier;
  g.rshift = rshift;
  g.do_relu = do_relu != 0;
  g_const_val = const_val;
  g_is_reverse = is_reverse != 0;
  g_relu_limit = relu_limit;
  module::g_module_asym = false;
  InferenceParameter p;
  p.inputs = {x};
  p.outputs = {y};
  subconst(p);
}

void ref_top_cast(float* x, float* y, long long n, const char* to, int round_mode) {
  g.out_shape = {(int64_t)n};
  g.round_mode = round_mode;
  g_cast_to = to;
  InferenceParameter p;
  p.inputs = {x};
  p.outputs = {y};
  top_cast(p);
}

void ref_sub_int8(const float* a, const float* b, float* out, long long count, long long m0, long long s0, long long m1, long long s1,
                  int do_relu, int out_width, int out_unsigned) {
  g = Ctx();
  g.multipliers = std::vector<int64_t>{m0, m1};
  g.rshifts = std::vector<int64_t>{s0, s1};
  g.out_shape = {count};
  set_out_type(out_width, out_unsigned);
  Binary bin;
  bin.dst = out;
  bin.count = count;
  bin.relu = do_relu != 0;
  bin.sub = true;
  InferenceParameter p;
  p.inputs = {const_cast<float*>(a), const_cast<float*>(b)};
  p.outputs = {out};
  p.handle = &bin;
  sub_int8(p, count);
}

void ref_reduce_tail(float* values, long long count, long long multiplier, long long rshift) { reduce_tail(values, (size_t)count, multiplier, rshift); }

}  // extern "C"
