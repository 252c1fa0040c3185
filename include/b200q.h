/*
 * b200q — C ABI of the B200 (sm_100a) backend for tpu-mlir's quantized-inference hot path.
 *
 * Two faces:
 *   (1) the operator face mirrors the interpreter's per-op interface
 *       (init / inference / deinit over an InferenceParameter of host float buffers,
 *       include/tpu_mlir/Interfaces/InferenceInterface.td:16-58, InferenceInterface.h:15-19):
 *       inputs[i] / outputs[i] are HOST float* in operand order, integer tensors stored as
 *       integral floats exactly as ModuleInterpreter keeps them; attributes that the reference
 *       reads from the MLIR op arrive in a plain descriptor struct.
 *   (2) the device face takes native-dtype DEVICE pointers and a CUDA stream and is asynchronous;
 *       it is what a GPU-resident executor (the role of bindings/pymlir/pycuda.cpp) calls.
 *
 * All functions return B200Q_OK (0) or a negative b200q_status; b200q_last_error() gives the
 * message of the calling thread's last failure.  Nothing here aborts, exits or falls back to the CPU.
 * Paths in the comments are paths inside the tpu-mlir source tree.
 *
 * Threads and streams.  The reference walks a graph on one interpreter thread (ModuleInterpreter.cpp:957-965) and
 * only reads tensors from a small thread pool after invoke has returned (kld_calibrator.py:606-615); this library
 * assumes the same.  The operator face runs on the legacy default stream (and, for Conv2D, on three streams private
 * to the handle), is synchronous (results are in the output buffers on return) and synchronises the default stream
 * first, so work the caller queued there is finished before it starts.  A handle (the void* of init / dev_create,
 * a calibration context) holds staging buffers and device-side status words that every call on it reuses: calls on
 * ONE handle must not overlap, whichever threads make them; calls on DIFFERENT handles may run from different
 * threads at the same time.  The device face is asynchronous on the stream it is given; two calls on one handle are
 * ordered by issuing them on the same stream (or by the caller's events).  b200q_last_error() is per thread.
 */
#ifndef B200Q_H_
#define B200Q_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  B200Q_OK = 0,
  B200Q_ERR_INVALID = -1,     /* bad argument / descriptor */
  B200Q_ERR_UNSUPPORTED = -2, /* valid in the reference but not implemented by this backend */
  B200Q_ERR_CUDA = -3,        /* a CUDA call failed */
  B200Q_ERR_NO_DEVICE = -4,   /* no sm_100 device */
  B200Q_ERR_TIMEOUT = -5,     /* a bounded device-side wait ran out */
  B200Q_ERR_NOMEM = -6
} b200q_status;

/* tpu::RequantMode, include/tpu_mlir/Dialect/Tpu/IR/TpuOps.td:160-172 (same numbering) */
typedef enum {
  B200Q_QM_TFLITE_LSHIFT = 0,
  B200Q_QM_TFLITE = 1,
  B200Q_QM_MULTIPLIER_SHIFT = 2,
  B200Q_QM_ONLY_SHIFT = 3,
  B200Q_QM_QDM = 4,
  B200Q_QM_ONLY_SCALE = 5
} b200q_requant_mode;

/* RoundingMode, include/tpu_mlir/Support/MathUtils.h:28-42 (same numbering) */
typedef enum {
  B200Q_ROUND_HALF_AWAY_FROM_ZERO = 0,
  B200Q_ROUND_HALF_UP = 1,
  B200Q_ROUND_HALF_DOWN = 2,
  B200Q_ROUND_HALF_TO_EVEN = 3,
  B200Q_ROUND_HALF_TO_ODD = 4,
  B200Q_ROUND_HALF_TOWARDS_ZERO = 5,
  B200Q_ROUND_TOWARDS_ZERO = 6,
  B200Q_ROUND_AWAY_FROM_ZERO = 7,
  B200Q_ROUND_UP = 8,
  B200Q_ROUND_DOWN = 9
} b200q_round_mode;

/* storage type of a tensor on the device face (module::getStorageType in the reference) */
typedef enum {
  B200Q_DT_I8 = 0,
  B200Q_DT_U8 = 1,
  B200Q_DT_I16 = 2,
  B200Q_DT_U16 = 3,
  B200Q_DT_I32 = 4,
  B200Q_DT_F32 = 5,
  B200Q_DT_BF16 = 6,
  B200Q_DT_F16 = 7
} b200q_dtype;

/* The arithmetic form a (RequantMode, chip family, op) triple resolves to on the device face;
 * lib/Support/MathUtils.cpp:538-562.  `shift` below is the per-form shift operand. */
typedef enum {
  B200Q_RQ_NONE = 0,                 /* raw int32 accumulator out */
  B200Q_RQ_MULTIPLIER_SHIFT = 1,     /* RightShiftRound(acc*M, shift, round): shift > 0 right, < 0 left */
  B200Q_RQ_QDM = 2,                  /* MultiplyByQuantizedMultiplier(acc, M, shift, round): shift > 0 LEFT, < 0 right */
  B200Q_RQ_MULTIPLIER_SHIFT_F32 = 3, /* CV18xx MultiplierShift: to_int((float)acc*M / (1<<shift), round) */
  B200Q_RQ_ONLY_SHIFT = 4,           /* RightShiftRound(acc, shift, round) */
  B200Q_RQ_ONLY_SCALE = 5            /* (int32)roundf(acc * scale) */
} b200q_rq_dialect;

typedef enum {
  B200Q_RELU_NONE = 0,
  B200Q_RELU_BEFORE_REQUANT = 1, /* MatMul order: max(acc+bias, 0) then requant (MatMul.cpp:599-603) */
  B200Q_RELU_AFTER_REQUANT = 2   /* Conv2D order: max(requant+zp, zp) (Conv2D.cpp:334-336) */
} b200q_relu_order;

/* Epilogue of the device face: out = saturate(relu(requant(acc + bias[c]) + out_zp)).
 * All pointers are DEVICE pointers. */
typedef struct {
  int32_t dialect;           /* b200q_rq_dialect */
  int32_t round_mode;        /* b200q_round_mode */
  int32_t per_channel;       /* 1: multiplier[c], shift[c]; 0: multiplier[0], shift[0] */
  int32_t out_zp;
  int32_t relu;              /* b200q_relu_order */
  int32_t out_dtype;         /* I8 / U8 / I16 / U16 / I32 */
  float scale;               /* B200Q_RQ_ONLY_SCALE */
  const int32_t *bias;       /* [C] or NULL */
  const int32_t *multiplier; /* [C] or [1] */
  const int32_t *shift;      /* [C] or [1] */
} b200q_epilogue;

/* ------------------------------------------------------------------ library */
const char *b200q_version(void);
const char *b200q_last_error(void);
/* number of sm_100 devices visible; 0 is not an error */
int b200q_device_count(void);

/* ------------------------------------------------------------------ tpu.MatMul (INT8)
 * Descriptor = the attributes tpu::MatMulOp::parseParam derives (matmul_attr_t,
 * include/tpu_mlir/Support/AttrStruct.h:82-101) plus the requant attributes of the op
 * (include/tpu_mlir/Dialect/Tpu/IR/TpuOps.td:4592-4616). */
typedef struct {
  int64_t batch, M, K, N;
  int32_t with_bias, do_relu;
  int32_t right_transpose;   /* right operand stored [N,K] instead of [K,N] */
  int32_t left_transpose, output_transpose; /* input stored [batch][K][M] / output stored [batch][N][M] */
  int32_t hdim_is_batch;                    /* batch x batch_low independent products; a transposed operand / output keeps
                                             * batch_low between its matrix dimensions (see batch_low) */
  int32_t right_batched;     /* right operand has the batch dimension (activation x activation) */
  int32_t right_is_weight;   /* constant right operand: uploaded once per (handle, weight_version) */
  int32_t weight_version;    /* bump after rewriting the weight buffers in place */
  int32_t input_zp, right_zp;
  int32_t input_dtype, right_dtype, out_dtype; /* b200q_dtype: I8/U8 (out also I16/U16/I32) */
  int32_t quant_mode;        /* b200q_requant_mode */
  int32_t is_cv18xx;         /* module::isCV18xx(): per-batch requant, half-away rounding, no zero point */
  int32_t fuse_rq;           /* per-channel multipliers arrive float-stored in operand 3 (MatMul.cpp:709-716) */
  int32_t out_zp;
  int32_t n_quant;           /* entries of multipliers / rshifts */
  const int64_t *multipliers;
  const int64_t *rshifts;
  double out_scale;          /* B200Q_QM_ONLY_SCALE */
  int32_t algo;              /* 0 = auto, 1 = tensor cores only, 2 = CUDA cores only */
  int64_t batch_low;         /* matmul_attr_t::batch_low, read with hdim_is_batch (0 = 1).  The layouts are those of
                              * lib/Support/Dnnl/MatMul.cpp:172-241: left_transpose: input [batch][M][batch_low][K];
                              * right_transpose: right [batch][K][batch_low][N]; output_transpose: output
                              * [batch][M][batch_low][N]; an operand without its flag is [batch*batch_low][rows][cols]. */
} b200q_matmul_desc;

/* Operator face of tpu::MatMulOp::{init,inference,deinit}
 * (lib/Dialect/Tpu/Interfaces/Common/MatMul.cpp:400-440,:440-733).  inputs = {input, right, bias, multi,
 * buffer} as HOST float*, NULL for absent operands (ModuleInterpreter.cpp:456-458); outputs[0] HOST float*.
 * Like the reference, inference accepts *handle == NULL (it then sets up and tears down its own state). */
int b200q_matmul_init(const b200q_matmul_desc *desc, void **handle);
int b200q_matmul_inference(const b200q_matmul_desc *desc, float *const *inputs, int n_inputs,
                           float *const *outputs, int n_outputs, void **handle);
void b200q_matmul_deinit(void **handle);

/* Device face: out[M,N] = epilogue(A[M,K] * B^T) with B given K-major as [N,K]; native dtypes, device
 * pointers, asynchronous on `stream` (a cudaStream_t).  a_dtype / b_dtype are B200Q_DT_I8 or _U8.
 * `status` is an optional device int that receives a non-zero code if a bounded wait in the kernel ran out.
 * Replaces MatMul::run (lib/Support/Dnnl/MatMul.cpp:223-241) + the requant loop (MatMul.cpp:636-728). */
int b200q_gemm_i8_dev(const void *a, int a_dtype, const void *b_nk, int b_dtype, int64_t M, int64_t N, int64_t K,
                      const b200q_epilogue *epilogue, void *out, int32_t *status, int algo, void *stream);
/* The same product with operand zero points subtracted first, (A - input_zp) * (B - right_zp)^T, as
 * lib/Support/Dnnl/MatMul.cpp:193-205 does before the product; non-zero zero points take the CUDA-core kernel. */
int b200q_gemm_i8_zp_dev(const void *a, int a_dtype, const void *b_nk, int b_dtype, int64_t M, int64_t N, int64_t K,
                         int32_t input_zp, int32_t right_zp, const b200q_epilogue *epilogue, void *out, int32_t *status,
                         int algo, void *stream);

/* ------------------------------------------------------------------ tpu.Conv2D (INT8)
 * conv_attr_t (include/tpu_mlir/Support/AttrStruct.h:15-43) + the requant attributes of tpu.Conv2D
 * (TpuOps.td:1557-1595).  NCHW activations, OIHW filter, like module::getNCHW (Conv2D.cpp:19-72). */
typedef struct {
  int64_t n, ic, ih, iw, oc, kh, kw, sh, sw, dh, dw, pht, phb, pwl, pwr, groups;
  int32_t pad_value;         /* input zero point used for padding */
  int32_t with_bias, do_relu;
  int32_t input_dtype, out_dtype;
  int32_t quant_mode;        /* b200q_requant_mode */
  int32_t is_cv18xx;
  int32_t out_zp;
  int32_t n_quant;           /* oc (per-axis) or 1 */
  const int64_t *multipliers; /* I64 array attribute `multiplier` (Conv2D.cpp:299-301) */
  const int64_t *rshifts;     /* I64 array attribute `rshift` */
  int32_t weight_version;
  int32_t algo;              /* 0 = auto, 1 = tensor cores only, 2 = CUDA cores only */
} b200q_conv2d_desc;

/* Operator face of tpu::Conv2DOp::{init,inference,deinit} (Conv2D.cpp:74-86,:88-344).
 * inputs = {input, filter, bias} HOST float*; outputs[0] HOST float*.  init uploads and repacks the filter
 * and bias; inference requires a handle (Conv2D.cpp:89-91 fails without one).  Unlike the reference the
 * bias buffer is NOT zeroed in place (Conv2D.cpp:94-99 mutates its input).  The handle keeps its device copy of
 * the filter until inference is called with a descriptor whose weight_version differs from the one the copy was made
 * with, or with another filter pointer (the interpreter rewrites filters in place: setTensor, fake_quant_weight,
 * ModuleInterpreter.cpp:583-612); then filter and bias are uploaded and repacked again.  A NULL descriptor keeps
 * the copy. */
int b200q_conv2d_init(const b200q_conv2d_desc *desc, float *const *inputs, int n_inputs, void **handle);
int b200q_conv2d_inference(const b200q_conv2d_desc *desc, float *const *inputs, int n_inputs,
                           float *const *outputs, int n_outputs, void **handle);
void b200q_conv2d_deinit(void **handle);

/* Device face: prepare once (filter s8 OIHW and bias s32 are DEVICE pointers and are repacked into the
 * handle), then run on native NCHW device tensors, asynchronous on `stream`.  b200q_conv2d_dev_status
 * synchronises the stream and reports a kernel-side timeout, if any.
 * Replaces Conv::run (lib/Support/Dnnl/Conv.cpp:234-253) + the requant loop (Conv2D.cpp:295-341). */
int b200q_conv2d_dev_create(const b200q_conv2d_desc *desc, const void *filter_oihw_s8, const int32_t *bias_s32,
                            void **handle);
int b200q_conv2d_dev_run(void *handle, const void *x_nchw, void *y_nchw, void *stream);
/* The same run with the activation layouts named: B200Q_LAYOUT_NHWC tensors are [N][H][W][C] bytes (channels a
 * multiple of 16, 16-byte aligned).  A graph that keeps its activations channels-last between ops runs no
 * transposing kernel: a 1x1 stride-1 filter reads x in place, other filters copy it into the zero-bordered
 * image, and the output is stored as whole channel runs.  Only the tensor-core routes take NHWC tensors
 * (B200Q_ERR_UNSUPPORTED otherwise).  The values are those of b200q_conv2d_dev_run, permuted. */
enum { B200Q_LAYOUT_NCHW = 0, B200Q_LAYOUT_NHWC = 1 };
int b200q_conv2d_dev_run_layout(void *handle, const void *x, int32_t x_layout, void *y, int32_t y_layout, void *stream);
/* The same run with the tpu.Add that consumes the convolution's output fused into the kernel (a residual connection:
 * Add.cpp:177-207, symmetric 8-bit form).  `residual` is the Add's other operand, a device tensor of the output's shape
 * in the output's layout; y receives clamp(((v * conv_multiplier + 2^(conv_rshift-1)) >> conv_rshift) +
 * ((r * residual_multiplier + 2^(residual_rshift-1)) >> residual_rshift)) in `out_dtype` (with do_relu the lower bound
 * is 0), where v is the convolution's own requantised, saturated output, which is not stored.  Multipliers below 2^23
 * in magnitude and shifts in [1,31] (what the lowering emits; B200Q_ERR_UNSUPPORTED otherwise, also for the CUDA-core
 * route).  The values are those of b200q_conv2d_dev_run_layout followed by b200q_add_i8_dev. */
typedef struct b200q_fused_add {
  const void *residual;
  int32_t residual_dtype;                       /* B200Q_DT_I8 / B200Q_DT_U8 */
  int32_t conv_multiplier, conv_rshift;         /* the Add's pair for the operand that is this convolution's output */
  int32_t residual_multiplier, residual_rshift; /* the Add's pair for the other operand */
  int32_t do_relu;
  int32_t out_dtype;                            /* the Add's output type, B200Q_DT_I8 / B200Q_DT_U8 */
} b200q_fused_add;
int b200q_conv2d_dev_run_add(void *handle, const void *x, int32_t x_layout, void *y, int32_t y_layout,
                             const b200q_fused_add *add, void *stream);
/* Which kernels serve this handle: 1 = tensor cores on the (bordered) channels-last image, 2 = tensor cores on
 * gathered im2col rows, 0 = the CUDA-core kernel (groups, dilation, odd channel counts); negative = error. */
int b200q_conv2d_dev_route(void *handle);
int b200q_conv2d_dev_status(void *handle, void *stream);
void b200q_conv2d_dev_destroy(void **handle);
/* Optional timing of the device face: while enabled, every b200q_conv2d_dev_run records CUDA events on its
 * stream before the layout kernel, between the two kernels and after the tensor-core kernel (no host
 * synchronisation).  b200q_conv2d_dev_profile waits for the recorded runs and returns their number and the
 * summed durations in milliseconds; enabling again starts a new measurement.  (No counterpart in the
 * reference, whose CUDA path is untimed.) */
int b200q_conv2d_dev_set_profiling(void *handle, int enable);
int b200q_conv2d_dev_profile(void *handle, int64_t *runs, double *layout_ms_total, double *kernel_ms_total);

/* ------------------------------------------------------------------ tpu.RequantIntAxis / tpu.RequantInt
 * Operator face of tpu::RequantIntAxisOp::inference (lib/Dialect/Tpu/Interfaces/Common/RequantIntAxis.cpp:17-123,
 * BM1684X quant layout {multiplier, shift, zero point} x C in operand 1, float-stored) and, with per_axis = 0,
 * of tpu::RequantIntOp::inference (RequantInt.cpp:17-71: multiplier / rshift attributes, output zero point).
 * The tensor is viewed [outer][channels][inner]; with fuse_rq_axis the channel is the last axis (inner = 1). */
typedef struct {
  int64_t outer, channels, inner;
  int32_t per_axis;       /* 1: RequantIntAxis (quant operand), 0: RequantInt (attributes below) */
  int32_t quant_mode;     /* TFLite / TFLite_LShift / MultiplierShift */
  int32_t round_mode;     /* b200q_round_mode (the op's round_mode attribute) */
  int32_t fuse_rq_axis;
  int32_t in_zp;          /* input zero point (MultiplierShift only) */
  int32_t out_dtype;
  int64_t multiplier, rshift; /* RequantInt attributes */
  int32_t out_zp;             /* RequantInt: zero point of the output type */
  int32_t quant_words;        /* RequantIntAxis: words per channel of the quant operand: 3 = {multiplier, shift, zero
                               * point} (BM1684X, RequantIntAxis.cpp:45-48; also meant by 0), 2 = {multiplier, shift in
                               * the low byte | zero point in the high half-word} (every other chip, :49-54) */
} b200q_requant_desc;
int b200q_requant_int_axis_inference(const b200q_requant_desc *desc, float *const *inputs, int n_inputs,
                                     float *const *outputs, int n_outputs);

/* ------------------------------------------------------------------ glue ops of an INT8 graph, device face
 * Native NCHW device tensors, asynchronous on `stream`. */
/* x int32 [outer][C][inner]; per channel multiplier / shift (sign convention of `dialect`) / zero point. */
int b200q_requant_int_axis_dev(const int32_t *x, int64_t outer, int64_t C, int64_t inner, const int32_t *multiplier,
                               const int32_t *shift, const int32_t *zero_point, int32_t dialect, int32_t round_mode,
                               int32_t in_zp, int32_t out_dtype, void *out, void *stream);
/* tpu.Add, symmetric int8 (lib/Dialect/Tpu/Interfaces/Common/Add.cpp:177-207):
 * out = saturate(relu(RSR(a*m0, s0, half-up) + RSR(b*m1, s1, half-up))). */
int b200q_add_i8_dev(const void *a, int32_t a_dtype, const void *b, int32_t b_dtype, int64_t count, int32_t m0,
                     int32_t s0, int32_t m1, int32_t s1, int32_t do_relu, int32_t out_dtype, void *out, void *stream);
/* tpu.MaxConst (form 0) / tpu.MinConst (1) with a uniform-quantized output (MaxConst.cpp:27-42): the float (x - in_zp) * multiplier is
 * compared with float(const_val), cut to an integer toward zero, shifted half-up by rshift, ReLU'd and saturated (no output
 * zero point is added, as there).  tpu.SubConst, symmetric (SubConst.cpp:26-112): form 2 float(x * multiplier - const_val),
 * form 3 (is_reverse) float(const_val - x * multiplier), the ReLU (with its limit) on that float, then the same cut, shift,
 * ReLU and saturation. */
int b200q_constop_i8_dev(int32_t form, const void *x, int32_t dtype, int64_t count, int32_t multiplier, double const_val,
                         int32_t rshift, int32_t in_zp, int32_t do_relu, float relu_limit, int32_t out_dtype, void *out,
                         void *stream);
/* tpu.Sub, symmetric 8-bit operands of equal shape (lib/Dialect/Tpu/Interfaces/Common/Sub.cpp:88-113):
 * out = saturate(relu(RSR(a*m0, s0, half-up) - RSR(b*m1, s1, half-up))). */
int b200q_sub_i8_dev(const void *a, int32_t a_dtype, const void *b, int32_t b_dtype, int64_t count, int32_t m0, int32_t s0,
                     int32_t m1, int32_t s1, int32_t do_relu, int32_t out_dtype, void *out, void *stream);
/* tpu.Lut (lib/Dialect/Tpu/Interfaces/Common/Lut.cpp:20-32): out[i] = table[x[i] mod 256] (a negative int8 index
 * wraps by +256).  x is 8-bit; `table` holds 256 entries of `table_dtype`, which is also the output type. */
int b200q_lut_dev(const void *x, int64_t count, const void *table, int32_t table_dtype, void *out, void *stream);
/* tpu.MulShift (MulShift.cpp:19-41): out = saturate(RSR((x - in_zp) * multiplier, rshift, half-up) + out_zp). */
int b200q_mulshift_i8_dev(const void *x, int32_t dtype, int64_t count, int32_t multiplier, int32_t rshift,
                          int32_t in_zp, int32_t out_zp, int32_t out_dtype, void *out, void *stream);
/* tpu.AddConst with a uniform-quantized output (lib/Dialect/Tpu/Interfaces/Common/AddConst.cpp:26-47):
 * out = saturate(relu(RSR((x - in_zp) * multiplier + const_val, rshift, half-up))); with const_val = 0 and in_zp = 0 it is the
 * symmetric tpu.MulConst (MulConst.cpp:50-62). */
int b200q_addconst_i8_dev(const void *x, int32_t dtype, int64_t count, int32_t multiplier, double const_val, int32_t rshift,
                          int32_t in_zp, int32_t do_relu, int32_t out_dtype, void *out, void *stream);
/* tpu.RequantFp to an integer type (lib/Dialect/Tpu/Interfaces/Common/RequantFp.cpp:17-66): x is f32, or int32 converted to
 * float the way the reference's interpreter stores it.  TFLite / TFLite_LShift: saturate(to_int(x * scale) + out_zp);
 * MultiplierShift: saturate(to_int(x * scale + offset)).  The 8-bit float outputs of OnlyScale are not implemented. */
int b200q_requant_fp_dev(const void *x, int32_t dtype, int64_t count, double scale, double offset, int32_t out_zp,
                         int32_t quant_mode, int32_t round_mode, int32_t out_dtype, void *out, void *stream);
/* tpu.PRelu (lib/Dialect/Tpu/Interfaces/Common/PRelu.cpp:35-88); slope index c = (i / inner) % num_slope.  f32 -> f32 with
 * float slopes: x > 0 ? x : x * slope[c].  8-bit -> 8-bit (symmetric) with int8 slopes: x < 0 becomes
 * saturate(RSR(x * slope[c], rshift, half-up)), other values pass through. */
int b200q_prelu_dev(const void *x, int32_t dtype, const void *slope, int64_t count, int64_t inner, int32_t num_slope,
                    int32_t rshift, int32_t out_dtype, void *out, void *stream);
/* tpu.Mul, symmetric int8 operands of equal shape (Mul.cpp:23-29,:72-85): the op's ReLU acts on the product, then
 * out = saturate(RSR(product * multiplier, rshift, half-up)).  Broadcasting operands are not implemented. */
int b200q_mul_i8_dev(const void *a, int32_t a_dtype, const void *b, int32_t b_dtype, int64_t count,
                     int32_t multiplier, int32_t rshift, int32_t do_relu, int32_t out_dtype, void *out, void *stream);
/* tpu.Pool2D int8 (Pool2D.cpp:160-192): max, or average as RSR(window_sum * multiplier, rshift, half-up);
 * x is [nc][ih][iw] (N and C merged). */
int b200q_pool2d_i8_dev(const void *x, int32_t dtype, int64_t nc, int32_t ih, int32_t iw, int32_t kh, int32_t kw,
                        int32_t sh, int32_t sw, int32_t pht, int32_t phb, int32_t pwl, int32_t pwr, int32_t is_avg,
                        int32_t multiplier, int32_t rshift, int32_t do_relu, int32_t out_dtype, void *out, void *stream);
/* The same op on a channels-last tensor x [n][ih][iw][c] -> out [n][oh][ow][c] (max pooling: equal 8-bit types,
 * c a multiple of 16, 16-byte aligned buffers). */
int b200q_pool2d_i8_nhwc_dev(const void *x, int32_t dtype, int64_t n, int32_t c, int32_t ih, int32_t iw, int32_t kh,
                             int32_t kw, int32_t sh, int32_t sw, int32_t pht, int32_t phb, int32_t pwl, int32_t pwr,
                             int32_t is_avg, int32_t multiplier, int32_t rshift, int32_t do_relu, int32_t out_dtype,
                             void *out, void *stream);
/* tpu.Cast f32 <-> int8/uint8 (Cast.cpp:75-116, lib/Support/CastUtils.cpp:15-47):
 * q = saturate(to_int(round(x * (float)(1/scale)) + zp, round_mode));  x = (float)scale * (q - zp). */
int b200q_cast_f32_to_q8_dev(const float *x, int64_t count, double scale, int32_t zero_point, int32_t round_mode,
                             int32_t out_dtype, void *out, void *stream);
int b200q_cast_q8_to_f32_dev(const void *x, int32_t dtype, int64_t count, double scale, int32_t zero_point, float *out,
                             void *stream);

/* ------------------------------------------------------------------ tpu.A16MatMul (w4 bf16)
 * Attributes of tpu.A16MatMul (TpuOps.td:495-530) for the static 4-bit path of
 * tpu::A16MatMulOp::inference (lib/Dialect/Tpu/Interfaces/Common/A16MatMul.cpp:171-208,:240-246):
 * weight bytes [N, K/2] (w_transpose = true), even k in the low nibble, one bf16 scale and one uint8 zero
 * point per q_group_size consecutive k of a row: W[n,k] = (q - zp) * scale. */
typedef struct {
  int64_t M, K, N;
  int32_t weight_bits;    /* 4; 8 (weight [N, K] one value per float, dequantised weight rounded to bf16, or to f16 in an
                           * F16 mode, as A16MatMul.cpp:213-232 does) */
  int32_t q_group_size;   /* weights per scale / zero point along k; 0 = one per output channel (A16MatMul.cpp:176-187) */
  int32_t w_transpose;    /* 1 */
  int32_t with_bias;
  int32_t out_dtype;      /* B200Q_DT_BF16 (w4bf16, w8bf16) or B200Q_DT_F16 (w4f16, w8f16): the type of input, scale and output */
  int32_t weight_version; /* bump after rewriting the weight buffers in place */
} b200q_a16matmul_desc;

/* Operator face of tpu::A16MatMulOp::{init,inference,deinit} (A16MatMul.cpp:16-22,:22-249).
 * inputs = {input, weight, scale, zp, bias} HOST float* (every one float-stored, like the interpreter's
 * buffers); outputs[0] HOST float* holding bf16-representable values. */
int b200q_a16matmul_init(const b200q_a16matmul_desc *desc, void **handle);
int b200q_a16matmul_inference(const b200q_a16matmul_desc *desc, float *const *inputs, int n_inputs,
                              float *const *outputs, int n_outputs, void **handle);
void b200q_a16matmul_deinit(void **handle);

/* Device face: x bf16 [M,K], wq bytes [N,K/2], scale bf16 [N*K/group], zp uint8 [N*K/group] (each <= 127),
 * bias f32 [N] or NULL, y bf16 [M,N]; asynchronous on `stream`.  `status` is an optional device int that
 * receives a non-zero code if a bounded wait in the kernel ran out.  Replaces the per-call fp32
 * dequantisation and sgemm of A16MatMul.cpp:171-208. */
int b200q_a16_w4_dev(const void *x_bf16, const void *wq, const void *scale_bf16, const void *zp_u8,
                     const float *bias_f32, void *y_bf16, int64_t M, int64_t N, int64_t K, int32_t group,
                     int32_t *status, void *stream);

/* The same call with the 16-bit type named: dtype = B200Q_DT_BF16 (w4bf16) or B200Q_DT_F16 (w4f16: x, scale and y are
 * IEEE half, the output is rounded to nearest even like F16(), lib/Support/Float16.cpp:763-767).  The f16 form runs the
 * CUDA-core kernel for one token (two where its shape limits allow) and the fused tensor-core kernel (kind::f16 on f16
 * operands) for everything else. */
int b200q_a16_w4_dev_dt(const void *x, const void *wq, const void *scale, const void *zp_u8, const float *bias_f32,
                        void *y, int64_t M, int64_t N, int64_t K, int32_t group, int32_t dtype, int32_t *status,
                        void *stream);

/* Test aid (no counterpart in the reference): makes a bounded wait of the tensor-core INT8 GEMM/convolution kernel run
 * out without faulting anything.  While extra_tx_bytes > 0 every pipeline stage's barrier expects that many bytes more
 * than the stage's loads deliver, so the consumer's wait ends after `budget_ns` (0 = the default of 2 s) with the
 * kernel's status set to the wait site; the calls then return B200Q_ERR_TIMEOUT and leave the context usable.
 * (0, 0) restores normal operation.  Process-wide; not for use while other threads launch. */
void b200q_debug_set_wait_fault(int32_t extra_tx_bytes, int64_t budget_ns);

/* Tensor-pipe peak probe (a measuring aid; no counterpart in the reference): every SM issues tcgen05.mma on operand
 * tiles resident in its shared memory and nothing else.  kind 0 = kind::i8 (s8 x s8 -> s32), 1 = kind::f16 on bf16
 * operands (f32 accumulate); pair != 0 uses cta_group::2 (256 x 256 x 32-byte MMAs over two SMs) instead of 128 x 256.
 * `launches` kernels of `kblocks` k-blocks (four MMAs each, a multiple of 8) per CTA run back to back on `stream`
 * inside one event pair; *ms receives the elapsed milliseconds and *ops the operations (2 x multiply-accumulates)
 * issued in that time.  Synchronises the stream.  B200Q_ERR_TIMEOUT if a wait inside the kernel ran out. */
int b200q_probe_tensor_peak(int32_t kind, int32_t pair, int32_t kblocks, int32_t launches, double *ms, double *ops,
                            void *stream);

/* Which kernel serves b200q_a16_*, process-wide: 0 = chosen per call (default: up to 8 tokens take the
 * decode kernels, and 9 to 16 tokens two launches of them where their shared-memory-resident form applies; a handle
 * that sees 64 tokens or more dequantises once into a bf16 copy and runs a bf16 GEMM;
 * everything else takes the fused-dequantisation tensor-core kernel on the packed weights); 1 = the decode kernels
 * only (8 tokens per launch); 2 = the fused tensor-core kernel for every M; 3 = handle API with M > 8: the bf16 copy
 * (rounds the weight to bf16, which the reference does not); 4 = the warpgroup kernel (up to 32 tokens: every lane
 * dequantises its own output channel into tensor memory as an exact hi + lo pair; measured no faster than the default
 * routes, kept for comparison).  A measuring control; no counterpart in the reference. */
void b200q_a16_set_route(int32_t route);

/* Device face with a handle: the tensors stay the caller's (not copied) and are declared constant for the life of
 * the handle (the decode kernel may request weights before the previous kernel of the stream has finished).  M <= 8
 * runs the decode kernels on the packed weights, M < 64 the fused tensor-core kernel on the packed weights; from 64
 * tokens on the weight is dequantised once into bf16 (kept in the handle, N*K*2 bytes) for a bf16 tensor-core GEMM
 * with fp32 accumulation.  b200q_a16_dev_status synchronises the stream and reports a kernel-side timeout. */
int b200q_a16_dev_create(const void *wq, const void *scale_bf16, const void *zp_u8, const float *bias_f32,
                         int64_t N, int64_t K, int32_t group, void **handle);
int b200q_a16_dev_create_dt(const void *wq, const void *scale, const void *zp_u8, const float *bias_f32, int64_t N,
                            int64_t K, int32_t group, int32_t dtype, void **handle); /* dtype: B200Q_DT_BF16 / _F16 */
int b200q_a16_dev_run(void *handle, const void *x_bf16, void *y_bf16, int64_t M, void *stream);
int b200q_a16_dev_status(void *handle, void *stream);
void b200q_a16_dev_destroy(void **handle);

/* ------------------------------------------------------------------ calibration math
 * A context owns the scratch memory of the kernels; one context per thread/stream.
 * All tensor pointers are DEVICE pointers unless named *_host. */
int b200q_calib_create(void **ctx);
void b200q_calib_destroy(void **ctx);

/* out[s] = {min, max} (float32) of each of `samples` contiguous runs of n_per_sample floats: the running
 * min/max of ActivationCalibrator.process_statistic (python/calibration/kld_calibrator.py:391-393) takes
 * its per-sample values from here.  NaNs are ignored.  Asynchronous on `stream`. */
int b200q_calib_minmax(void *ctx, const float *x, int64_t n_per_sample, int64_t samples, float *out_minmax,
                       void *stream);

/* Same result as b200q_calib_minmax for callers that are not allowed to allocate device memory: code that runs
 * inside someone else's memory plan (a serving process whose HBM is fully pre-partitioned, a host that forbids
 * cudaMalloc after start-up because an allocation synchronises the device) still needs per-sample min/max.
 * This entry point has no counterpart in the reference.  It needs no context: the kernel's scratch (block
 * partials and ticket counters) lives in a fixed 36 KB device array inside the library, which every GPU that
 * loads the library holds until the process exits.  It calls no cudaMalloc / cudaFree and no allocating library
 * routine.  Limits: at most 1024 samples per call (B200Q_ERR_UNSUPPORTED beyond that); x and out_minmax are the
 * caller's device buffers.  The first call on each device looks up the array's device address (with that device
 * current); make that first call before starting any stream capture.  All calls on a device share the one
 * array and it keeps the last call's contents (the counters are cleared on the stream before each launch), so
 * two calls whose kernels can overlap on the GPU (different streams) race: keep them on one stream or
 * otherwise ordered.  Asynchronous on `stream`, which must belong to the device that is current at the call (the
 * array's address is looked up per current device). */
int b200q_calib_minmax_noalloc(const float *x, int64_t n_per_sample, int64_t samples, float *out_minmax,
                               void *stream);

/* CaliMathCpu.histogram (python/calibration/cali_math.py:68-80) for a batch of samples: sample s is
 * histogrammed over |x| with width th_host[s] / (nbins_host[s] - 1) into nbins_host[s] bins (zeros excluded,
 * float32 arithmetic, numpy.histogram's float32 bin edges) and ADDED into hist[0 .. nbins_host[s]);
 * nbins_host[s] == 0 skips the sample.  Because combine_histogram (cali_math.py:82-103) keeps old counts in
 * their bins, the streaming histogram of a tensor is the sum of such per-sample histograms with the
 * (threshold, bins) schedule derived from the running abs-max.  int32 counts, like the reference. */
int b200q_calib_histogram(void *ctx, const float *x, int64_t n_per_sample, int64_t samples, const float *th_host,
                          const int32_t *nbins_host, int32_t *hist, int64_t hist_len, void *stream);

/* Counter layout of the histogram kernel, process-wide: -1 = chosen per launch from the bin count and the work
 * per block (default); 0..4 = 2^mode 32-bit copies of every bin per block; 5 = one 16-bit counter per (bin, lane).
 * Every layout produces the same counts; this only exists to measure them against each other.  (No counterpart in
 * the reference, whose histogram is numpy's.) */
void b200q_calib_set_histogram_layout(int32_t mode);

/* ActivationCalibrator.find_threshold (kld_calibrator.py:321-347) for `tensors` histograms at once: zero-pad
 * to a multiple of dst_bins, fold pairwise while longer than 131072 bins (doubling the width), then the KLD
 * search of calibration_math.cpp:158-212,:273-323.  thresholds_host[t] is filled on return (synchronous);
 * kl_host, if not NULL, receives 1024 floats per tensor (the KL value of every candidate). */
int b200q_calib_find_thresholds(void *ctx, int32_t tensors, const int32_t *const *hist, const int64_t *n_bins,
                                const float *widths, int64_t dst_bins, float *thresholds_host, float *kl_host,
                                void *stream);

/* ------------------------------------------------------------------ fp32 Top-dialect forward (calibration's float graph)
 * conv_attr_t of top::ConvOp (lib/Dialect/Top/Interfaces/Conv.cpp:19-199); NCHW fp32, OIHW filter. */
typedef struct {
  int64_t n, ic, ih, iw, oc, kh, kw, sh, sw, dh, dw, pht, phb, pwl, pwr, groups;
  int32_t with_bias, do_relu;
  float relu_limit;          /* <= 0: none (function_relu, lib/Support/MathUtils.cpp:891-903) */
} b200q_top_conv_desc;

/* top::ConvOp::inference (Conv.cpp:222-231) over HOST float buffers: inputs = {input, filter OIHW, bias or NULL},
 * outputs[0] [n, oc, oh, ow].  Full fp32 products and sums on the CUDA cores (no tf32). */
int b200q_top_conv2d_inference(const b200q_top_conv_desc *desc, float *const *inputs, int n_inputs,
                               float *const *outputs, int n_outputs);
/* Device face: the handle keeps a transposed copy of the filter; `bias` stays the caller's.  run() takes any batch. */
int b200q_top_conv2d_dev_create(const b200q_top_conv_desc *desc, const float *filter_oihw, const float *bias, void **handle);
int b200q_top_conv2d_dev_run(void *handle, const float *x, float *y, int64_t batch, void *stream);
void b200q_top_conv2d_dev_output_shape(void *handle, int64_t *oh, int64_t *ow);
void b200q_top_conv2d_dev_destroy(void **handle);
/* top::MatMulOp without transposes: y[M,N] = relu(x[M,K] * w[K,N] + bias[N]) (lib/Dialect/Top/Interfaces/MatMul.cpp). */
int b200q_top_matmul_f32_dev(const float *x, const float *w_kn, const float *bias, float *y, int64_t M, int64_t K, int64_t N,
                             int32_t do_relu, float relu_limit, void *stream);
/* top::MaxPoolOp / top::AvgPoolOp, 2-D, over nc = n * c planes (lib/Support/Dnnl/Pool.cpp: -inf padding for max;
 * avg divides by the window clipped to the padded image when count_include_pad, else by the cells inside the image). */
int b200q_top_pool2d_f32_dev(const float *x, float *y, int64_t nc, int32_t ih, int32_t iw, int32_t kh, int32_t kw,
                             int32_t sh, int32_t sw, int32_t pht, int32_t phb, int32_t pwl, int32_t pwr, int32_t is_max,
                             int32_t count_include_pad, int32_t do_relu, float relu_limit, void *stream);
/* top::AddOp with two equal-shape inputs (Add.cpp:45-85) and top::ReluOp (Relu.cpp:17-24). */
int b200q_top_add_f32_dev(const float *a, const float *b, float *y, int64_t count, int32_t do_relu, float relu_limit,
                          void *stream);
int b200q_top_relu_f32_dev(const float *x, float *y, int64_t count, float relu_limit, void *stream);
/* Elementwise float ops of the Top dialect (lib/Dialect/Top/Interfaces/<Op>.cpp), y = relu(op(a, b or const_val)):
 * AddConst, SubConst (and its is_reverse form), MulConst, MaxConst, MinConst, Mul, Sub, Div (and reversed), Sigmoid (and its
 * log form), SiLU, GELU, Floor.  Every expression is evaluated in the type the reference's C++ evaluates it in. */
typedef enum {
  B200Q_TOP_ADD_CONST = 0, B200Q_TOP_SUB_CONST, B200Q_TOP_RSUB_CONST, B200Q_TOP_MUL_CONST, B200Q_TOP_MAX_CONST, B200Q_TOP_MIN_CONST,
  B200Q_TOP_MUL, B200Q_TOP_SUB, B200Q_TOP_RSUB, B200Q_TOP_DIV, B200Q_TOP_RDIV, B200Q_TOP_SIGMOID, B200Q_TOP_LOG_SIGMOID,
  B200Q_TOP_SILU, B200Q_TOP_GELU, B200Q_TOP_FLOOR
} b200q_top_eltwise_op;
int b200q_top_eltwise_f32_dev(int32_t op, const float *a, const float *b, double const_val, float *y, int64_t count,
                              int32_t do_relu, float relu_limit, void *stream);
/* tpu::ActiveOp on float tensors (lib/Dialect/Tpu/Interfaces/Common/Active.cpp:20-32 with the function table of
 * lib/Support/ActiveUtils.cpp:66-181): y = (float)func((double)x).  `mode` is the dialect's ActiveMode number (TANH 0 ... QGELU
 * 37); coeff0 / coeff1 are the op's `coeffs` (ELU alpha; SWISH beta; HSIGMOID beta, alpha).  Modes without a function in the
 * reference's table (RELU, IS_FINITE, ARCSIN, ARCSINH, ARCCOSH) return B200Q_ERR_UNSUPPORTED. */
int b200q_active_f32_dev(int32_t mode, const float *x, double coeff0, double coeff1, float *y, int64_t count, void *stream);
/* top::ScaleOp (Scale.cpp:19-44): y[o, c, i] = relu(x * scale[c] + bias[c]). */
int b200q_top_scale_f32_dev(const float *x, const float *scale, const float *bias, float *y, int64_t outer, int32_t channels,
                            int64_t inner, int32_t do_relu, float relu_limit, void *stream);
/* top::ReduceOp over one run of adjacent axes (Reduce.cpp:59-108): x [outer, axis, inner] -> y [outer, inner]; mode 0 ReduceMean,
 * 1 ReduceSum, 2 ReduceMax, 3 ReduceMin, 4 ReduceProd, 5 ReduceL2, 6 ReduceL1, 7 the mean of tpu::ReduceOp (the sum times
 * float(1.0 / axis), lib/Dialect/Tpu/Interfaces/Common/Reduce.cpp:132-138); sums run along the axis in order like the
 * reference's loop. */
int b200q_top_reduce_f32_dev(int32_t mode, const float *x, float *y, int64_t outer, int32_t axis, int64_t inner, void *stream);
/* top::SoftmaxOp (Softmax.cpp:53-80) over the middle dimension of [outer, channels, inner] (log_softmax when log_form), and
 * top::LayerNormOp (LayerNorm.cpp:24-78) over rows of `inner` values with optional weight / bias of that length. */
int b200q_top_softmax_f32_dev(const float *x, float *y, int64_t outer, int32_t channels, int64_t inner, int32_t log_form,
                              void *stream);
int b200q_top_layernorm_f32_dev(const float *x, const float *weight, const float *bias, float *y, int64_t outer,
                                int64_t inner, float eps, void *stream);
/* Data movement of either dialect (Slice, Permute, Tile, Upsample, Pad, Concat) as one index mapping over up to six
 * dimensions: walking dims[], the source coordinate of dimension d is ((i / div) % mod) * mul + off (mod 0: no wrap) and
 * must lie in [0, extent) or the element becomes *pad_value (zero bytes if NULL); src / dst strides in elements,
 * elem_bytes 1, 2 or 4.  Unused leading dimensions have dims = 1. */
typedef struct {
  int64_t dims[6], src_stride[6], mul[6], div[6], mod[6], off[6], extent[6], dst_stride[6];
  int64_t dst_offset;
} b200q_remap_desc;
int b200q_remap_dev(const void *src, void *dst, int32_t elem_bytes, const b200q_remap_desc *desc, const void *pad_value,
                    void *stream);
/* top::InterpOp / tpu::InterpOp, modes "nearest" (0) and "linear" (1), over nc = n * c planes [ih, iw] -> [oh, ow]
 * (lib/Dialect/Top/Interfaces/Interp.cpp:28-181,:226-287).  coord_mode: 0 half_pixel, 1 pytorch_half_pixel, 2 align_corners,
 * 3 asymmetric; platform (module::getPlatform() of the model): 0 ONNX or any other, 1 TORCH, 2 TFLITE, 3 CAFFE. */
int b200q_interp_f32_dev(const float *x, float *y, int64_t nc, int32_t ih, int32_t iw, int32_t oh, int32_t ow, int32_t mode,
                         int32_t coord_mode, int32_t platform, void *stream);
/* top::GridSamplerOp / tpu::GridSamplerOp with a 4-D grid (GridSamplerFunc::invoke, lib/Support/GenericCpuFunc.cpp:3390-3455):
 * x [n, c, ih, iw], grid [n, oh, ow, 2] of (x, y) in [-1, 1], y [n, c, oh, ow]; mode 0 bilinear / 1 nearest, padding_mode 0 zeros /
 * 1 border / 2 reflection (the reference's numbering).  5-D grids are not implemented. */
int b200q_grid_sampler_f32_dev(const float *x, const float *grid, float *y, int32_t n, int32_t c, int32_t ih, int32_t iw,
                               int32_t oh, int32_t ow, int32_t mode, int32_t padding_mode, int32_t align_corners, void *stream);
/* top::ArgOp / tpu::ArgOp (lib/Dialect/Top/Interfaces/Arg.cpp:39-83): over x [outer, axis, inner] the index of the maximum
 * (is_max) or minimum along the axis, as float or int32, and the value itself when `values` is not NULL; ties keep the first
 * index, or the last when select_last_index. */
int b200q_arg_f32_dev(const float *x, int64_t outer, int32_t axis, int64_t inner, int32_t is_max, int32_t select_last_index,
                      void *indices, int32_t index_is_float, float *values, void *stream);
/* top::CastOp (lib/Dialect/Top/Interfaces/Cast.cpp:18-68): saturate(to_int(x, round_mode)) to `to_dtype` (a b200q_dtype; F32
 * copies), stored as float like the reference's tensors (out_dtype F32) or in the integer type itself (out_dtype = to_dtype). */
int b200q_top_cast_f32_dev(const float *x, int64_t count, int32_t to_dtype, int32_t round_mode, int32_t out_dtype, void *out,
                           void *stream);
/* top::GatherOp / tpu::GatherOp (lib/Dialect/Top/Interfaces/Gather.cpp:17-49): dst[o, j, k] = src[o, indices[j], k] over
 * src [outer, axis_dim, inner]; a negative index counts from the end.  top::GatherElementsOp (GatherElements.cpp:20-79): dst
 * has the shape of `indices` and takes src at the same coordinate except on `axis`, where the index stands (rank <= 8).
 * Indices are float (the reference interpreter's storage) or int32; one outside the axis yields 0 rather than a read outside
 * the tensor.  elem_bytes 1, 2 or 4. */
int b200q_gather_dev(const void *src, int32_t elem_bytes, const void *indices, int32_t index_is_float, void *dst, int64_t outer,
                     int64_t axis_dim, int64_t num_indices, int64_t inner, void *stream);
int b200q_gather_elements_dev(const void *src, int32_t elem_bytes, const void *indices, int32_t index_is_float, void *dst,
                              int32_t ndim, const int64_t *src_shape, const int64_t *indices_shape, int32_t axis, void *stream);
/* The two array operations of the threshold tuner (python/calibration/simple_tunner.py): import_quant_bias (:43-50),
 * y = clip(round_half_even(x * 127 / threshold), -128, 127) * threshold / 127; and the sums behind calc_distance
 * (:334-358), ACCUMULATED into five device doubles: sum (ref - x)^2, sum |ref|, sum x * ref, sum x^2, sum ref^2. */
int b200q_top_fake_quant_f32_dev(const float *x, float *y, int64_t count, double threshold, void *stream);
int b200q_top_distance_f32_dev(const float *x, const float *ref, int64_t count, double *sums5, void *stream);

/* The two symbols of the reference's calibration_math.so (bindings/kld/calibration_math.cpp:326-337), with
 * HOST buffers, so python/calibration/kld_calibrator.py:50-59 can load this library in its place.
 * Failure is reported as NaN (see b200q_last_error). */
float kl_diversity_hist(int *data, float width, long long num_bins, long long dst_bins);
float kl_diversity(float *data, long long count, long long num_bins);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H_ */
