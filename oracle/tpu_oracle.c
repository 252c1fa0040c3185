/*
 * CPU oracle for the quantized-inference hot path of tpu-mlir's Tpu-dialect interpreter.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic the reference
 * interpreter performs for INT8 MatMul / Conv2D / RequantInt(Axis) / Add / Pool2D / Cast, the
 * A16MatMul w4 group-dequant GEMM, bf16 rounding, the calibration histogram and the KLD
 * threshold search.  It is the checker the CUDA kernels are compared against; nothing in the
 * shipped library may call it.
 *
 * Pinning: the rounding / requantisation helpers (to_int, RightShiftRound, MultiplyByQuantizedMultiplier,
 * applyMultiplierAndRShift) are checked against the reference's OWN functions, cut out of
 * lib/Support/MathUtils.cpp:179-213,:474-562 by the build recipe and compiled into oracle/_ref/
 * (tests/test_oracle_golden.py), the bf16 rounding against the reference's lib/Support/Float16.cpp compiled
 * whole the same way, and both against the known answers written in the reference header
 * include/tpu_mlir/Support/MathUtils.h:29-40; the histogram and KLD parts
 * are checked against outputs of the reference's own python/calibration/cali_math.py and
 * bindings/kld/calibration_math.cpp (golden vectors under tests/golden/).  The MatMul/Conv2D
 * op-level code cannot be pinned against a run of the reference (it needs MLIR + oneDNN to
 * build), so for those ops parity is "unpinned" above the pinned requantisation arithmetic: the
 * loops around it (operand order, bias, ReLU placement, saturation) are restated from the cited lines.
 *
 * Every function cites the reference file:line it follows (paths inside the reference tree).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* tpu::RequantMode, include/tpu_mlir/Dialect/Tpu/IR/TpuOps.td:160-172 */
enum { QM_TFLITE_LSHIFT = 0, QM_TFLITE = 1, QM_MULTIPLIER_SHIFT = 2, QM_ONLY_SHIFT = 3, QM_QDM = 4,
       QM_ONLY_SCALE = 5 };
/* RoundingMode, include/tpu_mlir/Support/MathUtils.h:28-42 */
enum { RM_HALF_AWAY = 0, RM_HALF_UP = 1, RM_HALF_DOWN = 2, RM_HALF_EVEN = 3, RM_HALF_ODD = 4,
       RM_HALF_TOWARDS_ZERO = 5, RM_TOWARDS_ZERO = 6, RM_AWAY_FROM_ZERO = 7, RM_UP = 8, RM_DOWN = 9 };
/* storage types of quantized tensors */
enum { DT_I8 = 0, DT_U8 = 1, DT_I16 = 2, DT_U16 = 3, DT_I32 = 4 };

/* lib/Support/MathUtils.cpp:474-514 RightShiftRound<int64_t> */
int64_t orc_rshift_round(int64_t src, int shift_num, int rmode) {
  if (shift_num == 0) return src;
  if (shift_num > 63) shift_num = 63;
  if (shift_num < 0) return (int64_t)((uint64_t)src << (-shift_num));
  int64_t val = src >> shift_num;
  int64_t res = val;
  int64_t lo_mask = (int64_t)((1ull << shift_num) - 1);
  int64_t mant = src & lo_mask;
  int64_t half = (int64_t)(1ull << (shift_num - 1));
  switch (rmode) {
  case RM_HALF_EVEN:
    if (mant == half) res = val + (val & 1);
    else if (mant > half) res = val + 1;
    break;
  case RM_HALF_AWAY:
    if (src >= 0 && mant >= half) res = val + 1;
    else if (src < 0 && mant > half) res = val + 1;
    break;
  case RM_TOWARDS_ZERO:
    if (src < 0) res = val + (mant != 0);
    break;
  case RM_DOWN: res = val; break;
  case RM_UP: res = val + (mant != 0); break;
  case RM_HALF_UP:
    if (mant >= half) res = val + 1;
    break;
  case RM_HALF_DOWN:
    if (mant > half) res = val + 1;
    break;
  default: break;
  }
  return res;
}

/* lib/Support/MathUtils.cpp:179-213 to_int<float> */
int64_t orc_to_int_f32(float v, int rmode) {
  switch (rmode) {
  case RM_HALF_AWAY: return (int64_t)roundf(v);
  case RM_UP: return (int64_t)ceilf(v);
  case RM_DOWN: return (int64_t)floorf(v);
  case RM_HALF_EVEN: {
    float ip;
    float fr = modff(fabsf(v), &ip);
    int64_t r = (int64_t)ip;
    if (fr > 0.5f) r += 1;
    else if (fr == 0.5f && (r & 1)) r += 1;
    return v < 0 ? -r : r;
  }
  case RM_HALF_UP: return (int64_t)floor((double)v + 0.5);   /* std::floor(v + 0.5): double literal */
  case RM_HALF_DOWN: return (int64_t)ceil((double)v - 0.5);
  case RM_TOWARDS_ZERO: return (int64_t)v;
  default: return (int64_t)roundf(v);
  }
}

/* lib/Support/MathUtils.cpp:523-536 MultiplyByQuantizedMultiplier */
int32_t orc_mbqm(int32_t x, int32_t multiplier, int shift, int rmode) {
  int64_t value = shift > 0 ? (int64_t)(int32_t)((uint32_t)x << shift) : (int64_t)x;
  value = orc_rshift_round(value * (int64_t)multiplier, 31, RM_HALF_UP);
  if (value > 2147483647ll) value = 2147483647ll;
  else if (value < -2147483648ll) value = -2147483648ll;
  if (shift < 0) value = orc_rshift_round(value, -shift, rmode);
  return (int32_t)value;
}

/* lib/Support/MathUtils.cpp:538-562 applyMultiplierAndRShift */
int64_t orc_apply_multiplier_rshift(int64_t v, int64_t multiplier, int64_t rshift, int qmode,
                                    int rmode, int is_cv18xx) {
  switch (qmode) {
  case QM_MULTIPLIER_SHIFT:
    if (is_cv18xx) {
      float f = ((float)v * (float)multiplier) / (float)(1 << rshift);
      return orc_to_int_f32(f, rmode);
    }
    return orc_rshift_round(v * multiplier, (int)rshift, rmode);
  case QM_ONLY_SHIFT: return orc_rshift_round(v, (int)rshift, rmode);
  case QM_QDM:
  case QM_TFLITE:
  case QM_TFLITE_LSHIFT:
    if (is_cv18xx) rshift = -rshift;
    return orc_mbqm((int32_t)v, (int32_t)multiplier, (int32_t)rshift, rmode);
  default: return 0;
  }
}

static void dt_range(int dt, int64_t *lo, int64_t *hi) {
  switch (dt) {
  case DT_I8: *lo = -128; *hi = 127; break;
  case DT_U8: *lo = 0; *hi = 255; break;
  case DT_I16: *lo = -32768; *hi = 32767; break;
  case DT_U16: *lo = 0; *hi = 65535; break;
  default: *lo = -2147483648ll; *hi = 2147483647ll; break;
  }
}

/* lib/Support/MathUtils.cpp:849-872 saturate (integer argument: to_int is the identity) */
int64_t orc_saturate(int64_t v, int dt) {
  int64_t lo, hi;
  dt_range(dt, &lo, &hi);
  return v > hi ? hi : (v < lo ? lo : v);
}

static void store_q(void *out, int64_t i, int dt, int64_t v) {
  switch (dt) {
  case DT_I8: ((int8_t *)out)[i] = (int8_t)v; break;
  case DT_U8: ((uint8_t *)out)[i] = (uint8_t)v; break;
  case DT_I16: ((int16_t *)out)[i] = (int16_t)v; break;
  case DT_U16: ((uint16_t *)out)[i] = (uint16_t)v; break;
  default: ((int32_t *)out)[i] = (int32_t)v; break;
  }
}

static inline int32_t load_q8(const void *p, int64_t i, int is_unsigned) {
  return is_unsigned ? (int32_t)((const uint8_t *)p)[i] : (int32_t)((const int8_t *)p)[i];
}

/* The reference accumulates integer-valued floats with an fp32 oneDNN primitive
 * (lib/Support/Dnnl/MatMul.cpp:223-227, lib/Support/Dnnl/Conv.cpp:248-252); that equals exact
 * integer accumulation only while every partial sum stays below 2^24 in magnitude.  The oracle
 * accumulates exactly and counts outputs outside that domain so tests can assert there are none. */
#define FP32_EXACT_LIMIT 16777216ll

/*
 * Requantise one MatMul accumulator the way tpu::MatMulOp::inference does,
 * lib/Dialect/Tpu/Interfaces/Common/MatMul.cpp:636-728.
 *   mult/rshift: per-batch (cv18xx), per-channel (fuse_rq) or single entries as the branch needs.
 */
static int64_t matmul_requant(int64_t acc, int qmode, int is_cv18xx, int fuse_rq, const int64_t *mult,
                              const int64_t *rshift, int64_t b, int64_t n, float only_scale, int out_zp,
                              int out_dt) {
  int64_t v;
  if (is_cv18xx) { /* :638-664 */
    v = orc_apply_multiplier_rshift(acc, mult[b], rshift[b], qmode, RM_HALF_AWAY, 1);
    return orc_saturate(v, out_dt);
  }
  if (qmode == QM_ONLY_SCALE) { /* :673-695 */
    float f = (float)acc * only_scale;
    v = (int64_t)((int32_t)roundf(f) + out_zp);
  } else if (qmode == QM_TFLITE || qmode == QM_TFLITE_LSHIFT) { /* :696-707 */
    v = (int64_t)orc_mbqm((int32_t)acc, (int32_t)mult[0], -(int32_t)rshift[0], RM_HALF_AWAY) + out_zp;
  } else if (qmode == QM_MULTIPLIER_SHIFT) { /* :708-726 */
    int64_t m = fuse_rq ? mult[n] : mult[0];
    v = orc_apply_multiplier_rshift(acc, m, rshift[0], QM_MULTIPLIER_SHIFT, RM_HALF_UP, 0) + out_zp;
  } else {
    v = acc; /* the reference leaves other modes untouched */
  }
  return orc_saturate(v, out_dt);
}

/*
 * tpu::MatMulOp::inference for quantized operands, MatMul.cpp:599-603 + :636-728, with the GEMM
 * of lib/Support/Dnnl/MatMul.cpp:151-241 (zero points subtracted, bias and ReLU inside the GEMM).
 *   A: [batch, M, K] (s8 or u8), B: [batch or 1, K, N] or [.., N, K] when right_transpose.
 *   out_dt == DT_I32 gives the un-requantised int32 MatMul (mult may be NULL).
 * Returns the number of accumulators outside the fp32-exact domain.
 */
int64_t orc_matmul_int8(const void *A, int a_unsigned, const void *B, int b_unsigned, const int32_t *bias,
                        int64_t batch, int b_batched, int64_t M, int64_t K, int64_t N, int right_transpose,
                        int input_zp, int right_zp, int do_relu, int qmode, int is_cv18xx, int fuse_rq,
                        const int64_t *mult, const int64_t *rshift, float only_scale, int out_zp, int out_dt,
                        void *out) {
  int64_t viol = 0;
#pragma omp parallel for collapse(2) reduction(+ : viol) schedule(static)
  for (int64_t b = 0; b < batch; ++b) {
    for (int64_t m = 0; m < M; ++m) {
      int32_t *row = (int32_t *)malloc(sizeof(int32_t) * (size_t)K);
      for (int64_t k = 0; k < K; ++k) row[k] = load_q8(A, (b * M + m) * K + k, a_unsigned) - input_zp;
      const int64_t boff = b_batched ? b * K * N : 0;
      for (int64_t n = 0; n < N; ++n) {
        int64_t acc = 0, amax = 0;
        if (right_transpose) {
          for (int64_t k = 0; k < K; ++k)
            acc += (int64_t)row[k] * (load_q8(B, boff + n * K + k, b_unsigned) - right_zp);
        } else {
          for (int64_t k = 0; k < K; ++k)
            acc += (int64_t)row[k] * (load_q8(B, boff + k * N + n, b_unsigned) - right_zp);
        }
        amax = acc < 0 ? -acc : acc;
        if (bias) acc += bias[n];
        if ((acc < 0 ? -acc : acc) > amax) amax = acc < 0 ? -acc : acc;
        if (amax >= FP32_EXACT_LIMIT) viol++;
        if (do_relu && acc < 0) acc = 0;
        int64_t o = (b * M + m) * N + n;
        if (out_dt == DT_I32 && mult == NULL) store_q(out, o, DT_I32, acc);
        else
          store_q(out, o, out_dt,
                  matmul_requant(acc, qmode, is_cv18xx, fuse_rq, mult, rshift, b, n, only_scale, out_zp, out_dt));
      }
      free(row);
    }
  }
  return viol;
}

/*
 * tpu::Conv2DOp::inference for a uniform-quantized output,
 * lib/Dialect/Tpu/Interfaces/Common/Conv2D.cpp:94-99 (bias removed from the fp32 conv, ReLU off),
 * :264-265 (direct conv, NCHW / OIHW, padding with pad_value, lib/Support/Dnnl/Conv.cpp:98-145),
 * :295-341 (bias added after the conv, requant, +zp, ReLU as max(v, zp), saturate).
 *   n_q: number of multiplier/rshift entries (oc = per-axis, else entry 0 is used).
 * Returns the number of accumulators outside the fp32-exact domain.
 */
int64_t orc_conv2d_int8(const void *x, int x_unsigned, const int8_t *w, const int32_t *bias, int64_t n, int64_t ic,
                        int64_t ih, int64_t iw, int64_t oc, int64_t kh, int64_t kw, int64_t sh, int64_t sw,
                        int64_t dh, int64_t dw, int64_t pht, int64_t phb, int64_t pwl, int64_t pwr, int64_t groups,
                        int pad_value, int do_relu, int qmode, int is_cv18xx, const int64_t *mult,
                        const int64_t *rshift, int64_t n_q, int out_zp, int out_dt, void *out) {
  const int64_t oh = (ih + pht + phb - dh * (kh - 1) - 1) / sh + 1;
  const int64_t ow = (iw + pwl + pwr - dw * (kw - 1) - 1) / sw + 1;
  const int64_t icg = ic / groups, ocg = oc / groups;
  const int per_axis = (n_q == oc);
  const int is_tf = (qmode == QM_QDM || qmode == QM_TFLITE || qmode == QM_TFLITE_LSHIFT);
  const int rmode = is_tf ? RM_HALF_AWAY : RM_HALF_UP; /* Conv2D.cpp:312-315 */
  int64_t viol = 0;
#pragma omp parallel for collapse(2) reduction(+ : viol) schedule(dynamic)
  for (int64_t in = 0; in < n; ++in) {
    for (int64_t o = 0; o < oc; ++o) {
      const int64_t g = o / ocg;
      const int64_t shift = per_axis ? rshift[o] : rshift[0];
      const int64_t multi = (qmode == QM_ONLY_SHIFT) ? 1 : (per_axis ? mult[o] : mult[0]);
      const int32_t b = bias ? bias[o] : 0;
      int32_t *acc = (int32_t *)calloc((size_t)(oh * ow), sizeof(int32_t));
      int64_t *absmax = (int64_t *)calloc((size_t)(oh * ow), sizeof(int64_t));
      for (int64_t c = 0; c < icg; ++c) {
        const int64_t cin = g * icg + c;
        for (int64_t fy = 0; fy < kh; ++fy) {
          for (int64_t fx = 0; fx < kw; ++fx) {
            const int32_t wv = w[((o * icg + c) * kh + fy) * kw + fx];
            if (wv == 0) continue;
            for (int64_t y = 0; y < oh; ++y) {
              const int64_t iy = y * sh - pht + fy * dh;
              const int in_y = (iy >= 0 && iy < ih);
              for (int64_t xo = 0; xo < ow; ++xo) {
                const int64_t ix = xo * sw - pwl + fx * dw;
                int32_t xv = pad_value;
                if (in_y && ix >= 0 && ix < iw) xv = load_q8(x, ((in * ic + cin) * ih + iy) * iw + ix, x_unsigned);
                acc[y * ow + xo] += wv * xv;
              }
            }
          }
        }
      }
      for (int64_t p = 0; p < oh * ow; ++p) {
        /* Conv2D.cpp:331: float accumulator + int32 bias, evaluated in float */
        int64_t tmp = (int64_t)acc[p] + b;
        int64_t a1 = acc[p] < 0 ? -(int64_t)acc[p] : acc[p], a2 = tmp < 0 ? -tmp : tmp;
        (void)absmax;
        if (a1 >= FP32_EXACT_LIMIT || a2 >= FP32_EXACT_LIMIT || (b < 0 ? -(int64_t)b : b) >= FP32_EXACT_LIMIT) viol++;
        int64_t v = orc_apply_multiplier_rshift(tmp, multi, shift, qmode, rmode, is_cv18xx) + out_zp;
        if (do_relu && v < out_zp) v = out_zp;
        store_q(out, (in * oc + o) * oh * ow + p, out_dt, orc_saturate(v, out_dt));
      }
      free(acc);
      free(absmax);
    }
  }
  return viol;
}

/*
 * The requant half of tpu::Conv2DOp::inference alone (Conv2D.cpp:295-341), applied to the float output of
 * an fp32 convolution the way the reference does it: `int64_t tmp = p.outputs[0][offset] + bias` is a FLOAT
 * addition of the float accumulator and the int32 bias (:331).  Used with an fp32 oneDNN convolution
 * (torch on CPU) to time the reference's own arithmetic path.
 */
void orc_conv_requant_from_f32(const float *acc, const int32_t *bias, int64_t n, int64_t oc, int64_t hw, int do_relu,
                               int qmode, int is_cv18xx, const int64_t *mult, const int64_t *rshift, int64_t n_q,
                               int out_zp, int out_dt, void *out) {
  const int per_axis = (n_q == oc);
  const int is_tf = (qmode == QM_QDM || qmode == QM_TFLITE || qmode == QM_TFLITE_LSHIFT);
  const int rmode = is_tf ? RM_HALF_AWAY : RM_HALF_UP;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t in = 0; in < n; ++in)
    for (int64_t o = 0; o < oc; ++o) {
      const int64_t shift = per_axis ? rshift[o] : rshift[0];
      const int64_t multi = (qmode == QM_ONLY_SHIFT) ? 1 : (per_axis ? mult[o] : mult[0]);
      const int32_t b = bias ? bias[o] : 0;
      for (int64_t p = 0; p < hw; ++p) {
        const int64_t off = (in * oc + o) * hw + p;
        int64_t tmp = (int64_t)(acc[off] + (float)b);
        int64_t v = orc_apply_multiplier_rshift(tmp, multi, shift, qmode, rmode, is_cv18xx) + out_zp;
        if (do_relu && v < out_zp) v = out_zp;
        store_q(out, off, out_dt, orc_saturate(v, out_dt));
      }
    }
}

/*
 * tpu::RequantIntAxisOp::inference, lib/Dialect/Tpu/Interfaces/Common/RequantIntAxis.cpp:17-123,
 * BM1684X quant layout {multiplier, shift, zero_point} x C (:45-48).  The triples arrive as the
 * interpreter sees them: float-stored words converted to int64 (so a multiplier above 2^24 has
 * already lost its low bits); the caller does that conversion.
 *   outer x C x inner view; fuse_rq_axis uses the LAST axis as the channel (:70-93).
 */
void orc_requant_int_axis(const int32_t *x, int64_t outer, int64_t C, int64_t inner, const int64_t *quant3,
                          int qmode, int rmode, int fuse_rq_axis, int in_zp, int out_dt, void *out) {
#pragma omp parallel for schedule(static)
  for (int64_t c = 0; c < C; ++c) {
    const int64_t multi = quant3[c * 3], sv = quant3[c * 3 + 1], zp = quant3[c * 3 + 2];
    for (int64_t o = 0; o < outer; ++o) {
      for (int64_t i = 0; i < inner; ++i) {
        const int64_t off = (o * C + c) * inner + i;
        int32_t v;
        if (qmode == QM_TFLITE || qmode == QM_TFLITE_LSHIFT) { /* :41-66 */
          v = (int32_t)(zp + orc_mbqm(x[off], (int32_t)multi, (int32_t)sv, rmode));
        } else if (fuse_rq_axis) { /* :70-93, shift used as given */
          v = (int32_t)(zp + orc_apply_multiplier_rshift((int64_t)x[off] - in_zp, multi, sv, QM_MULTIPLIER_SHIFT,
                                                         rmode, 0));
        } else { /* :95-121, rshift = -shift word */
          v = (int32_t)(zp + orc_apply_multiplier_rshift((int64_t)x[off] - in_zp, multi, -sv, QM_MULTIPLIER_SHIFT,
                                                         rmode, 0));
        }
        store_q(out, off, out_dt, orc_saturate(v, out_dt));
      }
    }
  }
}

/* tpu::RequantIntOp::inference, lib/Dialect/Tpu/Interfaces/Common/RequantInt.cpp:17-71: one
 * (multiplier, rshift) for the whole tensor.  shift = -rshift for the TFLite modes (:40-47), the
 * MultiplierShift branch shifts right by rshift (:48-58). */
void orc_requant_int(const int32_t *x, int64_t count, int64_t multi, int64_t rshift, int qmode, int rmode,
                     int in_zp, int out_zp, int out_dt, void *out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < count; ++i) {
    int64_t v;
    if (qmode == QM_TFLITE || qmode == QM_TFLITE_LSHIFT)
      v = out_zp + (int64_t)orc_mbqm(x[i], (int32_t)multi, (int32_t)(-rshift), rmode);
    else
      v = out_zp +
          orc_apply_multiplier_rshift((int64_t)x[i] - in_zp, multi, rshift, QM_MULTIPLIER_SHIFT, rmode, 0);
    store_q(out, i, out_dt, orc_saturate(v, out_dt));
  }
}

/* tpu::AddOp::inference, symmetric int8, non-cv18xx: lib/Dialect/Tpu/Interfaces/Common/Add.cpp:177-207.
 * Each input is rescaled with MultiplierShift/half-up, the sum (+ReLU) is saturated. */
void orc_add_int8(const void *a, int a_unsigned, const void *b, int b_unsigned, int64_t count, int64_t m0,
                  int64_t s0, int64_t m1, int64_t s1, int do_relu, int out_dt, void *out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < count; ++i) {
    int64_t l = orc_apply_multiplier_rshift(load_q8(a, i, a_unsigned), m0, s0, QM_MULTIPLIER_SHIFT, RM_HALF_UP, 0);
    int64_t r = orc_apply_multiplier_rshift(load_q8(b, i, b_unsigned), m1, s1, QM_MULTIPLIER_SHIFT, RM_HALF_UP, 0);
    int64_t v = l + r;
    if (do_relu && v < 0) v = 0;
    store_q(out, i, out_dt, orc_saturate(v, out_dt));
  }
}

/* tpu::LutOp::inference, lib/Dialect/Tpu/Interfaces/Common/Lut.cpp:20-32: out[i] = table[x[i] mod 256]
 * (a negative index wraps by +256); `esize` bytes per table entry / output element. */
void orc_lut(const void *x, int x_unsigned, int64_t count, const void *table, int esize, void *out) {
  for (int64_t i = 0; i < count; ++i) {
    int64_t off = load_q8(x, i, x_unsigned);
    if (off < 0) off += 256;
    memcpy((char *)out + i * esize, (const char *)table + off * esize, (size_t)esize);
  }
}

/* tpu::MulShiftOp::inference, lib/Dialect/Tpu/Interfaces/Common/MulShift.cpp:19-41:
 * out = saturate(applyMultiplierAndRShift(x - in_zp, multiplier, rshift) + out_zp)  (MultiplierShift, half-up). */
void orc_mulshift_int8(const void *x, int x_unsigned, int64_t count, int64_t multiplier, int64_t rshift, int64_t in_zp,
                       int64_t out_zp, int out_dt, void *out) {
  for (int64_t i = 0; i < count; ++i) {
    int64_t v = orc_apply_multiplier_rshift(load_q8(x, i, x_unsigned) - in_zp, multiplier, rshift, QM_MULTIPLIER_SHIFT,
                                            RM_HALF_UP, 0);
    store_q(out, i, out_dt, orc_saturate(v + out_zp, out_dt));
  }
}

/* tpu::MulOp::inference, symmetric int8, equal shapes, non-cv18xx: lib/Dialect/Tpu/Interfaces/Common/Mul.cpp:72-85:
 * the product (exact in the reference's float) is rescaled with MultiplierShift/half-up and saturated; the ReLU of
 * the op is applied to the product by the binary primitive (Mul.cpp:23-29: do_relu is an argument of its set-up). */
void orc_mul_int8(const void *a, int a_unsigned, const void *b, int b_unsigned, int64_t count, int64_t multiplier,
                  int64_t rshift, int do_relu, int out_dt, void *out) {
  for (int64_t i = 0; i < count; ++i) {
    int64_t prod = load_q8(a, i, a_unsigned) * load_q8(b, i, b_unsigned);
    if (do_relu && prod < 0) prod = 0;
    int64_t v = orc_apply_multiplier_rshift(prod, multiplier, rshift, QM_MULTIPLIER_SHIFT, RM_HALF_UP, 0);
    store_q(out, i, out_dt, orc_saturate(v, out_dt));
  }
}

/* tpu::Pool2DOp::inference, lib/Dialect/Tpu/Interfaces/Common/Pool2D.cpp:160-192.
 *   mode 0 = max (pad cells never win), mode 1 = avg: the window SUM (count_include_pad, zero pad) is
 *   recovered as to_int(avg*kh*kw) and rescaled with MultiplierShift/half-up, ReLU, saturate. */
void orc_pool2d_int8(const void *x, int x_unsigned, int64_t n, int64_t c, int64_t ih, int64_t iw, int64_t kh,
                     int64_t kw, int64_t sh, int64_t sw, int64_t pht, int64_t phb, int64_t pwl, int64_t pwr,
                     int mode, int64_t multi, int64_t rshift, int do_relu, int out_dt, void *out) {
  const int64_t oh = (ih + pht + phb - kh) / sh + 1, ow = (iw + pwl + pwr - kw) / sw + 1;
#pragma omp parallel for schedule(static)
  for (int64_t nc = 0; nc < n * c; ++nc) {
    for (int64_t y = 0; y < oh; ++y)
      for (int64_t xo = 0; xo < ow; ++xo) {
        int64_t best = INT64_MIN, sum = 0;
        for (int64_t fy = 0; fy < kh; ++fy)
          for (int64_t fx = 0; fx < kw; ++fx) {
            int64_t iy = y * sh - pht + fy, ix = xo * sw - pwl + fx;
            if (iy < 0 || iy >= ih || ix < 0 || ix >= iw) continue;
            int64_t v = load_q8(x, (nc * ih + iy) * iw + ix, x_unsigned);
            if (v > best) best = v;
            sum += v;
          }
        int64_t v;
        if (mode == 0) {
          v = best;
          if (do_relu && v < 0) v = 0;
        } else {
          v = orc_apply_multiplier_rshift(sum, multi, rshift, QM_MULTIPLIER_SHIFT, RM_HALF_UP, 0);
          if (do_relu && v < 0) v = 0;
          v = orc_saturate(v, out_dt);
        }
        store_q(out, (nc * oh + y) * ow + xo, out_dt, v);
      }
  }
}

/* tpu::CastOp f32 -> int8/uint8: lib/Dialect/Tpu/Interfaces/Common/Cast.cpp:75-93 with
 * lib/Support/CastUtils.cpp:15-20: round(x * (float)(1/scale)) + zp, then saturate(to_int(., rmode)). */
void orc_cast_f32_to_q8(const float *x, int64_t count, double scale, int zp, int rmode, int out_dt, void *out) {
  const float inv = (float)(1.0 / scale);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < count; ++i) {
    float v = roundf(x[i] * inv) + (float)zp;
    store_q(out, i, out_dt, orc_saturate(orc_to_int_f32(v, rmode), out_dt));
  }
}

/* tpu::CastOp int8/uint8 -> f32: Cast.cpp:94-116: (float)scale * (q - (float)zp). */
void orc_cast_q8_to_f32(const void *x, int x_unsigned, int64_t count, double scale, int zp, float *out) {
  const float s = (float)scale;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < count; ++i) out[i] = s * ((float)load_q8(x, i, x_unsigned) - (float)zp);
}

/* BF16(): lib/Support/Float16.cpp:603-645 (fp32_to_bf16_all, round-half-to-even), :550-601 (fp32
 * denormals flush to signed zero except the top half-ulp band which becomes the smallest normal). */
uint16_t orc_f32_to_bf16_bits(float f) {
  uint32_t bits;
  memcpy(&bits, &f, 4);
  const uint32_t exp = (bits >> 23) & 0xff, frac = bits & 0x7fffff, sign = bits >> 31;
  if (exp > 0 && exp < 255) {
    int64_t r = orc_rshift_round((int64_t)bits, 16, RM_HALF_EVEN);
    uint32_t b32 = (uint32_t)((r << 16) & 0xFFFFFFFFll);
    return (uint16_t)(b32 >> 16);
  }
  if (exp == 0xff) return frac ? 0x7fff : (uint16_t)(sign ? 0xff80 : 0x7f80);
  if (frac == 0) return (uint16_t)(sign << 15);
  if (((frac >> 16) & 0x7f) == 0x7f && (frac & 0x8000)) return (uint16_t)((sign << 15) | 0x80);
  return (uint16_t)(sign << 15);
}

/* F16(): lib/Support/Float16.cpp:763-767 f32_to_f16 -> fp32_to_fp16_all (:663-714) with ROUNDING_HALF_TO_EVEN:
 * normal range (biased fp32 exponent 113..254): the 32-bit pattern is rounded half-to-even at bit 13 and converted
 * exactly (a carry past 65504 gives infinity); exponent 1..112: the 24-bit significand is shifted right by
 * (113 - exp) + 13 with the same rounding (fp16 subnormals; shifts of 64 and more are undefined in the reference and
 * give zero here); NaN -> 0x7fff; infinities and zeros keep their sign; fp32 denormals -> signed zero. */
uint16_t orc_f32_to_f16_bits(float f) {
  uint32_t bits;
  memcpy(&bits, &f, 4);
  const uint32_t exp = (bits >> 23) & 0xff, frac = bits & 0x7fffff, sign = bits >> 31;
  if (exp > 112 && exp < 255) {
    const int64_t r = orc_rshift_round((int64_t)bits, 13, RM_HALF_EVEN);
    const uint32_t b32 = (uint32_t)((r << 13) & 0xFFFFFFFFll);
    const uint32_t e = (b32 >> 23) & 0xff, m = b32 & 0x7fffff;      /* m has 13 zero low bits now */
    if (e >= 143) return (uint16_t)((sign << 15) | 0x7c00);          /* 2^16 and above: infinity */
    return (uint16_t)((sign << 15) | ((e - 112) << 10) | (m >> 13));
  }
  if (exp > 0 && exp <= 112) {
    const int shift = (113 - (int)exp) + 13;
    if (shift >= 64) return (uint16_t)(sign << 15);
    const int64_t mant = (int64_t)frac + (1 << 23);
    const int64_t r = orc_rshift_round(mant, shift, RM_HALF_EVEN);   /* magnitude: the reference negates around the shift */
    return (uint16_t)((sign << 15) | (uint32_t)(r & 0x7fff));
  }
  if (exp == 0xff) return frac ? 0x7fff : (uint16_t)(sign ? 0xfc00 : 0x7c00);
  return (uint16_t)(sign << 15);
}

/* f16_to_f32 (Float16.cpp:776-786): NaN -> 0xFFC00000, everything else exact. */
float orc_f16_bits_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 0x1f, m = h & 0x3ff;
  uint32_t bits;
  if (e == 31) bits = m ? 0xFFC00000u : (sign | 0x7f800000u);
  else if (e != 0) bits = sign | ((e + 112) << 23) | (m << 13);
  else if (m == 0) bits = sign;
  else {
    int sh = 0;
    uint32_t mm = m;
    while (!(mm & 0x400)) { mm <<= 1; ++sh; }
    bits = sign | ((uint32_t)(113 - sh) << 23) | ((mm & 0x3ff) << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

float orc_bf16_bits_to_f32(uint16_t b) {
  uint32_t bits = (uint32_t)b << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/*
 * tpu::A16MatMulOp::inference, static 4-bit path with q_group_size and w_transpose,
 * lib/Dialect/Tpu/Interfaces/Common/A16MatMul.cpp:171-208 (dequant, even flat index = low nibble, NOT
 * rounded to bf16) and :240-246 (output rounded to bf16).  The fp32 GEMM of the reference is an
 * oneDNN sgemm whose summation order is unspecified; this restatement accumulates in fp32 in
 * increasing k, which is one admissible order (tolerance, not bit parity, applies to this op).
 *   x: bf16 bits [M,K]; wq: bytes [N, K/2]; scale: bf16 bits [N*K/g]; zp: u8 [N*K/g]; bias f32 [N] or NULL.
 */
static void a16matmul_w4_any(const uint16_t *x, const uint8_t *wq, const uint16_t *scale, const uint8_t *zp,
                             const float *bias, int64_t M, int64_t K, int64_t N, int64_t group, uint16_t *y, int is_f16) {
  float *W = (float *)malloc(sizeof(float) * (size_t)(N * K));
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < N * K; i += 2) {
    /* group > 0 and even => i and i+1 share a group */
    int64_t qi = i / group;
    float s = is_f16 ? orc_f16_bits_to_f32(scale[qi]) : orc_bf16_bits_to_f32(scale[qi]);
    int z = zp[qi];
    W[i] = (float)(((int)wq[i / 2] & 0x0F) - z) * s;
    int64_t qj = (i + 1) / group;
    float s1 = is_f16 ? orc_f16_bits_to_f32(scale[qj]) : orc_bf16_bits_to_f32(scale[qj]);
    int z1 = zp[qj];
    W[i + 1] = (float)(((int)wq[(i + 1) / 2] >> 4) - z1) * s1;
  }
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      float acc = 0.f;
      for (int64_t k = 0; k < K; ++k)
        acc += (is_f16 ? orc_f16_bits_to_f32(x[m * K + k]) : orc_bf16_bits_to_f32(x[m * K + k])) * W[n * K + k];
      if (bias) acc += bias[n];
      y[m * N + n] = is_f16 ? orc_f32_to_f16_bits(acc) : orc_f32_to_bf16_bits(acc);
    }
  free(W);
}

void orc_a16matmul_w4(const uint16_t *x, const uint8_t *wq, const uint16_t *scale, const uint8_t *zp,
                      const float *bias, int64_t M, int64_t K, int64_t N, int64_t group, uint16_t *y) {
  a16matmul_w4_any(x, wq, scale, zp, bias, M, K, N, group, y, 0);
}

/* The same op with f16 activations, scales and output (the op's storage type decides, A16MatMul.cpp:240-246). */
void orc_a16matmul_w4_f16(const uint16_t *x, const uint8_t *wq, const uint16_t *scale, const uint8_t *zp,
                          const float *bias, int64_t M, int64_t K, int64_t N, int64_t group, uint16_t *y) {
  a16matmul_w4_any(x, wq, scale, zp, bias, M, K, N, group, y, 1);
}

/* fp32 dequantised weight only (used by the fp32-GEMM timing leg and by tests) */
void orc_a16_dequant_w4(const uint8_t *wq, const uint16_t *scale, const uint8_t *zp, int64_t N, int64_t K,
                        int64_t group, float *W) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < N * K; ++i) {
    int64_t qi = i / group;
    int q = (i & 1) ? ((int)wq[i / 2] >> 4) : ((int)wq[i / 2] & 0x0F);
    W[i] = (float)(q - (int)zp[qi]) * orc_bf16_bits_to_f32(scale[qi]);
  }
}

/*
 * CaliMathCpu.histogram, python/calibration/cali_math.py:68-80, in float32:
 *   width = abs_max / (bins - 1); k = floor(|x| / width + 0.5) for x != 0; values with k outside
 *   [0, bins-1] are dropped (np.histogram range semantics).
 * The bin is NOT always k.  np.histogram(k, bins, range=(0, bins-1)) on float32 input builds its bins+1
 * edges with linspace in float64 and stores them as float32, E[j] = (float)(j * ((bins-1)/bins)), then
 * puts k into bin k and moves it up one bin when k >= E[k+1] (its "increment" fix-up; the last bin is
 * closed).  Rounding E to float32 makes that true for the top few bins once bins reaches a few thousand,
 * so those counts land one bin higher than k.  Reproduced here exactly.
 * Counts are ADDED into hist (int32, like the reference's astype(int32) and int32 adds), so a
 * zero-extended running histogram can be passed.
 */
int64_t orc_histogram_bin(float k, int64_t bins) {
  int64_t idx = (int64_t)k;
  if (idx >= bins - 1) return bins - 1;
  const double step = (double)(bins - 1) / (double)bins;
  const float edge = (idx + 1 == bins) ? (float)(bins - 1) : (float)((double)(idx + 1) * step);
  if (k >= edge) idx += 1;
  return idx;
}

void orc_histogram_f32(const float *x, int64_t count, float abs_max, int64_t bins, int32_t *hist) {
  const float width = abs_max / (float)(bins - 1);
  for (int64_t i = 0; i < count; ++i) {
    float t = fabsf(x[i]);
    if (t == 0.f || t != t) continue;
    float k = floorf(t / width + 0.5f);
    if (k >= 0.f && k <= (float)(bins - 1)) hist[orc_histogram_bin(k, bins)] += 1;
  }
}

/*
 * kl_diversity_hist -> real_multi_thread_kl_diversity_hist -> kl_calc_thread,
 * bindings/kld/calibration_math.cpp:158-212,:273-323, the_min_index :71-83.  Sequential float32 sums
 * in the reference's order, log10 in double.  kl_out (optional) receives the per-candidate KL values.
 */
float orc_kl_diversity_hist(const int32_t *data, float width, int64_t N, int64_t BINS, float *kl_out) {
  const int64_t KL_NUM = N / BINS;
  int64_t *hist = (int64_t *)malloc(sizeof(int64_t) * (size_t)N);
  float *kl = (float *)calloc((size_t)KL_NUM, sizeof(float));
  int64_t count = 0;
  for (int64_t i = 0; i < N; ++i) {
    hist[i] = data[i];
    count += hist[i];
  }
#pragma omp parallel for schedule(dynamic)
  for (int64_t m = 0; m < KL_NUM; ++m) {
    const int64_t i = (m + 1) * BINS;
    float *P = (float *)calloc((size_t)i, sizeof(float));
    float *Q = (float *)malloc(sizeof(float) * (size_t)i);
    for (int64_t j = 0; j < N; ++j) {
      int64_t index = (j > (i - 1)) ? (i - 1) : j;
      P[index] += (float)hist[j];
    }
    for (int64_t j = 0; j < i; ++j) P[j] /= (float)count;
    float sum = 0.f;
    const int64_t expand = i / BINS;
    int64_t idx = 0;
    for (int64_t j = 0; j < i; ++j) sum += (float)hist[j];
    for (int64_t j = 0; j < BINS; ++j) {
      float sum_bin = 0.f, positive = 0.f;
      int64_t bin_idx = idx;
      for (int64_t k = 0; k < expand; ++k) {
        sum_bin += (float)hist[idx];
        positive += (hist[idx] > 0) ? 1.f : 0.f;
        idx++;
      }
      if (positive == 0.f) positive = 1.f;
      float Q_base = sum_bin / positive / sum;
      while (bin_idx < idx) {
        Q[bin_idx] = hist[bin_idx] ? Q_base : 0.f;
        bin_idx++;
      }
    }
    float acc = 0.f;
    for (idx = 0; idx < i; ++idx)
      acc = (float)((double)acc + (double)P[idx] * (log10((double)P[idx] + 1e-30) - log10((double)Q[idx] + 1e-30)));
    kl[m] = acc;
    free(P);
    free(Q);
  }
  int64_t m_min = 0;
  float best = kl[0];
  for (int64_t m = 1; m < KL_NUM; ++m)
    if (best > kl[m]) {
      best = kl[m];
      m_min = m;
    }
  if (kl_out) memcpy(kl_out, kl, sizeof(float) * (size_t)KL_NUM);
  float threshold = width * (float)(m_min + 1) * (float)BINS;
  free(hist);
  free(kl);
  return threshold;
}

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------------------------------------ fp32 Top-dialect forward
 * top::ConvOp::inference (lib/Dialect/Top/Interfaces/Conv.cpp:222-231: oneDNN fp32 convolution, NCHW / OIHW, zero
 * padding, bias, then ReLU with relu_limit, lib/Support/Dnnl/Conv.cpp:98-215).  oneDNN does not define its summation
 * order, so this restatement sums k = (c, kh, kw) in index order with a double accumulator and the comparison with
 * either implementation is by tolerance. */
void orc_top_conv2d_f32(const float *x, const float *w, const float *bias, int64_t n, int64_t ic, int64_t ih, int64_t iw,
                        int64_t oc, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t dh, int64_t dw, int64_t pht,
                        int64_t phb, int64_t pwl, int64_t pwr, int64_t groups, int do_relu, float relu_limit, float *out) {
  const int64_t oh = (ih + pht + phb - dh * (kh - 1) - 1) / sh + 1;
  const int64_t ow = (iw + pwl + pwr - dw * (kw - 1) - 1) / sw + 1;
  const int64_t icg = ic / groups, ocg = oc / groups;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int64_t in = 0; in < n; ++in) {
    for (int64_t o = 0; o < oc; ++o) {
      const int64_t g = o / ocg;
      for (int64_t y = 0; y < oh; ++y) {
        for (int64_t xo = 0; xo < ow; ++xo) {
          double acc = 0.0;
          for (int64_t c = 0; c < icg; ++c) {
            for (int64_t a = 0; a < kh; ++a) {
              const int64_t h = y * sh - pht + a * dh;
              if (h < 0 || h >= ih) continue;
              for (int64_t b = 0; b < kw; ++b) {
                const int64_t ww = xo * sw - pwl + b * dw;
                if (ww < 0 || ww >= iw) continue;
                acc += (double)x[((in * ic + g * icg + c) * ih + h) * iw + ww] * (double)w[((o * icg + c) * kh + a) * kw + b];
              }
            }
          }
          float v = (float)acc + (bias ? bias[o] : 0.f);
          if (do_relu) { /* function_relu, lib/Support/MathUtils.cpp:891-903 */
            v = v > 0.f ? v : 0.f;
            if (relu_limit > 0.f && v > relu_limit) v = relu_limit;
          }
          out[((in * oc + o) * oh + y) * ow + xo] = v;
        }
      }
    }
  }
}

/* top::MaxPoolOp / top::AvgPoolOp through lib/Support/Dnnl/Pool.cpp: max ignores the padding; avg divides by the
 * window clipped to the padded image when count_include_pad, else by the number of cells inside the image. */
void orc_top_pool2d_f32(const float *x, int64_t nc, int64_t ih, int64_t iw, int64_t kh, int64_t kw, int64_t sh, int64_t sw,
                        int64_t pht, int64_t phb, int64_t pwl, int64_t pwr, int is_max, int count_include_pad, int do_relu,
                        float relu_limit, float *out) {
  const int64_t oh = (ih + pht + phb - kh) / sh + 1, ow = (iw + pwl + pwr - kw) / sw + 1;
#pragma omp parallel for schedule(static)
  for (int64_t p = 0; p < nc; ++p) {
    for (int64_t y = 0; y < oh; ++y) {
      for (int64_t xo = 0; xo < ow; ++xo) {
        const int64_t h0 = y * sh - pht, w0 = xo * sw - pwl;
        float acc = is_max ? -INFINITY : 0.f;
        int64_t inside = 0;
        for (int64_t a = 0; a < kh; ++a) {
          for (int64_t b = 0; b < kw; ++b) {
            const int64_t h = h0 + a, ww = w0 + b;
            if (h < 0 || h >= ih || ww < 0 || ww >= iw) continue;
            const float v = x[(p * ih + h) * iw + ww];
            acc = is_max ? (v > acc ? v : acc) : acc + v;
            ++inside;
          }
        }
        if (!is_max) {
          int64_t div = inside;
          if (count_include_pad) {
            const int64_t he = h0 + kh < ih + phb ? h0 + kh : ih + phb, we = w0 + kw < iw + pwr ? w0 + kw : iw + pwr;
            div = (he - h0) * (we - w0);
          }
          acc = div > 0 ? acc / (float)div : 0.f;
        }
        if (do_relu) {
          acc = acc > 0.f ? acc : 0.f;
          if (relu_limit > 0.f && acc > relu_limit) acc = relu_limit;
        }
        out[(p * oh + y) * ow + xo] = acc;
      }
    }
  }
}
