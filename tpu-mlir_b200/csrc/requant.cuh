// Exact integer requantisation, shared by every kernel epilogue.
//
// Reference semantics (paths inside the tpu-mlir tree):
//   RightShiftRound                lib/Support/MathUtils.cpp:474-514
//   MultiplyByQuantizedMultiplier  lib/Support/MathUtils.cpp:523-536
//   applyMultiplierAndRShift       lib/Support/MathUtils.cpp:538-562
//   to_int                         lib/Support/MathUtils.cpp:179-213
//   saturate                       lib/Support/MathUtils.cpp:849-872
#pragma once
#include <stdint.h>

#include "../../include/b200q.h"

namespace b200q {

struct Epilogue {
  int dialect;     // b200q_rq_dialect
  int round_mode;  // b200q_round_mode
  int per_channel; // multiplier/shift indexed by channel (else entry 0)
  int out_zp;
  int relu;        // b200q_relu_order
  int out_dtype;   // b200q_dtype
  float scale;     // B200Q_RQ_ONLY_SCALE
  const int32_t* bias;        // [C] or nullptr
  const int32_t* multiplier;  // [C] or [1] (nullptr only for B200Q_RQ_NONE / ONLY_SHIFT / ONLY_SCALE)
  const int32_t* shift;       // [C] or [1]
};

__host__ __device__ __forceinline__ int64_t rshift_round(int64_t src, int s, int rmode) {
  if (s == 0) return src;
  if (s > 63) s = 63;
  if (s < 0) return (int64_t)((uint64_t)src << (-s));
  const int64_t val = src >> s;
  const int64_t mant = src & (int64_t)((1ull << s) - 1ull);
  const int64_t half = (int64_t)(1ull << (s - 1));
  switch (rmode) {
    case B200Q_ROUND_HALF_UP: return val + (mant >= half);
    case B200Q_ROUND_HALF_AWAY_FROM_ZERO: return val + ((src >= 0) ? (mant >= half) : (mant > half));
    case B200Q_ROUND_HALF_TO_EVEN: return (mant == half) ? val + (val & 1) : val + (mant > half);
    case B200Q_ROUND_HALF_DOWN: return val + (mant > half);
    case B200Q_ROUND_TOWARDS_ZERO: return (src < 0) ? val + (mant != 0) : val;
    case B200Q_ROUND_UP: return val + (mant != 0);
    default: return val;  // ROUND_DOWN and the modes RightShiftRound leaves untouched
  }
}

__host__ __device__ __forceinline__ int64_t to_int_f32(float v, int rmode) {
  switch (rmode) {
    case B200Q_ROUND_UP: return (int64_t)ceilf(v);
    case B200Q_ROUND_DOWN: return (int64_t)floorf(v);
    case B200Q_ROUND_HALF_TO_EVEN: {
      float ip;
      const float fr = modff(fabsf(v), &ip);
      int64_t r = (int64_t)ip;
      if (fr > 0.5f) r += 1;
      else if (fr == 0.5f && (r & 1)) r += 1;
      return v < 0 ? -r : r;
    }
    case B200Q_ROUND_HALF_UP: return (int64_t)floor((double)v + 0.5);
    case B200Q_ROUND_HALF_DOWN: return (int64_t)ceil((double)v - 0.5);
    case B200Q_ROUND_TOWARDS_ZERO: return (int64_t)v;
    default: return (int64_t)roundf(v);  // half away from zero
  }
}

__host__ __device__ __forceinline__ int32_t mul_by_quantized_multiplier(int32_t x, int32_t m, int shift, int rmode) {
  int64_t value = shift > 0 ? (int64_t)(int32_t)((uint32_t)x << shift) : (int64_t)x;
  value = rshift_round(value * (int64_t)m, 31, B200Q_ROUND_HALF_UP);
  if (value > 2147483647ll) value = 2147483647ll;
  else if (value < -2147483648ll) value = -2147483648ll;
  if (shift < 0) value = rshift_round(value, -shift, rmode);
  return (int32_t)value;
}

__host__ __device__ __forceinline__ int64_t clamp_dtype(int64_t v, int dt) {
  int64_t lo, hi;
  switch (dt) {
    case B200Q_DT_I8: lo = -128; hi = 127; break;
    case B200Q_DT_U8: lo = 0; hi = 255; break;
    case B200Q_DT_I16: lo = -32768; hi = 32767; break;
    case B200Q_DT_U16: lo = 0; hi = 65535; break;
    default: lo = -2147483648ll; hi = 2147483647ll; break;
  }
  return v > hi ? hi : (v < lo ? lo : v);
}

// acc: int32 accumulator with bias already added (and the pre-requant ReLU already applied).
// Returns the saturated quantized value (still widened to int32).
template <int DIALECT, int RMODE>
__host__ __device__ __forceinline__ int32_t requant_value(int32_t acc, int32_t m, int32_t s, const Epilogue& e) {
  const int dialect = DIALECT >= 0 ? DIALECT : e.dialect;
  const int rmode = RMODE >= 0 ? RMODE : e.round_mode;
  int64_t v;
  switch (dialect) {
    case B200Q_RQ_MULTIPLIER_SHIFT:
      if (RMODE == B200Q_ROUND_HALF_UP && s >= 1 && s <= 62) {
        // half-up: val + (mant >= half) == floor((x + half) / 2^s); |x| < 2^62 so the add cannot overflow
        v = ((int64_t)acc * (int64_t)m + (int64_t)(1ull << (s - 1))) >> s;
      } else {
        v = rshift_round((int64_t)acc * (int64_t)m, s, rmode);
      }
      break;
    case B200Q_RQ_QDM:
      if (RMODE == B200Q_ROUND_HALF_AWAY_FROM_ZERO && s <= 0 && s >= -31) {
        // first stage in 64 bits (same floor((x + 2^30) / 2^31) identity), second stage in 32 bits:
        // the clamped first-stage value fits int32, and for a right shift by t in [1,31]
        //   half away from zero  <=>  (v >> t) + ((v & (2^t - 1)) + (v >= 0) > 2^(t-1))
        int64_t w = ((int64_t)acc * (int64_t)m + (1ll << 30)) >> 31;
        if (w > 2147483647ll) w = 2147483647ll;  // only acc == m == INT32_MIN gets here
        const int32_t v32 = (int32_t)w;
        const int t = -s;
        if (t == 0) {
          v = v32;
        } else {
          const int32_t mant = v32 & (int32_t)((1u << t) - 1u);
          v = (v32 >> t) + (int32_t)((mant + (int32_t)(v32 >= 0)) > (int32_t)(1u << (t - 1)));
        }
      } else {
        v = mul_by_quantized_multiplier(acc, m, s, rmode);
      }
      break;
    case B200Q_RQ_MULTIPLIER_SHIFT_F32: {
#ifdef __CUDA_ARCH__
      const float f = __fdiv_rn(__fmul_rn((float)acc, (float)m), (float)(1 << s));
#else
      const float f = ((float)acc * (float)m) / (float)(1 << s);
#endif
      v = to_int_f32(f, rmode);
      break;
    }
    case B200Q_RQ_ONLY_SHIFT: v = rshift_round((int64_t)acc, s, rmode); break;
    case B200Q_RQ_ONLY_SCALE: {
#ifdef __CUDA_ARCH__
      v = (int64_t)(int32_t)roundf(__fmul_rn((float)acc, e.scale));
#else
      v = (int64_t)(int32_t)roundf((float)acc * e.scale);
#endif
      break;
    }
    default: return acc;  // B200Q_RQ_NONE: raw int32
  }
  v += e.out_zp;
  if (e.relu == B200Q_RELU_AFTER_REQUANT && v < e.out_zp) v = e.out_zp;
  return (int32_t)clamp_dtype(v, e.out_dtype);
}

}  // namespace b200q
