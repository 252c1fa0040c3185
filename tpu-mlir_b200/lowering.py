"""Parameter generation for an INT8 Tpu-dialect graph (restating the parts of the TOP->TPU lowering that
produce the numbers the hot path consumes).  The lowering itself stays in the reference; these functions exist
so that a faithful INT8 ResNet-50 graph can be generated where no MLIR toolchain is available.

Sources (paths inside the tpu-mlir tree):
  get_scale_and_shift / _positive   lib/Support/MathUtils.cpp:20-51
  storage type and scale            lib/Support/Module.cpp:1844-1867,:1907-1916; lib/Conversion/TopToTpu/TopLowering.cpp:389-411
  Conv  INT8                        lib/Conversion/TopToTpu/BM1684X/Conv.cpp:56-212
  MatMul INT8 (weight right operand) lib/Conversion/TopToTpu/BM1684X/MatMul.cpp:96-277
  Add   INT8                        lib/Conversion/TopToTpu/BM1684X/Add.cpp:48-120
  AvgPool INT8                      lib/Conversion/TopToTpu/BM1684X/AvgPool.cpp:34-104
  calibration import (symmetric)    lib/Dialect/Top/Transforms/ImportCalibration.cpp:105-115,:171-236
"""
from __future__ import annotations

import numpy as np

INT_MAX, CHAR_MAX = 2**31 - 1, 127


def _c_int(v: float) -> int:
    """(int)double on x86: out-of-range values become INT_MIN."""
    if not np.isfinite(v) or v >= 2**31 or v < -2**31:
        return -2**31
    return int(v)


def _c_round(v: float) -> float:
    """std::round: half away from zero."""
    return float(np.floor(abs(v) + 0.5) * (1 if v >= 0 else -1))


def get_scale_and_shift(scale_f, bitwidth=32, n_range=range(-32, 31)):
    """MathUtils.cpp:20-36.  The argument is a C `float`; m/2^n and the error are evaluated in double and the
    error is stored in a float."""
    scale_f = float(np.float32(scale_f))
    m_limit = INT_MAX if bitwidth == 32 else CHAR_MAX
    min_err, shift = np.float32(np.finfo(np.float32).max), 0
    for n in n_range:
        p = 2.0 ** n
        m = _c_int(_c_round(scale_f * p))
        err = np.float32(abs(m / p - scale_f))
        if err < min_err and abs(m) < m_limit:
            min_err, shift = err, n
    return _c_int(_c_round(scale_f * 2.0 ** shift)), shift


def get_scale_and_shift_positive(scale_f, bitwidth=32):
    """MathUtils.cpp:38-51 (right shifts only)."""
    return get_scale_and_shift(scale_f, bitwidth, range(0, 31))


def to_int8(v):
    """to_int8 (MathUtils.h:325-330): round half away from zero, saturate."""
    v = np.asarray(v, dtype=np.float64)
    r = np.where(v >= 0, np.floor(v + 0.5), -np.floor(-v + 0.5))
    return np.clip(r, -128, 127).astype(np.int8)


def tensor_qtype(threshold: float, vmin: float, relu_output: bool):
    """Symmetric calibrated type -> (storage dtype, scale).  ImportCalibration sets min = -threshold when the
    observed minimum is negative, else 0, and 0 when the producing op has a fused ReLU; the storage type is
    unsigned when min >= 0 (Module.cpp:1907-1916) and the scale th/255 or th/127 (Module.cpp:1844-1867)."""
    signed = (vmin < 0) and not relu_output
    return ("i8", threshold / 127.0) if signed else ("u8", threshold / 255.0)


def lower_conv(w: np.ndarray, b, in_scale: float, out_scale: float):
    """Per-output-channel symmetric weights, MultiplierShift requant (Conv.cpp:82-212).  Returns
    (w_int8, bias_int32, multipliers, rshifts)."""
    oc = w.shape[0]
    wf = w.reshape(oc, -1).astype(np.float32)
    w_q = np.empty_like(wf, dtype=np.int8)
    mult, rshift = [], []
    bias_q = np.zeros(oc, np.int32)
    for c in range(oc):
        w_max = np.float32(np.abs(wf[c]).max())
        scale_w = float(max(np.float32(w_max / np.float32(127.0)), np.float32(1e-5)))
        m, s = get_scale_and_shift(scale_w * in_scale / out_scale, 32)
        mult.append(m)
        rshift.append(s)
        w_q[c] = to_int8(wf[c].astype(np.float64) / scale_w)
        if b is not None:
            bias_q[c] = int(_c_round(float(b[c]) / (scale_w * in_scale)))
    return w_q.reshape(w.shape), bias_q, np.array(mult, np.int64), np.array(rshift, np.int64)


def lower_fc(w_kn: np.ndarray, b, in_scale: float, out_scale: float):
    """Per-tensor symmetric weight [K,N], MultiplierShift (MatMul.cpp:96-277, no per-channel attribute)."""
    w_scale = float(np.float32(np.abs(w_kn).max())) / 127.0
    w_q = to_int8(w_kn.astype(np.float64) / w_scale)
    bias_q = None
    if b is not None:
        bias_q = np.array([int(_c_round(float(v) / (w_scale * in_scale))) for v in b], np.int32)
    m, s = get_scale_and_shift(np.float32(in_scale * w_scale / out_scale), 32)
    return w_q, bias_q, m, s


def lower_add(in_scales, out_scale: float):
    """Add.cpp:98-108: per input get_scale_and_shift_positive(scale_i / out_scale, 8)."""
    ms = [get_scale_and_shift_positive(s / out_scale, 8) for s in in_scales]
    return [m for m, _ in ms], [s for _, s in ms]


def lower_avgpool(in_scale: float, out_scale: float, kh: int, kw: int):
    """AvgPool.cpp:70-79: get_scale_and_shift(in_scale / (out_scale * kh * kw), 8)."""
    return get_scale_and_shift(in_scale / (out_scale * kh * kw), 8)
