"""CPU oracle (TEST INFRASTRUCTURE ONLY) for the quantized-inference hot path.

numpy/ctypes face of ``tpu_oracle.c`` plus the few lines of Python control flow the reference
keeps in ``python/calibration/kld_calibrator.py``.  Only the test-suite, the smoke check and the
CPU-baseline leg of the benchmark may import this package; the shipped library never does.

Pinning status
--------------
* rounding / requantisation helpers (to_int, RightShiftRound, MultiplyByQuantizedMultiplier,
  applyMultiplierAndRShift): pinned against the reference's own functions, compiled out of
  ``lib/Support/MathUtils.cpp:179-213,:474-562`` into ``oracle/_ref/mathutils_ref.so`` by ``oracle/Makefile``, and
  by the known answers in the reference header ``include/tpu_mlir/Support/MathUtils.h:29-40``.
* bf16 rounding: pinned against the reference's own ``lib/Support/Float16.cpp``, compiled whole from the checkout
  into ``oracle/_ref/float16_ref.so`` (``oracle/ref_shim`` stands in for the one header that needs MLIR).
* histogram / combine_histogram / find_threshold / KLD: pinned by golden vectors generated from the
  reference's own ``python/calibration/cali_math.py`` and ``bindings/kld/calibration_math.cpp``
  (``tests/golden/make_golden.py``), and, when ``oracle/_ref/calibration_math.so`` exists, by
  calling that compiled reference directly.
* MatMul / Conv2D / A16MatMul / RequantInt(Axis) / Add / Pool2D / Cast op-level arithmetic:
  restated from the cited lines; the reference interpreter cannot be built without MLIR and
  oneDNN, so the loops around the pinned requantisation arithmetic (operand order, bias, ReLU placement,
  saturation) are *parity unpinned*.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

# enums (same numbering as the reference: TpuOps.td:160-172, MathUtils.h:28-42)
QM_TFLITE_LSHIFT, QM_TFLITE, QM_MULTIPLIER_SHIFT, QM_ONLY_SHIFT, QM_QDM, QM_ONLY_SCALE = range(6)
(RM_HALF_AWAY, RM_HALF_UP, RM_HALF_DOWN, RM_HALF_EVEN, RM_HALF_ODD, RM_HALF_TOWARDS_ZERO,
 RM_TOWARDS_ZERO, RM_AWAY_FROM_ZERO, RM_UP, RM_DOWN) = range(10)
DT_I8, DT_U8, DT_I16, DT_U16, DT_I32 = range(5)
_NP_OF_DT = {DT_I8: np.int8, DT_U8: np.uint8, DT_I16: np.int16, DT_U16: np.uint16, DT_I32: np.int32}


def build(force: bool = False) -> str:
    """Compile liboracle.so (and oracle/_ref/ when the reference checkout is present)."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "tpu_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "all"], check=True, capture_output=True)
    return so


_lib = None


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(build())
        i64, i32, f32, vp = C.c_int64, C.c_int, C.c_float, C.c_void_p
        L.orc_rshift_round.restype = i64
        L.orc_rshift_round.argtypes = [i64, i32, i32]
        L.orc_to_int_f32.restype = i64
        L.orc_to_int_f32.argtypes = [f32, i32]
        L.orc_mbqm.restype = C.c_int32
        L.orc_mbqm.argtypes = [C.c_int32, C.c_int32, i32, i32]
        L.orc_apply_multiplier_rshift.restype = i64
        L.orc_apply_multiplier_rshift.argtypes = [i64, i64, i64, i32, i32, i32]
        L.orc_saturate.restype = i64
        L.orc_saturate.argtypes = [i64, i32]
        L.orc_matmul_int8.restype = i64
        L.orc_matmul_int8.argtypes = [vp, i32, vp, i32, vp, i64, i32, i64, i64, i64, i32, i32, i32, i32, i32, i32,
                                      i32, vp, vp, f32, i32, i32, vp]
        L.orc_conv2d_int8.restype = i64
        L.orc_conv2d_int8.argtypes = [vp, i32, vp, vp] + [i64] * 16 + [i32, i32, i32, i32, vp, vp, i64, i32, i32, vp]
        L.orc_conv_requant_from_f32.restype = None
        L.orc_conv_requant_from_f32.argtypes = [vp, vp, i64, i64, i64, i32, i32, i32, vp, vp, i64, i32, i32, vp]
        L.orc_requant_int_axis.restype = None
        L.orc_requant_int_axis.argtypes = [vp, i64, i64, i64, vp, i32, i32, i32, i32, i32, vp]
        L.orc_requant_int.restype = None
        L.orc_requant_int.argtypes = [vp, i64, i64, i64, i32, i32, i32, i32, i32, vp]
        L.orc_lut.restype = None
        L.orc_lut.argtypes = [vp, i32, i64, vp, i32, vp]
        L.orc_mulshift_int8.restype = None
        L.orc_mulshift_int8.argtypes = [vp, i32, i64, i64, i64, i64, i64, i32, vp]
        L.orc_mul_int8.restype = None
        L.orc_mul_int8.argtypes = [vp, i32, vp, i32, i64, i64, i64, i32, i32, vp]
        L.orc_add_int8.restype = None
        L.orc_add_int8.argtypes = [vp, i32, vp, i32, i64, i64, i64, i64, i64, i32, i32, vp]
        L.orc_pool2d_int8.restype = None
        L.orc_pool2d_int8.argtypes = [vp, i32] + [i64] * 12 + [i32, i64, i64, i32, i32, vp]
        L.orc_cast_f32_to_q8.restype = None
        L.orc_cast_f32_to_q8.argtypes = [vp, i64, C.c_double, i32, i32, i32, vp]
        L.orc_cast_q8_to_f32.restype = None
        L.orc_cast_q8_to_f32.argtypes = [vp, i32, i64, C.c_double, i32, vp]
        L.orc_f32_to_bf16_bits.restype = C.c_uint16
        L.orc_f32_to_bf16_bits.argtypes = [f32]
        L.orc_a16matmul_w4.restype = None
        L.orc_a16matmul_w4.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, vp]
        L.orc_a16matmul_w4_f16.restype = None
        L.orc_a16matmul_w4_f16.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, vp]
        L.orc_top_conv2d_f32.restype = None
        L.orc_top_conv2d_f32.argtypes = [vp, vp, vp] + [i64] * 16 + [i32, f32, vp]
        L.orc_top_pool2d_f32.restype = None
        L.orc_top_pool2d_f32.argtypes = [vp] + [i64] * 11 + [i32, i32, i32, f32, vp]
        L.orc_f32_to_f16_bits.restype = C.c_uint16
        L.orc_f32_to_f16_bits.argtypes = [f32]
        L.orc_f16_bits_to_f32.restype = C.c_float
        L.orc_f16_bits_to_f32.argtypes = [C.c_uint16]
        L.orc_a16_dequant_w4.restype = None
        L.orc_a16_dequant_w4.argtypes = [vp, vp, vp, i64, i64, i64, vp]
        L.orc_histogram_f32.restype = None
        L.orc_histogram_f32.argtypes = [vp, i64, f32, i64, vp]
        L.orc_kl_diversity_hist.restype = f32
        L.orc_kl_diversity_hist.argtypes = [vp, f32, i64, i64, vp]
        L.orc_num_threads.restype = i32
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt=None):
    return None if a is None else np.ascontiguousarray(a, dtype=dt)


def _is_u(a):
    assert a.dtype in (np.int8, np.uint8), a.dtype
    return int(a.dtype == np.uint8)


def num_threads() -> int:
    return int(lib().orc_num_threads())


# --------------------------------------------------------------------------- scalar helpers
def rshift_round(x, s, rmode):
    return int(lib().orc_rshift_round(int(x), int(s), int(rmode)))


def to_int(v, rmode):
    return int(lib().orc_to_int_f32(float(v), int(rmode)))


def mbqm(x, m, shift, rmode=RM_HALF_AWAY):
    return int(lib().orc_mbqm(int(x), int(m), int(shift), int(rmode)))


def apply_multiplier_rshift(v, m, s, qmode=QM_MULTIPLIER_SHIFT, rmode=RM_HALF_UP, is_cv18xx=False):
    return int(lib().orc_apply_multiplier_rshift(int(v), int(m), int(s), int(qmode), int(rmode), int(is_cv18xx)))


def saturate(v, dt):
    return int(lib().orc_saturate(int(v), int(dt)))


def through_f32(values) -> np.ndarray:
    """Integers as the interpreter sees them after a trip through its float32 operand buffers
    ((int64_t)float; MatMul.cpp:709-716, RequantIntAxis.cpp:45-48)."""
    return np.asarray(values, dtype=np.int64).astype(np.float32).astype(np.int64)


# --------------------------------------------------------------------------- ops
def matmul_int8(A, B, bias=None, *, right_transpose=False, input_zp=0, right_zp=0, do_relu=False,
                qmode=QM_MULTIPLIER_SHIFT, is_cv18xx=False, fuse_rq=False, mult=None, rshift=None,
                only_scale=0.0, out_zp=0, out_dt=DT_I8, return_violations=False):
    """tpu.MatMul on quantized operands (MatMul.cpp:599-603,:636-728).  A [..,M,K]; B [K,N], [N,K] when
    right_transpose, or batched [b,K,N].  mult=None with out_dt=DT_I32 returns the raw accumulator."""
    A = _c(A)
    B = _c(B)
    K = A.shape[-1]
    if B.ndim == 3:
        batch, b_batched = B.shape[0], 1
        M = A.size // (batch * K)
    else:
        batch, b_batched = 1, 0
        M = A.size // K
    N = B.shape[-2] if right_transpose else B.shape[-1]
    assert (B.shape[-1] if right_transpose else B.shape[-2]) == K
    bias = _c(bias, np.int32)
    mult = _c(mult, np.int64)
    rshift = _c(rshift, np.int64)
    out = np.empty(A.shape[:-1] + (N,), dtype=_NP_OF_DT[out_dt])
    viol = lib().orc_matmul_int8(_p(A), _is_u(A), _p(B), _is_u(B), _p(bias), batch, b_batched, M, K, N,
                                 int(right_transpose), input_zp, right_zp, int(do_relu), qmode, int(is_cv18xx),
                                 int(fuse_rq), _p(mult), _p(rshift), float(only_scale), out_zp, out_dt, _p(out))
    return (out, int(viol)) if return_violations else out


def conv2d_int8(x, w, bias=None, *, stride=(1, 1), pads=(0, 0, 0, 0), dilation=(1, 1), groups=1, pad_value=0,
                do_relu=False, qmode=QM_MULTIPLIER_SHIFT, is_cv18xx=False, mult=None, rshift=None, out_zp=0,
                out_dt=DT_I8, return_violations=False):
    """tpu.Conv2D with uniform-quantized output (Conv2D.cpp:88-344).  x NCHW s8/u8, w [OC,IC/g,KH,KW] s8,
    pads = (top, bottom, left, right) (pht, phb, pwl, pwr of conv_attr_t)."""
    x = _c(x)
    w = _c(w, np.int8)
    n, ic, ih, iw = x.shape
    oc, _, kh, kw = w.shape
    pht, phb, pwl, pwr = pads
    oh = (ih + pht + phb - dilation[0] * (kh - 1) - 1) // stride[0] + 1
    ow = (iw + pwl + pwr - dilation[1] * (kw - 1) - 1) // stride[1] + 1
    bias = _c(bias, np.int32)
    mult = _c(np.atleast_1d(mult), np.int64)
    rshift = _c(np.atleast_1d(rshift), np.int64)
    out = np.empty((n, oc, oh, ow), dtype=_NP_OF_DT[out_dt])
    viol = lib().orc_conv2d_int8(_p(x), _is_u(x), _p(w), _p(bias), n, ic, ih, iw, oc, kh, kw, stride[0], stride[1],
                                 dilation[0], dilation[1], pht, phb, pwl, pwr, groups, pad_value, int(do_relu),
                                 qmode, int(is_cv18xx), _p(mult), _p(rshift), rshift.size, out_zp, out_dt, _p(out))
    return (out, int(viol)) if return_violations else out


def conv2d_int8_fp32_path(x, w, bias=None, *, stride=(1, 1), pads=(0, 0, 0, 0), dilation=(1, 1), groups=1,
                          do_relu=False, qmode=QM_MULTIPLIER_SHIFT, is_cv18xx=False, mult=None, rshift=None, out_zp=0,
                          out_dt=DT_I8, threads=None):
    """The reference's own arithmetic route for an INT8 Conv2D: an fp32 oneDNN convolution over integer-valued
    floats (lib/Support/Dnnl/Conv.cpp:98-145,:234-253; here torch's CPU convolution, the same primitive family)
    followed by the float-plus-bias requant loop (Conv2D.cpp:295-341).  Symmetric zero padding only.
    This is what the CPU baseline times."""
    import torch
    import torch.nn.functional as F
    if threads:
        torch.set_num_threads(int(threads))
    xf = torch.from_numpy(np.ascontiguousarray(x)).to(torch.float32)
    wf = torch.from_numpy(np.ascontiguousarray(w)).to(torch.float32)
    pht, phb, pwl, pwr = pads
    if pht != phb or pwl != pwr:
        xf = F.pad(xf, (pwl, pwr, pht, phb))
        padding = (0, 0)
    else:
        padding = (pht, pwl)
    acc = F.conv2d(xf, wf, None, stride=stride, padding=padding, dilation=dilation, groups=groups).contiguous().numpy()
    n, oc, oh, ow = acc.shape
    mult = _c(np.atleast_1d(mult), np.int64)
    rshift = _c(np.atleast_1d(rshift), np.int64)
    out = np.empty(acc.shape, dtype=_NP_OF_DT[out_dt])
    lib().orc_conv_requant_from_f32(_p(acc), _p(_c(bias, np.int32)), n, oc, oh * ow, int(do_relu), qmode,
                                    int(is_cv18xx), _p(mult), _p(rshift), rshift.size, out_zp, out_dt, _p(out))
    return out


def requant_int_axis(x, quant3, *, qmode, rmode, fuse_rq_axis=False, in_zp=0, out_dt=DT_I8):
    """tpu.RequantIntAxis (RequantIntAxis.cpp:17-123); quant3 = int64 [C,3] {multiplier, shift, zp} as read
    back from the float operand (use through_f32)."""
    x = _c(x, np.int32)
    q = _c(quant3, np.int64)
    Cn = q.shape[0]
    if fuse_rq_axis:
        outer, inner = x.size // Cn, 1
        assert x.shape[-1] == Cn
    else:
        outer, inner = x.shape[0], x.size // (x.shape[0] * Cn)
        assert x.shape[1] == Cn
    out = np.empty(x.shape, dtype=_NP_OF_DT[out_dt])
    lib().orc_requant_int_axis(_p(x), outer, Cn, inner, _p(q), qmode, rmode, int(fuse_rq_axis), in_zp, out_dt,
                               _p(out))
    return out


def requant_int(x, multi, rshift, *, qmode, rmode, in_zp=0, out_zp=0, out_dt=DT_I8):
    """tpu.RequantInt (RequantInt.cpp:17-71)."""
    x = _c(x, np.int32)
    out = np.empty(x.shape, dtype=_NP_OF_DT[out_dt])
    lib().orc_requant_int(_p(x), x.size, int(multi), int(rshift), qmode, rmode, in_zp, out_zp, out_dt, _p(out))
    return out


def add_int8(a, b, m0, s0, m1, s1, *, do_relu=False, out_dt=DT_I8):
    """tpu.Add, symmetric int8 (Add.cpp:177-207)."""
    a, b = _c(a), _c(b)
    out = np.empty(a.shape, dtype=_NP_OF_DT[out_dt])
    lib().orc_add_int8(_p(a), _is_u(a), _p(b), _is_u(b), a.size, m0, s0, m1, s1, int(do_relu), out_dt, _p(out))
    return out


def lut(x, table):
    """tpu.Lut (Lut.cpp:20-32): out = table[x mod 256]; the table's dtype is the output's."""
    x, table = _c(x), _c(table)
    assert table.size == 256
    out = np.empty(x.shape, dtype=table.dtype)
    lib().orc_lut(_p(x), _is_u(x), x.size, _p(table), table.dtype.itemsize, _p(out))
    return out


def mulshift_int8(x, multiplier, rshift, *, in_zp=0, out_zp=0, out_dt=DT_I8):
    """tpu.MulShift (MulShift.cpp:19-41)."""
    x = _c(x)
    out = np.empty(x.shape, dtype=_NP_OF_DT[out_dt])
    lib().orc_mulshift_int8(_p(x), _is_u(x), x.size, multiplier, rshift, in_zp, out_zp, out_dt, _p(out))
    return out


def mul_int8(a, b, multiplier, rshift, *, do_relu=False, out_dt=DT_I8):
    """tpu.Mul, symmetric int8, equal shapes (Mul.cpp:72-85)."""
    a, b = _c(a), _c(b)
    out = np.empty(a.shape, dtype=_NP_OF_DT[out_dt])
    lib().orc_mul_int8(_p(a), _is_u(a), _p(b), _is_u(b), a.size, multiplier, rshift, int(do_relu), out_dt, _p(out))
    return out


def pool2d_int8(x, kernel, stride, pads, *, mode="max", multi=1, rshift=0, do_relu=False, out_dt=None):
    """tpu.Pool2D int8 (Pool2D.cpp:160-192); pads = (top, bottom, left, right)."""
    x = _c(x)
    n, c, ih, iw = x.shape
    if out_dt is None:
        out_dt = DT_U8 if x.dtype == np.uint8 else DT_I8
    oh = (ih + pads[0] + pads[1] - kernel[0]) // stride[0] + 1
    ow = (iw + pads[2] + pads[3] - kernel[1]) // stride[1] + 1
    out = np.empty((n, c, oh, ow), dtype=_NP_OF_DT[out_dt])
    lib().orc_pool2d_int8(_p(x), _is_u(x), n, c, ih, iw, kernel[0], kernel[1], stride[0], stride[1], pads[0], pads[1],
                          pads[2], pads[3], 0 if mode == "max" else 1, multi, rshift, int(do_relu), out_dt, _p(out))
    return out


def cast_f32_to_q8(x, scale, zp=0, *, rmode=RM_HALF_AWAY, out_dt=DT_I8):
    """tpu.Cast f32 -> int8/uint8 (Cast.cpp:75-93, CastUtils.cpp:15-20)."""
    x = _c(x, np.float32)
    out = np.empty(x.shape, dtype=_NP_OF_DT[out_dt])
    lib().orc_cast_f32_to_q8(_p(x), x.size, float(scale), zp, rmode, out_dt, _p(out))
    return out


def cast_q8_to_f32(x, scale, zp=0):
    """tpu.Cast int8/uint8 -> f32 (Cast.cpp:94-116)."""
    x = _c(x)
    out = np.empty(x.shape, dtype=np.float32)
    lib().orc_cast_q8_to_f32(_p(x), _is_u(x), x.size, float(scale), zp, _p(out))
    return out


def f32_to_bf16_bits(x):
    """BF16() of the reference (Float16.cpp:603-645), elementwise, returning uint16 bit patterns."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    f = lib().orc_f32_to_bf16_bits
    return np.array([f(float(v)) for v in x.ravel()], dtype=np.uint16).reshape(x.shape)


def f32_to_f16_bits(x):
    """F16() of the reference (Float16.cpp:763-767,:663-714), elementwise, returning uint16 bit patterns."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    f = lib().orc_f32_to_f16_bits
    return np.array([f(float(v)) for v in x.ravel()], dtype=np.uint16).reshape(x.shape)


def f16_bits_to_f32(b):
    """f16_to_f32 of the reference (Float16.cpp:776-786)."""
    b = np.asarray(b, dtype=np.uint16)
    f = lib().orc_f16_bits_to_f32
    return np.array([f(int(v)) for v in b.ravel()], dtype=np.float32).reshape(b.shape)


def bf16_bits_to_f32(b):
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits_fast(x):
    """Vectorised round-to-nearest-even for NORMAL finite values (what the generators need)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def a16matmul_w4(x_bits, wq, scale_bits, zp, bias=None, *, group=64, f16=False):
    """tpu.A16MatMul static w4 path with w_transpose=true (A16MatMul.cpp:171-208,:240-246).
    x_bits uint16 [M,K] (bf16, or f16 with ``f16=True``), wq uint8 [N,K/2], scale_bits uint16 [N*K/g] (same type as x),
    zp uint8 [N*K/g] -> uint16 [M,N] (same type)."""
    x_bits = _c(x_bits, np.uint16)
    wq = _c(wq, np.uint8)
    M, K = x_bits.shape
    N = wq.shape[0]
    assert wq.shape[1] * 2 == K
    y = np.empty((M, N), dtype=np.uint16)
    fn = lib().orc_a16matmul_w4_f16 if f16 else lib().orc_a16matmul_w4
    fn(_p(x_bits), _p(wq), _p(_c(scale_bits, np.uint16)), _p(_c(zp, np.uint8)), _p(_c(bias, np.float32)), M, K, N, group, _p(y))
    return y


def a16matmul_w8(x_bits, w, scale_bits, zp, bias=None, *, group=64, f16=False):
    """tpu.A16MatMul static w8 path with w_transpose=true (A16MatMul.cpp:209-246): w [N,K] integers (any of the 8-bit
    ranges), the dequantised weight (w - zp) * scale is rounded to bf16 (F16 modes: to IEEE half, :226-230) before the fp32
    matmul, the result rounded the same way.  ``group`` = K is the per-channel form (q_group_size = 0).  numpy: float64
    accumulation of exact products."""
    if f16:
        to_f = lambda b: _c(b, np.uint16).view(np.float16).astype(np.float32)  # noqa: E731
        rnd = lambda v: np.asarray(v, dtype=np.float32).astype(np.float16)  # noqa: E731  (round to nearest even, as F16())
    else:
        to_f = lambda b: bf16_bits_to_f32(_c(b, np.uint16))  # noqa: E731
        rnd = None
    x = to_f(x_bits).astype(np.float64)
    w = np.asarray(w, dtype=np.float32)
    N, K = w.shape
    s = np.repeat(to_f(scale_bits).reshape(N, K // group), group, axis=1)
    z = np.repeat(np.asarray(zp, dtype=np.float32).reshape(N, K // group), group, axis=1)
    prod = ((w - z) * s).astype(np.float32)
    W = (rnd(prod).astype(np.float64) if f16 else bf16_bits_to_f32(f32_to_bf16_bits_fast(prod)).astype(np.float64))
    y = x @ W.T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float64)
    return rnd(y.astype(np.float32)).view(np.uint16) if f16 else f32_to_bf16_bits_fast(y.astype(np.float32))


def a16_dequant_w4(wq, scale_bits, zp, *, group=64):
    wq = _c(wq, np.uint8)
    N, K = wq.shape[0], wq.shape[1] * 2
    W = np.empty((N, K), dtype=np.float32)
    lib().orc_a16_dequant_w4(_p(wq), _p(_c(scale_bits, np.uint16)), _p(_c(zp, np.uint8)), N, K, group, _p(W))
    return W


# --------------------------------------------------------------------------- calibration
def histogram(x, abs_max, bins=2048, into=None):
    """CaliMathCpu.histogram (cali_math.py:68-80).  Returns (int32 counts, float32 width); ``into`` adds the
    counts into the first ``bins`` entries of an existing (longer) int32 buffer."""
    x = _c(np.asarray(x).ravel(), np.float32)
    abs_max = np.float32(abs_max)
    hist = np.zeros(bins, dtype=np.int32) if into is None else into
    assert hist.dtype == np.int32 and hist.size >= bins and hist.flags.c_contiguous
    lib().orc_histogram_f32(_p(x), x.size, float(abs_max), bins, _p(hist))
    return hist, np.float32(abs_max / np.float32(bins - 1))


class StreamingHistogram:
    """Per-tensor state of ActivationCalibrator.process_statistic (kld_calibrator.py:391-398,:462-476)
    with CaliMathCpu.combine_histogram (cali_math.py:82-103), in float32 like the reference."""

    MAX_GROWN_BINS = 8000000

    def __init__(self, bin_num=2048):
        self.bin_num = bin_num
        self.min = float("inf")
        self.max = float("-inf")
        self.hist = None
        self.width = None
        self.th = None

    def update(self, activation):
        a = np.asarray(activation, dtype=np.float32).ravel()
        self.min = min(np.min(a), self.min)
        self.max = max(np.max(a), self.max)
        abs_value = max(abs(self.min), abs(self.max))
        if np.abs(a).max() < 1e-8:
            return
        if self.hist is None:
            self.hist, self.width = histogram(a, abs_value, self.bin_num)
            self.th = abs_value
            return
        if abs_value <= self.th:
            h, _ = histogram(a, self.th, len(self.hist))
            self.hist = self.hist + h
            return
        old_bins = len(self.hist)
        old_step = self.th / old_bins
        inc = int((abs_value - self.th) // old_step + 1)
        new_bins = inc + old_bins
        if new_bins > self.MAX_GROWN_BINS:
            self.hist, self.width = histogram(a, abs_value, self.bin_num)
            self.th = abs_value
            return
        new_th = inc * old_step + self.th
        h, w = histogram(a, new_th, new_bins)
        h[0:old_bins] += self.hist
        self.hist, self.width, self.th = h, w, new_th

    @property
    def abs_max(self):
        return max(abs(self.min), abs(self.max))


def bin_schedule(abs_values, contributes, bin_num=2048, max_bins=StreamingHistogram.MAX_GROWN_BINS):
    """The (threshold, bins) each sample's histogram is taken with, derived from the running abs-max alone
    (same arithmetic as StreamingHistogram.update).  Returns a list of (th: float32 | None, bins, reset)."""
    out = []
    th = None
    nb = None
    for a, ok in zip(abs_values, contributes):
        a = np.float32(a)
        if not ok:
            out.append((None, 0, False))
            continue
        if th is None:
            th, nb = a, bin_num
            out.append((th, nb, False))
            continue
        if a <= th:
            out.append((th, nb, False))
            continue
        step = th / nb
        inc = int((a - th) // step + 1)
        if inc + nb > max_bins:
            th, nb = a, bin_num
            out.append((th, nb, True))
            continue
        th = inc * step + th
        nb = inc + nb
        out.append((np.float32(th), nb, False))
    return out


def fold_for_kld(hist, width, dst_bins=128, max_bins=64 * 2048):
    """ActivationCalibrator.find_threshold's preparation (kld_calibrator.py:329-342): zero-pad to a multiple
    of dst_bins, pairwise-fold while longer than max_bins (doubling the width)."""

    def pad(h):
        r = len(h) % dst_bins
        return h if r == 0 else np.concatenate((h, np.zeros(dst_bins - r, dtype=h.dtype)))

    h = pad(np.asarray(hist))
    w = width
    while len(h) > max_bins:
        h = pad(h[::2] + h[1::2])
        w = w * 2.0
    return h, w


def kl_diversity_hist(hist, width, dst_bins=128, return_kl=False):
    """Restated kl_diversity_hist (calibration_math.cpp:158-212,:273-323)."""
    h = _c(hist, np.int32)
    kl = np.empty(h.size // dst_bins, dtype=np.float32)
    th = lib().orc_kl_diversity_hist(_p(h), float(np.float32(width)), h.size, dst_bins, _p(kl))
    return (np.float32(th), kl) if return_kl else np.float32(th)


_ref_kld = None


def ref_kld_available() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "calibration_math.so"))


def ref_kl_diversity_hist(hist, width, dst_bins=128):
    """The reference's own compiled bindings/kld/calibration_math.cpp (oracle/_ref/), called the way
    kld_calibrator.py:50-59 does."""
    global _ref_kld
    if _ref_kld is None:
        L = C.CDLL(os.path.join(_HERE, "_ref", "calibration_math.so"))
        L.kl_diversity_hist.restype = C.c_float
        _ref_kld = L
    h = _c(hist, np.int32)
    return np.float32(_ref_kld.kl_diversity_hist(h.ctypes.data_as(C.POINTER(C.c_int)), C.c_float(float(width)),
                                                 C.c_longlong(h.size), C.c_longlong(dst_bins)))


# ------------------------------------------------------------------------------------------------------------
# The reference's own rounding / requantisation functions (lib/Support/MathUtils.cpp:179-213,:474-562), compiled by
# oracle/Makefile (target ref_mathutils) out of the reference checkout into oracle/_ref/mathutils_ref.so.
_ref_mu = None


def ref_mathutils_available() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "mathutils_ref.so"))


def ref_mathutils():
    global _ref_mu
    if _ref_mu is None:
        L = C.CDLL(os.path.join(_HERE, "_ref", "mathutils_ref.so"))
        i32, i64 = C.c_int, C.c_longlong
        L.ref_to_int_f32.restype, L.ref_to_int_f32.argtypes = i64, [C.c_float, i32]
        L.ref_rshift_round.restype, L.ref_rshift_round.argtypes = i64, [i64, i32, i32]
        L.ref_mbqm.restype, L.ref_mbqm.argtypes = i32, [i32, i32, i32, i32]
        L.ref_apply_multiplier_rshift.restype = i64
        L.ref_apply_multiplier_rshift.argtypes = [i64, i64, i64, i32, i32, i32]
        _ref_mu = L
    return _ref_mu


_ref_f16 = None


def ref_float16_available() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "float16_ref.so"))


def ref_float16():
    """The reference's own lib/Support/Float16.cpp compiled into oracle/_ref/float16_ref.so (BM168x conversions)."""
    global _ref_f16
    if _ref_f16 is None:
        L = C.CDLL(os.path.join(_HERE, "_ref", "float16_ref.so"))
        L.ref_f32_to_bf16.restype, L.ref_f32_to_bf16.argtypes = C.c_uint, [C.c_float]
        L.ref_bf16_to_f32.restype, L.ref_bf16_to_f32.argtypes = C.c_float, [C.c_uint]
        L.ref_f32_to_f16.restype, L.ref_f32_to_f16.argtypes = C.c_uint, [C.c_float]
        L.ref_f16_to_f32.restype, L.ref_f16_to_f32.argtypes = C.c_float, [C.c_uint]
        _ref_f16 = L
    return _ref_f16


def ref_oploops_available() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "oploops_ref.so"))


_ref_oploops = None


def ref_oploops():
    """The reference's own operator loops (requantisation of Conv2D / MatMul, Add, average pool, A16 dequantisation,
    RequantInt(Axis), Cast, saturate), cut from the checkout and compiled by `make -C oracle ref_oploops`."""
    global _ref_oploops
    if _ref_oploops is None:
        L = C.CDLL(os.path.join(_HERE, "_ref", "oploops_ref.so"))
        i32, i64, f32, f64, vp = C.c_int, C.c_longlong, C.c_float, C.c_double, C.c_void_p
        L.ref_saturate_i64.restype, L.ref_saturate_i64.argtypes = i64, [i64, i32, i32]
        L.ref_saturate_f32.restype, L.ref_saturate_f32.argtypes = i64, [f32, i32, i32, i32]
        L.ref_conv2d_requant.restype = None
        L.ref_conv2d_requant.argtypes = [vp, i64, i64, i64, vp, i32, vp, i32, vp, i32, i32, i64, i32, i32, i32]
        L.ref_matmul_requant.restype = None
        L.ref_matmul_requant.argtypes = [vp, i64, i64, i64, vp, i32, vp, i32, vp, i32, i32, f64, i64, i32, i32, i32, i32]
        L.ref_add_int8.restype = None
        L.ref_add_int8.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i32, i32, i32]
        L.ref_avgpool_int8.restype = None
        L.ref_avgpool_int8.argtypes = [vp, i64, i32, i32, i32, i64, i32, i64, i32, i32, i32, i32]
        L.ref_a16_dequant_w4.restype = None
        L.ref_a16_dequant_w4.argtypes = [vp, vp, vp, i64, i64, i32, vp]
        L.ref_requant_int_axis.restype = None
        L.ref_requant_int_axis.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i64, i32, i32]
        L.ref_requant_int.restype = None
        L.ref_requant_int.argtypes = [vp, vp, vp, i32, i64, i64, i32, i32, i32, i64, i64, i32, i32]
        L.ref_cast_requant.restype, L.ref_cast_requant.argtypes = f32, [f32, f64, i64, i32]
        L.ref_cast_dequant.restype, L.ref_cast_dequant.argtypes = f32, [f32, f64, i64, i32]
        _ref_oploops = L
    return _ref_oploops


# ------------------------------------------------------------------ fp32 Top-dialect forward
def top_conv2d_f32(x, w, bias=None, *, stride=(1, 1), pads=(0, 0, 0, 0), dilation=(1, 1), groups=1, do_relu=False,
                   relu_limit=-1.0):
    """top::ConvOp::inference (lib/Dialect/Top/Interfaces/Conv.cpp:222-231): NCHW x, OIHW w, pads = (top, bottom, left,
    right); double accumulation in index order (oneDNN's order is not defined: compare by tolerance)."""
    x, w, bias = _c(x, np.float32), _c(w, np.float32), _c(bias, np.float32)
    n, ic, ih, iw = x.shape
    oc, icg, kh, kw = w.shape
    assert icg * groups == ic
    oh = (ih + pads[0] + pads[1] - dilation[0] * (kh - 1) - 1) // stride[0] + 1
    ow = (iw + pads[2] + pads[3] - dilation[1] * (kw - 1) - 1) // stride[1] + 1
    out = np.empty((n, oc, oh, ow), np.float32)
    lib().orc_top_conv2d_f32(_p(x), _p(w), _p(bias), n, ic, ih, iw, oc, kh, kw, stride[0], stride[1], dilation[0],
                             dilation[1], pads[0], pads[1], pads[2], pads[3], groups, int(do_relu), float(relu_limit), _p(out))
    return out


def top_pool2d_f32(x, *, kernel, stride, pads=(0, 0, 0, 0), is_max=True, count_include_pad=False, do_relu=False,
                   relu_limit=-1.0):
    """top::MaxPoolOp / top::AvgPoolOp over NCHW (lib/Support/Dnnl/Pool.cpp)."""
    x = _c(x, np.float32)
    n, c, ih, iw = x.shape
    oh = (ih + pads[0] + pads[1] - kernel[0]) // stride[0] + 1
    ow = (iw + pads[2] + pads[3] - kernel[1]) // stride[1] + 1
    out = np.empty((n, c, oh, ow), np.float32)
    lib().orc_top_pool2d_f32(_p(x), n * c, ih, iw, kernel[0], kernel[1], stride[0], stride[1], pads[0], pads[1], pads[2],
                             pads[3], int(is_max), int(count_include_pad), int(do_relu), float(relu_limit), _p(out))
    return out
