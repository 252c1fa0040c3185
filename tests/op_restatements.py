"""Numpy / Python restatements of some ops of the wider op set, written from the reference's loops.  The GPU tests hold
the kernels to them (tests/test_gpu_more_ops.py); the CPU test tests/test_oracle_more_ops.py holds THEM to the reference's own
code where that could be compiled here (oracle/_ref/moreops_ref.so)."""
import math

import numpy as np

# Tpu_ActiveMode numbering (include/tpu_mlir/Dialect/Tpu/IR/TpuOps.td:284-321)
ACTIVE_MODES = {n: i for i, n in enumerate(
    "TANH SIGMOID RELU EXP ELU SQRT SQUARE RSQRT ABSVAL LN ROUND CEIL FLOOR SIN COS IS_FINITE MISH SWISH HSWISH SILU ARCSIN ARCCOS "
    "ARCSINH ARCCOSH ARCTANH SINH COSH TAN SIGN GELU ERF HSIGMOID LOG_SIGMOID SOFT_PLUS SOFT_SIGN LOG2 TGELU QGELU".split())}


def active_table():
    """mode -> (input domain, double function, coeffs): lib/Support/ActiveUtils.cpp:16-149.  Domains: 'x' any value, 'pos'
    positive values, 'unit' values inside (-1, 1)."""
    sig = lambda v: 1 / (1 + math.exp(-v))  # noqa: E731
    return {
        "TANH": ("x", math.tanh, None), "SIGMOID": ("x", sig, None), "EXP": ("x", math.exp, None),
        "ELU": ("x", lambda v: v if v > 0 else 0.7 * (math.exp(v) - 1), [0.7]), "SQRT": ("pos", math.sqrt, None), "SQUARE": ("x", lambda v: v * v, None),
        "RSQRT": ("pos", lambda v: 1.0 / math.sqrt(v), None), "ABSVAL": ("x", abs, None), "LN": ("pos", math.log, None),
        "ROUND": ("x", lambda v: math.copysign(math.floor(abs(v) + 0.5), v), None), "CEIL": ("x", math.ceil, None), "FLOOR": ("x", math.floor, None),
        "SIN": ("x", math.sin, None), "COS": ("x", math.cos, None), "SWISH": ("x", lambda v: v / (1 + math.exp(-v * 1.3)), [1.3]),
        "HSWISH": ("x", lambda v: v * max(0.0, min(1.0, (v + 3.0) / 6.0)), None), "SILU": ("x", lambda v: v / (1 + math.exp(-v)), None),
        "ARCCOS": ("unit", math.acos, None), "ARCTANH": ("unit", math.atanh, None), "SINH": ("x", math.sinh, None), "COSH": ("x", math.cosh, None),
        "TAN": ("unit", math.tan, None), "SIGN": ("x", lambda v: -1.0 if v < 0 else 1.0, None),
        "GELU": ("x", lambda v: 0.5 * v * (1 + math.erf(v / math.sqrt(2.0))), None), "ERF": ("x", math.erf, None),
        "HSIGMOID": ("x", lambda v: max(0.0, min(1.0, 0.2 * v + 0.5)), [0.5, 0.2]), "LOG_SIGMOID": ("x", lambda v: math.log(sig(v)), None),
        "SOFT_PLUS": ("x", lambda v: v if v > 20 else math.log(math.exp(v) + 1), None), "SOFT_SIGN": ("x", lambda v: v / (1 + abs(v)), None),
        "LOG2": ("pos", math.log2, None),
        "TGELU": ("x", lambda v: 0.5 * v * (1.0 + math.tanh(v * 0.7978845608 * (1.0 + 0.044715 * v * v))), None),
        "QGELU": ("x", lambda v: v * sig(1.702 * v), None),
    }


def grid_sampler_ref(x, grid, mode, padding, align):
    """GridSamplerFunc::invoke for a 4-D grid (lib/Support/GenericCpuFunc.cpp:3332-3455) in numpy float32 scalars."""
    f = np.float32
    N, C, IH, IW = x.shape
    OH, OW = grid.shape[1:3]

    def clip(v, lim):
        return min(f(lim - 1), max(v, f(0)))

    def reflect(v, lo2, hi2):
        if lo2 == hi2:
            return f(0)
        mn, span = f(lo2) / f(2), f(hi2 - lo2) / f(2)
        v = f(abs(f(v - mn)))
        extra = f(math.fmod(v, span))
        flips = int(math.floor(f(v / span)))
        return f(extra + mn) if flips % 2 == 0 else f(f(span - extra) + mn)

    def index(coord, size):
        r = f(f(f(coord + f(1)) * f(.5)) * f(size - 1)) if align else f(f(f(f(coord + f(1)) * f(size)) - f(1)) * f(.5))
        if padding == 1:
            r = clip(r, size)
        elif padding == 2:
            r = clip(reflect(r, 0, 2 * (size - 1)) if align else reflect(r, -1, 2 * size - 1), size)
        return f(r)
    y = np.zeros((N, C, OH, OW), np.float32)
    for n in range(N):
        for h in range(OH):
            for w in range(OW):
                fx, fy = index(grid[n, h, w, 0], IW), index(grid[n, h, w, 1], IH)
                if mode == 0:
                    xx, yy = int(math.floor(fx)), int(math.floor(fy))
                    dx, dy = f(fx - f(xx)), f(fy - f(yy))
                    tx, ty = f(f(1) - dx), f(f(1) - dy)
                    for c in range(C):
                        o = f(0)
                        for (py, px, wt) in ((yy, xx, f(tx * ty)), (yy, xx + 1, f(dx * ty)), (yy + 1, xx, f(tx * dy)), (yy + 1, xx + 1, f(dx * dy))):
                            if 0 <= py < IH and 0 <= px < IW:
                                o = f(o + f(x[n, c, py, px] * wt))
                        y[n, c, h, w] = o
                else:
                    xx, yy = int(np.rint(fx)), int(np.rint(fy))
                    if 0 <= yy < IH and 0 <= xx < IW:
                        y[n, :, h, w] = x[n, :, yy, xx]
    return y


def interp_ref(x, oh, ow, mode, coord_mode, platform):
    """interp_core with the mode resolution of InterpOp::inference (lib/Dialect/Top/Interfaces/Interp.cpp:28-181,:226-287)."""
    f = np.float32
    coord = {"half_pixel": 0, "pytorch_half_pixel": 1, "align_corners": 2, "asymmetric": 3}[coord_mode]
    if mode == "nearest":
        sp = {"CAFFE": "caffe_nearest", "TORCH": "pytorch_nearest", "TFLITE": "tf_nearest"}.get(platform, "onnx_nearest")
        align, half = coord != 3, False
    else:
        sp = "caffe" if platform == "CAFFE" else "pytorch"
        align, half = coord == 2, coord in (0, 1)

    def scale(i, o):
        if sp in ("caffe", "caffe_nearest") or (sp in ("tf_nearest", "pytorch", "onnx_nearest") and align):
            if o <= 1:
                return f(0)
            i, o = i - 1, o - 1
        return f(i) / f(o)

    def bmap(o, sc, d):
        o, hi = f(o), f(d - 1)
        clampf = lambda v: min(max(f(v), f(0)), hi)  # noqa: E731
        rnd = lambda v: int(math.floor(abs(v) + 0.5) * (1 if v >= 0 else -1))  # noqa: E731
        if sp == "tf_nearest":
            xs = clampf(f(f(o + f(.5)) * sc) if half else f(o * sc))
            return xs, (rnd(xs) if align else int(math.floor(xs)))
        if sp == "pytorch":
            xs = clampf(f(o * sc) if align else f(f(f(o + f(.5)) * sc) - f(.5)))
            return xs, int(math.floor(xs))
        if sp == "onnx_nearest" and not half:
            xs = clampf(f(o * sc))
            return xs, (rnd(xs) if align else int(math.floor(xs)))
        xs = clampf(f(o * sc))
        return xs, int(math.floor(xs))
    n, c, ih, iw = x.shape
    hs, ws = scale(ih, oh), scale(iw, ow)
    Y = [bmap(o, hs, ih) for o in range(oh)]
    X = [bmap(o, ws, iw) for o in range(ow)]
    out = np.zeros((n, c, oh, ow), np.float32)
    for p_ in range(n):
        for q_ in range(c):
            src = x[p_, q_]
            if sp in ("pytorch", "caffe"):
                buf = np.zeros((oh, iw), np.float32)
                for yo, (ys, yi) in enumerate(Y):
                    buf[yo] = src[ih - 1] if yi == ih - 1 else src[yi] + f(ys - f(yi)) * (src[yi + 1] - src[yi])
                for xo, (xs, xi) in enumerate(X):
                    out[p_, q_, :, xo] = buf[:, iw - 1] if xi == iw - 1 else buf[:, xi] + f(xs - f(xi)) * (buf[:, xi + 1] - buf[:, xi])
            else:
                for yo, (_, yi) in enumerate(Y):
                    for xo, (_, xi) in enumerate(X):
                        out[p_, q_, yo, xo] = src[yi, xi]
    return out


def d2s_ref(x, out_shape, bh, bw, crd, inv, in_nchw, out_nchw, swap):
    """Depth2Space.cpp:19-103, loop for loop."""
    def nchw(shape, f):
        return (shape[0], shape[1], shape[2], shape[3]) if f else (shape[0], shape[3], shape[1], shape[2])
    n_, ic, ih, iw = nchw(x.shape, in_nchw)
    on, oc, oh, ow = nchw(out_shape, out_nchw)
    ist = [ic * ih * iw, ih * iw, iw, 1] if in_nchw else [ic * ih * iw, 1, iw * ic, ic]
    ost = [oc * oh * ow, oh * ow, ow, 1] if out_nchw else [oc * oh * ow, 1, ow * oc, oc]
    if inv:
        n_, on, ic, oc, ih, oh, iw, ow, ist, ost = on, n_, oc, ic, oh, ih, ow, iw, ost, ist
    src = x.ravel()
    dst = np.zeros(int(np.prod(out_shape)), x.dtype)
    for i in range(n_ * ic):
        n, c = divmod(i, ic)
        if crd:
            new_c, left = divmod(c, bh * bw)
        else:
            new_c, left = c % oc, c // oc
        if swap:
            c1, c2 = divmod(left, bw)
            rleft = c2 * bh + c1
            c = new_c * (bh * bw) + rleft if crd else rleft * oc + new_c
        for h in range(ih):
            for w in range(iw):
                ii = n * ist[0] + c * ist[1] + h * ist[2] + w * ist[3]
                oi = n * ost[0] + new_c * ost[1] + (h * bh + left // bw) * ost[2] + (w * bw + left % bw) * ost[3]
                if inv:
                    dst[ii] = src[oi]
                else:
                    dst[oi] = src[ii]
    return dst.reshape(out_shape)
