"""The tests' restatements of some ops of the wider op set (tests/op_restatements.py and the expressions the GPU tests use)
against the reference's OWN code for them, compiled from the checkout into oracle/_ref/moreops_ref.so (oracle/Makefile,
target ref_moreops): interp_core, GridSamplerFunc, the activation table, swap_dim_data, pad_tensor_for_deconv,
tensor_hc_transpose, and the whole inference bodies of top.Depth2Space, top.Gather, top.Arg and gather_dim8.  Skipped where that library could not be built."""
import ctypes as C
import os

import numpy as np
import pytest

from op_restatements import ACTIVE_MODES, active_table, d2s_ref, grid_sampler_ref, interp_ref

REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "moreops_ref.so")
pytestmark = pytest.mark.skipif(not os.path.exists(REF), reason="oracle/_ref/moreops_ref.so was not built (no reference checkout)")


@pytest.fixture(scope="module")
def ref():
    return C.CDLL(REF)


def fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


# PLATFORM_SUPPORT (include/tpu_mlir/Backend/BM168x/Param.h:197-206) as InterpOp::inference picks it (Interp.cpp:226-279)
def platform_sp(mode, coord_mode, platform):
    coord = {"half_pixel": 0, "pytorch_half_pixel": 1, "align_corners": 2, "asymmetric": 3}[coord_mode]
    if mode == "nearest":
        sp = {"CAFFE": 2, "TORCH": 5, "TFLITE": 3}.get(platform, 7)
        return sp, coord != 3, False
    return (0 if platform == "CAFFE" else 4), coord == 2, coord in (0, 1)


@pytest.mark.parametrize("mode", ["nearest", "linear"])
@pytest.mark.parametrize("coord", ["half_pixel", "pytorch_half_pixel", "align_corners", "asymmetric"])
@pytest.mark.parametrize("platform", ["ONNX", "TORCH", "TFLITE", "CAFFE"])
def test_interp_restatement(ref, mode, coord, platform):
    rng = np.random.default_rng(1)
    for (ih, iw, oh, ow) in ((5, 7, 9, 11), (6, 4, 3, 2), (4, 4, 8, 8), (3, 5, 1, 1), (1, 3, 4, 9)):
        x = rng.standard_normal((1, 1, ih, iw)).astype(np.float32)
        want = np.zeros((oh, ow), np.float32)
        sp, align, half = platform_sp(mode, coord, platform)
        ref.ref_interp_plane(fp(x), fp(want), ih, iw, oh, ow, int(align), int(half), sp)
        assert np.array_equal(interp_ref(x, oh, ow, mode, coord, platform)[0, 0], want), (ih, iw, oh, ow)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("padding", [0, 1, 2])
@pytest.mark.parametrize("align", [False, True])
def test_grid_sampler_restatement(ref, mode, padding, align):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((2, 3, 5, 7)).astype(np.float32)
    grid = (rng.random((2, 4, 6, 2)) * 3 - 1.5).astype(np.float32)
    grid[0, 0, 0] = [-1, 1]
    grid[0, 0, 1] = [0, 0]
    want = np.zeros((2, 3, 4, 6), np.float32)
    ref.ref_grid_sampler(fp(x), fp(grid), fp(want), 2, 3, 5, 7, 4, 6, mode, padding, int(align))
    assert np.array_equal(grid_sampler_ref(x, grid, mode, padding, align), want)


def test_activation_table_restatement(ref):
    ref.ref_active.argtypes = [C.c_int, C.c_int, C.c_double, C.c_double, C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_longlong]
    rng = np.random.default_rng(3)
    x = np.concatenate([(rng.standard_normal(3000) * 2).astype(np.float32), np.float32([0, -0.0, 1, -1, 25, -25, 0.5])])
    doms = {"x": x, "pos": np.abs(x) + np.float32(0.01), "unit": np.clip(x / 4, -0.99, 0.99).astype(np.float32)}
    for mode, (dom, fn, coeffs) in active_table().items():
        inp = np.ascontiguousarray(doms[dom])
        want = np.zeros_like(inp)
        co = list(coeffs or []) + [0.0, 0.0]
        ref.ref_active(ACTIVE_MODES[mode], len(coeffs or []), co[0], co[1], fp(inp), fp(want), inp.size)
        got = np.array([fn(float(v)) for v in inp], dtype=np.float64).astype(np.float32)
        assert np.array_equal(got, want), mode       # Python's math functions are the C library's: equal to the last bit
    # MISH works in float there (GenericCpuFunc.cpp:25-33)
    want = np.zeros_like(x)
    ref.ref_active(ACTIVE_MODES["MISH"], 0, 0.0, 0.0, fp(x), fp(want), x.size)
    f = np.float32
    got = x * (f(2) / (f(1) + np.exp(f(-2) * np.log(np.exp(x) + f(1)))) - f(1))
    np.testing.assert_allclose(got, want, rtol=2e-6, atol=1e-6)


def test_swap_dim_inner_is_a_roll(ref):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((2, 5, 6, 7)).astype(np.float32)
    for offs in ([0, 0, 2, 0], [0, 3, 0, 4], [0, 0, 0, 7], [1, 0, 5, 1]):
        want = np.zeros_like(x)
        ref.ref_swap_dim_inner(fp(x), fp(want), 4, (C.c_int64 * 4)(*x.shape), (C.c_int64 * 4)(*offs))
        got = x
        for ax, o in enumerate(offs):
            if o:
                got = np.roll(got, -o, axis=ax)
        assert np.array_equal(got, want), offs


def test_deconv_input_spreading(ref):
    """pad_tensor_for_deconv (MathUtils.cpp:673-705) against the slicing the tests' deconvolution restatement and the executor's
    plan use: the input lands at (k - 1) * d - pad with the stride between its elements, everything else holds the pad value."""
    rng = np.random.default_rng(5)
    ref.ref_pad_tensor_for_deconv.argtypes = [C.POINTER(C.c_float)] * 2 + [C.c_int] * 16 + [C.c_float]
    for (h, w, kh, kw, sh, sw, pads, opad) in ((5, 6, 3, 3, 2, 2, (1, 1, 1, 1), (1, 1)), (4, 3, 4, 2, 2, 3, (1, 0, 0, 1), (0, 0)),
                                               (3, 3, 3, 3, 1, 1, (0, 2, 2, 0), (0, 0))):
        x = rng.standard_normal((2, 3, h, w)).astype(np.float32)
        pt, pl, pb, pr = pads
        hs = (h - 1) * sh + 1 + 2 * (kh - 1) - pt - pb + opad[0]
        ws = (w - 1) * sw + 1 + 2 * (kw - 1) - pl - pr + opad[1]
        want = np.zeros((2, 3, hs, ws), np.float32)
        ref.ref_pad_tensor_for_deconv(fp(want), fp(x), 2, 3, h, w, kh, kw, 1, 1, sh, sw, pt, pb, pl, pr, opad[0], opad[1], 7.0)
        got = np.full((2, 3, hs, ws), 7.0, np.float32)
        got[:, :, kh - 1 - pt:kh - 1 - pt + (h - 1) * sh + 1:sh, kw - 1 - pl:kw - 1 - pl + (w - 1) * sw + 1:sw] = x
        assert np.array_equal(got, want)


def test_hc_transpose(ref):
    ref.ref_tensor_hc_transpose.argtypes = [C.POINTER(C.c_float)] * 2 + [C.c_longlong] * 4
    x = np.random.default_rng(6).standard_normal((2, 3, 4, 5)).astype(np.float32)
    want = np.zeros((2, 4, 3, 5), np.float32)
    ref.ref_tensor_hc_transpose(fp(want), fp(x), 2, 3, 4, 5)
    assert np.array_equal(np.ascontiguousarray(x.transpose(0, 2, 1, 3)), want)


@pytest.mark.parametrize("crd", [False, True])
@pytest.mark.parametrize("inv", [False, True])
@pytest.mark.parametrize("in_nchw,out_nchw", [(True, True), (False, True), (True, False), (False, False)])
@pytest.mark.parametrize("swap", [False, True])
def test_depth2space_restatement(ref, crd, inv, in_nchw, out_nchw, swap):
    rng = np.random.default_rng(7)
    bh, bw, c, h, w = 2, 3, 4, 3, 2
    deep, shallow = (2, c * bh * bw, h, w), (2, c, h * bh, w * bw)
    lay = lambda shp, f: shp if f else (shp[0], shp[2], shp[3], shp[1])  # noqa: E731
    in_shape, out_shape = (lay(shallow, in_nchw), lay(deep, out_nchw)) if inv else (lay(deep, in_nchw), lay(shallow, out_nchw))
    x = rng.standard_normal(in_shape).astype(np.float32)
    want = np.zeros(out_shape, np.float32)
    ref.ref_depth2space(fp(x), fp(want), (C.c_int64 * 4)(*in_shape), (C.c_int64 * 4)(*out_shape), bh, bw, int(crd), int(inv), int(in_nchw),
                        int(out_nchw), int(swap))
    assert np.array_equal(d2s_ref(x, out_shape, bh, bw, crd, inv, in_nchw, out_nchw, swap), want)


def test_gather_arg_gather_elements_restatements(ref):
    """The numpy expressions the GPU tests use for Gather (np.take with negative indices wrapped), Arg (first / last extreme)
    and GatherElements (np.take_along_axis on the indices' extent)."""
    rng = np.random.default_rng(8)
    x = rng.standard_normal((3, 6, 4)).astype(np.float32)
    idx = np.float32([[5, 0, -1], [2, 2, -6]])
    want = np.zeros((3, 2, 3, 4), np.float32)
    ref.ref_gather(fp(x), fp(idx), fp(want), 3, (C.c_int64 * 3)(*x.shape), 2, (C.c_int64 * 2)(*idx.shape), 1)
    assert np.array_equal(np.take(x, idx.astype(np.int64), axis=1), want)
    t = rng.integers(-3, 4, (3, 9, 5)).astype(np.float32)
    for is_max in (1, 0):
        for last in (1, 0):
            wi, wv = np.zeros((3, 5), np.float32), np.zeros((3, 5), np.float32)
            ref.ref_arg(fp(t), fp(wi), fp(wv), 3, (C.c_int64 * 3)(*t.shape), 1, is_max, last)
            ext = t.max(axis=1) if is_max else t.min(axis=1)
            hit = t == ext[:, None, :]
            gi = (t.shape[1] - 1 - hit[:, ::-1, :].argmax(axis=1)) if last else hit.argmax(axis=1)
            assert np.array_equal(gi.astype(np.float32), wi) and np.array_equal(ext, wv), (is_max, last)
    src = rng.standard_normal((4, 5, 6)).astype(np.float32)
    ind = rng.integers(0, 5, (3, 2, 6)).astype(np.float32)
    wg = np.zeros(ind.shape, np.float32)
    ref.ref_gather_elements(fp(wg), fp(src), fp(ind), (C.c_int * 3)(*ind.shape), (C.c_int * 3)(*src.shape), 3, 1)
    got = np.zeros(ind.shape, np.float32)
    for a_ in range(3):
        for b_ in range(2):
            for c_ in range(6):
                got[a_, b_, c_] = src[a_, int(ind[a_, b_, c_]), c_]
    assert np.array_equal(got, wg)


# ------------------------------------------------------------------ loops compiled into oracle/_ref/oploops_ref.so
OPLOOPS = os.path.join(os.path.dirname(REF), "oploops_ref.so")


@pytest.fixture(scope="module")
def loops():
    if not os.path.exists(OPLOOPS):
        pytest.skip("oracle/_ref/oploops_ref.so was not built")
    lib = C.CDLL(OPLOOPS)
    if not hasattr(lib, "ref_requant_fp"):
        pytest.skip("an older oploops_ref.so")
    lib.ref_requant_fp.argtypes = [C.POINTER(C.c_float)] * 2 + [C.c_longlong, C.c_double, C.c_double, C.c_int, C.c_int, C.c_int, C.c_int, C.c_longlong]
    lib.ref_maxmin_const.argtypes = [C.c_int] + [C.POINTER(C.c_float)] * 2 + [C.c_longlong, C.c_double, C.c_float, C.c_longlong, C.c_longlong, C.c_int,
                                                                              C.c_int, C.c_int]
    lib.ref_prelu_int8.argtypes = [C.POINTER(C.c_float)] * 3 + [C.c_longlong] * 4 + [C.c_int, C.c_int]
    return lib


def _rsr(v, s):
    return (v + (1 << (s - 1))) >> s if s > 0 else v


def test_requant_fp_expressions(loops):
    """tpu.RequantFp::inference (RequantFp.cpp:19-67) against the expressions of tests/test_gpu_more_ops.py."""
    rng = np.random.default_rng(9)
    acc = rng.integers(-60000, 60000, 4000).astype(np.float32)
    acc[:4] = [250, -250, 750, -750]
    sc, of = 0.002, 0.5
    want = np.zeros_like(acc)
    loops.ref_requant_fp(fp(acc), fp(want), acc.size, sc, of, 2, 0, 8, 0, 0)          # MultiplierShift, half away from zero, int8
    f = acc * np.float32(sc) + np.float32(of)
    assert np.array_equal(np.clip(np.sign(f) * np.floor(np.abs(f) + np.float32(0.5)), -128, 127), want)
    loops.ref_requant_fp(fp(acc), fp(want), acc.size, sc, 0.0, 1, 3, 8, 1, 7)           # TFLite, half to even, uint8, zero point 7
    assert np.array_equal(np.clip(np.rint(acc * np.float32(sc)).astype(np.int64) + 7, 0, 255).astype(np.float32), want)


def test_max_min_const_expressions(loops):
    rng = np.random.default_rng(10)
    q = rng.integers(-128, 128, 3000).astype(np.float32)
    want = np.zeros_like(q)
    loops.ref_maxmin_const(1, fp(q), fp(want), q.size, 3.0, np.float32(-150.7), 9, 3, 0, 8, 0)
    pf = np.maximum(((q.astype(np.int64) - 3) * 9).astype(np.float32), np.float32(-150.7))
    assert np.array_equal(np.clip(_rsr(np.trunc(pf).astype(np.int64), 3), -128, 127).astype(np.float32), want)
    loops.ref_maxmin_const(0, fp(q), fp(want), q.size, 0.0, np.float32(200.25), 7, 2, 1, 8, 0)
    pf = np.minimum((q.astype(np.int64) * 7).astype(np.float32), np.float32(200.25))
    assert np.array_equal(np.clip(np.maximum(_rsr(np.trunc(pf).astype(np.int64), 2), 0), -128, 127).astype(np.float32), want)


def test_prelu_int8_expression(loops):
    rng = np.random.default_rng(11)
    q = rng.integers(-128, 128, (2, 3, 4, 5)).astype(np.float32)
    slope = np.float32([13, -7, 100])
    want = np.zeros_like(q)
    loops.ref_prelu_int8(fp(q), fp(slope), fp(want), 6, 20, 3, 5, 8, 0)
    prod = q.astype(np.int64) * slope.astype(np.int64).reshape(1, 3, 1, 1)
    neg = np.clip((prod + 16) >> 5, -128, 127)
    assert np.array_equal(np.where(q < 0, neg, q).astype(np.float32), want)


def test_subconst_and_top_cast_expressions(loops):
    """tpu.SubConst::inference (SubConst.cpp:19-111, symmetric 8-bit) and top.Cast::inference (Cast.cpp:18-64) against the
    expressions of tests/test_gpu_more_ops.py."""
    if not hasattr(loops, "ref_subconst"):
        pytest.skip("an older oploops_ref.so")
    loops.ref_subconst.argtypes = [C.POINTER(C.c_float)] * 2 + [C.c_longlong, C.c_double, C.c_int, C.c_longlong, C.c_longlong, C.c_int, C.c_double,
                                                                C.c_int, C.c_int]
    loops.ref_top_cast.argtypes = [C.POINTER(C.c_float)] * 2 + [C.c_longlong, C.c_char_p, C.c_int]
    rng = np.random.default_rng(12)
    q = rng.integers(-128, 128, 3000).astype(np.float32)
    want = np.zeros_like(q)
    for rev in (0, 1):
        loops.ref_subconst(fp(q), fp(want), q.size, 33.5, rev, 11, 4, 0, -1.0, 8, 0)
        prod = (q.astype(np.int64) * 11).astype(np.float64)
        f = (33.5 - prod if rev else prod - 33.5).astype(np.float32)
        assert np.array_equal(np.clip(_rsr(np.trunc(f).astype(np.int64), 4), -128, 127).astype(np.float32), want), rev
    # with the ReLU and its limit acting on the float before the shift
    loops.ref_subconst(fp(q), fp(want), q.size, 10.25, 0, 5, 2, 1, 300.0, 8, 0)
    f = np.minimum(np.maximum(((q.astype(np.int64) * 5).astype(np.float64) - 10.25).astype(np.float32), 0), np.float32(300.0))
    assert np.array_equal(np.clip(np.maximum(_rsr(np.trunc(f).astype(np.int64), 2), 0), -128, 127).astype(np.float32), want)
    v = np.float32([-300.5, -128.5, -2.5, -1.5, -0.5, 0.5, 1.5, 2.5, 126.5, 127.5, 255.5, 300.2, 40000.7, -40000.7])
    away = np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))
    out = np.zeros_like(v)
    # RoundingMode numbering of MathUtils.h:28-42: 0 half away, 3 half to even, 6 towards zero, 8 up, 9 down
    for to, rm, expect in ((b"INT8", 0, np.clip(away, -128, 127)), (b"UINT8", 3, np.clip(np.rint(v), 0, 255)), (b"INT16", 9, np.clip(np.floor(v), -32768, 32767)),
                           (b"UINT16", 8, np.clip(np.ceil(v), 0, 65535)), (b"INT32", 6, np.trunc(v)), (b"F32", 0, v)):
        loops.ref_top_cast(fp(v), fp(out), v.size, to, rm)
        assert np.array_equal(out, expect.astype(np.float32)), to


@pytest.mark.parametrize("mode", ["reflect", "edge"])
def test_pad_modes_are_numpy_pads(ref, mode):
    """top.Pad's reflect / edge loops (Pad.cpp:121-213) against numpy.pad, which the GPU test holds the executor to."""
    if not hasattr(ref, "ref_pad_mode"):
        pytest.skip("an older moreops_ref.so")
    rng = np.random.default_rng(13)
    for (h, w, pt, pl, pb, pr) in ((5, 6, 2, 1, 3, 4), (4, 4, 1, 3, 1, 0), (3, 7, 0, 0, 2, 2)):
        x = rng.standard_normal((2, 3, h, w)).astype(np.float32)
        want = np.zeros((2, 3, h + pt + pb, w + pl + pr), np.float32)
        ref.ref_pad_mode(fp(x), fp(want), 2, 3, h, w, pt, pl, pb, pr, mode.encode())
        assert np.array_equal(np.pad(x, ((0, 0), (0, 0), (pt, pb), (pl, pr)), mode=mode), want)


def test_sub_int8_and_reduce_tail_expressions(loops):
    """tpu.Sub's symmetric int8 branch (Sub.cpp:160-185) and the requantisation tail of tpu.Reduce (Reduce.cpp:206-213)."""
    if not hasattr(loops, "ref_sub_int8"):
        pytest.skip("an older oploops_ref.so")
    loops.ref_sub_int8.argtypes = [C.POINTER(C.c_float)] * 3 + [C.c_longlong] * 5 + [C.c_int] * 3
    loops.ref_reduce_tail.argtypes = [C.POINTER(C.c_float)] + [C.c_longlong] * 3
    rng = np.random.default_rng(14)
    a_ = rng.integers(-128, 128, 4000).astype(np.float32)
    b_ = rng.integers(-128, 128, 4000).astype(np.float32)
    want = np.zeros_like(a_)
    loops.ref_sub_int8(fp(a_), fp(b_), fp(want), a_.size, 90, 7, 70, 6, 0, 8, 0)
    diff = ((a_.astype(np.int64) * 90 + 64) >> 7) - ((b_.astype(np.int64) * 70 + 32) >> 6)
    assert np.array_equal(np.clip(diff, -128, 127).astype(np.float32), want)
    loops.ref_sub_int8(fp(a_), fp(b_), fp(want), a_.size, 90, 7, 70, 6, 1, 8, 0)
    assert np.array_equal(np.clip(np.maximum(diff, 0), -128, 127).astype(np.float32), want)
    # the mean of int8 values as the float loop leaves it (sum * float(1 / n)), then cut, multiplied, shifted, saturated to int8
    q = rng.integers(-128, 128, (300, 7)).astype(np.float32)
    ssum = np.zeros(300, np.float32)
    for k in range(7):
        ssum = ssum + q[:, k]
    vals = (ssum * np.float32(1.0 / 7)).astype(np.float32)
    got = np.clip((np.trunc(vals).astype(np.int64) * 77 + 32) >> 6, -128, 127).astype(np.float32)
    loops.ref_reduce_tail(fp(vals), vals.size, 77, 6)
    assert np.array_equal(got, vals)
