"""Glue ops of an INT8 graph (Add, Pool2D, Cast, RequantInt/RequantIntAxis) on the GPU, bit-exact vs the oracle."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import tpu_mlir_b200._lib as L

from gpu_util import dev, dt_of, empty_dev, ptr

pytestmark = pytest.mark.gpu
lib = L.lib


@pytest.mark.parametrize("n", [1, 7, 4096, 100003])
def test_add(n):
    rng = np.random.default_rng(n)
    a = rng.integers(0, 256, n, dtype=np.uint8)
    b = rng.integers(-128, 128, n, dtype=np.int8)
    for (m0, s0, m1, s1, relu, odt) in [(77, 6, 100, 7, True, L.DT_U8), (3, 0, 125, 9, False, L.DT_I8)]:
        want = oracle.add_int8(a, b, m0, s0, m1, s1, do_relu=relu, out_dt=odt)
        out = empty_dev((n,), odt)
        a_d, b_d = dev(a), dev(b)          # keep the device tensors alive across the asynchronous call
        L.check(lib().b200q_add_i8_dev(ptr(a_d), L.DT_U8, ptr(b_d), L.DT_I8, n, m0, s0, m1, s1, int(relu), odt, ptr(out), None))
        assert np.array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("a_unsigned,b_unsigned", [(True, True), (True, False), (False, True), (False, False)])
def test_add_wide_kernel_all_sign_combinations(a_unsigned, b_unsigned):
    """n % 16 == 0 with 8-bit multipliers takes the 16-elements-per-thread kernel (32-bit arithmetic)."""
    n = 16 * 4099
    rng = np.random.default_rng(11)
    a = rng.integers(0, 256, n, dtype=np.uint8) if a_unsigned else rng.integers(-128, 128, n, dtype=np.int8)
    b = rng.integers(0, 256, n, dtype=np.uint8) if b_unsigned else rng.integers(-128, 128, n, dtype=np.int8)
    a_d, b_d = dev(a), dev(b)
    for (m0, s0, m1, s1, relu, odt) in [(127, 1, -128, 31, True, L.DT_I8), (64, 6, 127, 7, False, L.DT_I8),
                                        (99, 5, 17, 3, True, L.DT_U8), (1, 1, 1, 1, False, L.DT_U8)]:
        want = oracle.add_int8(a, b, m0, s0, m1, s1, do_relu=relu, out_dt=odt)
        out = empty_dev((n,), odt)
        L.check(lib().b200q_add_i8_dev(ptr(a_d), dt_of(a), ptr(b_d), dt_of(b), n, m0, s0, m1, s1, int(relu), odt, ptr(out), None))
        assert np.array_equal(out.cpu().numpy(), want), (m0, s0, m1, s1, relu, odt)


def test_pool():
    rng = np.random.default_rng(4)
    x = rng.integers(0, 256, (3, 5, 17, 14), dtype=np.uint8)
    xs = rng.integers(-128, 128, (2, 4, 7, 7), dtype=np.int8)
    want = oracle.pool2d_int8(x, (3, 3), (2, 2), (1, 1, 1, 1), mode="max")
    out = empty_dev(want.shape, L.DT_U8)
    x_d, xs_d = dev(x), dev(xs)
    L.check(lib().b200q_pool2d_i8_dev(ptr(x_d), L.DT_U8, 15, 17, 14, 3, 3, 2, 2, 1, 1, 1, 1, 0, 1, 0, 0, L.DT_U8, ptr(out), None))
    assert np.array_equal(out.cpu().numpy(), want)
    want = oracle.pool2d_int8(xs, (7, 7), (1, 1), (0, 0, 0, 0), mode="avg", multi=83, rshift=12, do_relu=True)
    out = empty_dev(want.shape, L.DT_I8)
    L.check(lib().b200q_pool2d_i8_dev(ptr(xs_d), L.DT_I8, 8, 7, 7, 7, 7, 1, 1, 0, 0, 0, 0, 1, 83, 12, 1, L.DT_I8, ptr(out), None))
    assert np.array_equal(out.cpu().numpy(), want)


def test_pool_channels_last():
    """b200q_pool2d_i8_nhwc_dev: the NCHW op's values on [N][H][W][C] tensors."""
    rng = np.random.default_rng(14)
    for dt, lo, hi, relu in ((np.uint8, 0, 256, False), (np.int8, -128, 128, False), (np.int8, -128, 128, True)):
        x = rng.integers(lo, hi, (3, 32, 17, 14), dtype=dt)
        odt = L.DT_U8 if dt == np.uint8 else L.DT_I8
        for kernel, stride, pads in (((3, 3), (2, 2), (1, 1, 1, 1)), ((2, 3), (1, 2), (0, 1, 1, 0))):
            want = oracle.pool2d_int8(x, kernel, stride, pads, mode="max", do_relu=relu)
            x_d = dev(np.ascontiguousarray(x.transpose(0, 2, 3, 1)))
            out = empty_dev((want.shape[0], want.shape[2], want.shape[3], want.shape[1]), odt)
            # oracle pads are (top, bottom, left, right), the order of the C arguments
            L.check(lib().b200q_pool2d_i8_nhwc_dev(ptr(x_d), odt, 3, 32, 17, 14, kernel[0], kernel[1], stride[0], stride[1],
                                                   pads[0], pads[1], pads[2], pads[3], 0, 1, 0, int(relu), odt, ptr(out), None))
            assert np.array_equal(out.cpu().numpy().transpose(0, 3, 1, 2), want), (dt, kernel)
    xs = rng.integers(-128, 128, (2, 24, 7, 7), dtype=np.int8)
    want = oracle.pool2d_int8(xs, (7, 7), (1, 1), (0, 0, 0, 0), mode="avg", multi=83, rshift=12, do_relu=True)
    xs_d = dev(np.ascontiguousarray(xs.transpose(0, 2, 3, 1)))
    out = empty_dev((2, 1, 1, 24), L.DT_I8)
    L.check(lib().b200q_pool2d_i8_nhwc_dev(ptr(xs_d), L.DT_I8, 2, 24, 7, 7, 7, 7, 1, 1, 0, 0, 0, 0, 1, 83, 12, 1, L.DT_I8,
                                           ptr(out), None))
    assert np.array_equal(out.cpu().numpy().transpose(0, 3, 1, 2), want)
    # max pooling of a channel count that is not a multiple of 16 is refused, not silently mis-indexed
    assert lib().b200q_pool2d_i8_nhwc_dev(ptr(xs_d), L.DT_I8, 2, 24, 7, 7, 3, 3, 1, 1, 0, 0, 0, 0, 0, 1, 0, 0, L.DT_I8,
                                          ptr(out), None) == L.ERR_UNSUPPORTED


@pytest.mark.parametrize("n", [1, 15, 16, 4099, 1 << 20])
def test_lut(n):
    rng = np.random.default_rng(n)
    for xdt in (np.int8, np.uint8):
        x = rng.integers(np.iinfo(xdt).min, np.iinfo(xdt).max + 1, n, dtype=xdt)
        for tdt, code in ((np.int8, L.DT_I8), (np.uint8, L.DT_U8), (np.float32, L.DT_F32)):
            table = (rng.integers(-128, 128, 256).astype(tdt) if tdt != np.float32
                     else rng.standard_normal(256).astype(np.float32))
            want = oracle.lut(x, table)
            x_d, t_d = dev(x), dev(table)
            out = torch.empty(n, dtype=getattr(torch, np.dtype(tdt).name), device="cuda")
            L.check(lib().b200q_lut_dev(ptr(x_d), n, ptr(t_d), code, ptr(out), None))
            assert np.array_equal(out.cpu().numpy(), want), (xdt, tdt)


def test_lut_unaligned_views():
    rng = np.random.default_rng(3)
    x = rng.integers(-128, 128, 1000, dtype=np.int8)
    table = rng.integers(0, 256, 256).astype(np.uint8)
    x_d, t_d = dev(x), dev(table)
    out = torch.zeros(1000, dtype=torch.uint8, device="cuda")
    L.check(lib().b200q_lut_dev(C.c_void_p(x_d.data_ptr() + 3), 900, ptr(t_d), L.DT_U8, C.c_void_p(out.data_ptr() + 5), None))
    assert np.array_equal(out.cpu().numpy()[5:905], oracle.lut(x[3:903], table))


def test_mulshift_and_mul():
    rng = np.random.default_rng(12)
    n = 70001
    a = rng.integers(-128, 128, n, dtype=np.int8)
    b = rng.integers(0, 256, n, dtype=np.uint8)
    a_d, b_d = dev(a), dev(b)
    for x, x_d, m, s, izp, ozp, odt in ((a, a_d, 77, 5, 0, 0, L.DT_I8), (b, b_d, 19000, 14, 128, -3, L.DT_I8),
                                        (a, a_d, -3, 0, 0, 7, L.DT_U8), (b, b_d, 2**30, 31, 5, 0, L.DT_U8)):
        want = oracle.mulshift_int8(x, m, s, in_zp=izp, out_zp=ozp, out_dt=odt)
        out = empty_dev((n,), odt)
        L.check(lib().b200q_mulshift_i8_dev(ptr(x_d), dt_of(x), n, m, s, izp, ozp, odt, ptr(out), None))
        assert np.array_equal(out.cpu().numpy(), want), (m, s, izp, ozp, odt)
    for m, s, relu, odt in ((3, 4, True, L.DT_U8), (1200, 17, False, L.DT_I8), (1, 0, False, L.DT_I8), (2**20, 30, True, L.DT_I8)):
        want = oracle.mul_int8(a, b, m, s, do_relu=relu, out_dt=odt)
        out = empty_dev((n,), odt)
        L.check(lib().b200q_mul_i8_dev(ptr(a_d), dt_of(a), ptr(b_d), dt_of(b), n, m, s, int(relu), odt, ptr(out), None))
        assert np.array_equal(out.cpu().numpy(), want), (m, s, relu, odt)


def test_cast_both_ways():
    rng = np.random.default_rng(6)
    x = (rng.standard_normal(50001) * 3).astype(np.float32)
    x[:6] = [0.5 * 0.0371, -0.5 * 0.0371, 1.5 * 0.0371, 1e9, -1e9, 0.0]
    for scale, zp, odt in [(0.0371, 0, L.DT_I8), (4.1 / 255, 3, L.DT_U8)]:
        want = oracle.cast_f32_to_q8(x, scale, zp, out_dt=odt)
        out = empty_dev(x.shape, odt)
        x_d = dev(x)
        L.check(lib().b200q_cast_f32_to_q8_dev(ptr(x_d), x.size, scale, zp, L.ROUND_HALF_AWAY_FROM_ZERO, odt, ptr(out), None))
        assert np.array_equal(out.cpu().numpy(), want)
        back = torch.empty(x.shape, dtype=torch.float32, device="cuda")
        L.check(lib().b200q_cast_q8_to_f32_dev(ptr(out), odt, x.size, scale, zp, ptr(back), None))
        assert np.array_equal(back.cpu().numpy(), oracle.cast_q8_to_f32(want, scale, zp))


@pytest.mark.parametrize("mode", ["tflite", "ms", "ms_fuse_axis"])
def test_requant_int_axis_operator_face(mode):
    rng = np.random.default_rng(9)
    Cn = 24
    x = rng.integers(-2**20, 2**20, (3, Cn, 5, 4) if mode != "ms_fuse_axis" else (3, 5, 4, Cn), dtype=np.int32)
    if mode == "tflite":
        quant = np.stack([rng.integers(2**30, 2**31, Cn), -rng.integers(4, 16, Cn), rng.integers(-5, 5, Cn)], axis=1)
        qmode, rmode = oracle.QM_TFLITE, oracle.RM_HALF_AWAY
    else:
        quant = np.stack([rng.integers(1000, 30000, Cn), (-1 if mode == "ms" else 1) * rng.integers(12, 24, Cn), rng.integers(-5, 5, Cn)], axis=1)
        qmode, rmode = oracle.QM_MULTIPLIER_SHIFT, oracle.RM_HALF_UP
    quant_f = quant.astype(np.float32)                    # the operand as the interpreter stores it
    seen = quant_f.astype(np.int64)
    fuse = mode == "ms_fuse_axis"
    want = oracle.requant_int_axis(x, seen, qmode=qmode, rmode=rmode, fuse_rq_axis=fuse, out_dt=oracle.DT_I8)
    d = L.RequantDesc(outer=x.size // Cn if fuse else x.shape[0], channels=Cn, inner=1 if fuse else 20, per_axis=1,
                      quant_mode=qmode, round_mode=rmode, fuse_rq_axis=int(fuse), in_zp=0, out_dtype=L.DT_I8)
    out = np.zeros(x.shape, np.float32)
    L.check(lib().b200q_requant_int_axis_inference(C.byref(d), L.float_pp([x.astype(np.float32), quant_f.reshape(-1)]), 2,
                                                   L.float_pp([out]), 1))
    assert np.array_equal(out, want.astype(np.float32))


@pytest.mark.parametrize("mode", ["tflite", "ms", "ms_fuse_axis"])
def test_requant_int_axis_two_word_quant_operand(mode):
    """Chips other than BM1684X pack the quant operand in two words per channel: the multiplier, then the shift in the
    low byte (signed char) and the zero point in the high half-word (signed short), RequantIntAxis.cpp:49-54."""
    rng = np.random.default_rng(21)
    Cn = 7
    x = rng.integers(-2**20, 2**20, (3, Cn, 5, 4) if mode != "ms_fuse_axis" else (3, 5, 4, Cn), dtype=np.int32)
    zp = rng.integers(0, 90, Cn)       # non-negative: the packed word stays below 2^24 and survives its float buffer
    if mode == "tflite":
        mult, shift = oracle.through_f32(rng.integers(2**30, 2**31, Cn)), -rng.integers(4, 16, Cn)
        qmode, rmode = oracle.QM_TFLITE, oracle.RM_HALF_AWAY
    else:
        mult, shift = rng.integers(1000, 30000, Cn), (-1 if mode == "ms" else 1) * rng.integers(12, 24, Cn)
        qmode, rmode = oracle.QM_MULTIPLIER_SHIFT, oracle.RM_HALF_UP
    packed = (shift.astype(np.int64) & 0xFF) | (zp.astype(np.int64) << 16)
    quant2 = np.stack([mult, packed], axis=1).astype(np.float32)
    assert np.array_equal(quant2[:, 1].astype(np.int64), packed)
    fuse = mode == "ms_fuse_axis"
    want = oracle.requant_int_axis(x, np.stack([mult, shift, zp], axis=1), qmode=qmode, rmode=rmode, fuse_rq_axis=fuse,
                                   out_dt=oracle.DT_I8)
    d = L.RequantDesc(outer=x.size // Cn if fuse else x.shape[0], channels=Cn, inner=1 if fuse else 20, per_axis=1,
                      quant_mode=qmode, round_mode=rmode, fuse_rq_axis=int(fuse), in_zp=0, out_dtype=L.DT_I8, quant_words=2)
    out = np.zeros(x.shape, np.float32)
    L.check(lib().b200q_requant_int_axis_inference(C.byref(d), L.float_pp([x.astype(np.float32), quant2.reshape(-1)]), 2,
                                                   L.float_pp([out]), 1))
    assert np.array_equal(out, want.astype(np.float32))


def test_requant_int_operator_face():
    rng = np.random.default_rng(10)
    x = rng.integers(-2**18, 2**18, (2, 6, 9), dtype=np.int32)
    for qmode, rmode, multi, rshift in [(oracle.QM_TFLITE, oracle.RM_HALF_AWAY, 1518500250, 9),
                                        (oracle.QM_MULTIPLIER_SHIFT, oracle.RM_HALF_UP, 12345, 20)]:
        want = oracle.requant_int(x, multi, rshift, qmode=qmode, rmode=rmode, out_zp=-3, out_dt=oracle.DT_I8)
        d = L.RequantDesc(outer=2, channels=6, inner=9, per_axis=0, quant_mode=qmode, round_mode=rmode, fuse_rq_axis=0, in_zp=0,
                          out_dtype=L.DT_I8, multiplier=multi, rshift=rshift, out_zp=-3)
        out = np.zeros(x.shape, np.float32)
        L.check(lib().b200q_requant_int_axis_inference(C.byref(d), L.float_pp([x.astype(np.float32)]), 1, L.float_pp([out]), 1))
        assert np.array_equal(out, want.astype(np.float32))


def test_executor_loads_mlir_text(tmp_path):
    """The same small graph through module.load(dict) and module.load(<file>.mlir) gives identical tensors."""
    from test_mlir_text import small_graph
    from tpu_mlir_b200 import mlir_text as MT
    from tpu_mlir_b200.module import module
    graph, weights = small_graph()
    (tmp_path / "m.mlir").write_text(MT.emit_module(graph, weights, weight_file="w.npz"))
    np.savez(tmp_path / "w.npz", **weights)
    x = np.random.default_rng(3).standard_normal((2, 3, 8, 8)).astype(np.float32)
    outs = []
    for src in ((graph, weights), (str(tmp_path / "m.mlir"), None)):
        m = module()
        m.load(*src)
        m.set_tensor("input", x)
        m.invoke(fixed_to_float=False)
        outs.append({n: m.get_tensor(n) for n in ("conv", "pool", "sum", "fc", "output")})
    for n in outs[0]:
        assert np.array_equal(outs[0][n], outs[1][n]), n
    assert outs[0]["fc"].any()


@pytest.mark.parametrize("channels_last", [False, True])
def test_executor_runs_lut_mulshift_mul(channels_last):
    """A small graph of the element-wise ops through the executor, every tensor against the oracle functions."""
    from tpu_mlir_b200.module import module
    rng = np.random.default_rng(8)
    oc = 32
    w = rng.integers(-20, 20, (oc, 16, 1, 1), dtype=np.int8)
    mult, rs = rng.integers(900, 1500, oc), rng.integers(9, 12, oc)
    table = rng.integers(-128, 128, 256).astype(np.int8)
    shp = [2, oc, 6, 5]
    tens = {"input": dict(shape=[2, 16, 6, 5], dtype="f32"),
            "q": dict(shape=[2, 16, 6, 5], dtype="i8", scale=0.05, zp=0),
            "conv": dict(shape=shp, dtype="i8", scale=0.1, zp=0),
            "lut": dict(shape=shp, dtype="i8", scale=0.1, zp=0),
            "ms": dict(shape=shp, dtype="i8", scale=0.1, zp=0),
            "mul": dict(shape=shp, dtype="u8", scale=0.1, zp=0)}
    ops = [dict(type="tpu.Cast", name="q", inputs=["input"]),
           dict(type="tpu.Conv2D", name="conv", inputs=["q"],
                attrs=dict(kernel_shape=[1, 1], group=1, quant_mode="MultiplierShift", multiplier=mult.tolist(),
                           rshift=rs.tolist(), do_relu=False)),
           dict(type="tpu.Lut", name="lut", inputs=["conv"]),
           dict(type="tpu.MulShift", name="ms", inputs=["conv"], attrs=dict(multiplier=90, rshift=6)),
           dict(type="tpu.Mul", name="mul", inputs=["lut", "ms"], attrs=dict(multiplier=5, rshift=7, do_relu=True))]
    graph = dict(inputs=["input"], outputs=["mul"], tensors=tens, ops=ops)
    weights = {"conv_filter": w, "lut_table": table}
    x = rng.standard_normal((2, 16, 6, 5)).astype(np.float32)
    m = module(channels_last=channels_last)
    m.load(graph, weights)
    m.set_tensor("input", x)
    m.invoke(fixed_to_float=False)
    conv = m.get_tensor("conv")
    assert conv.shape == tuple(shp) and len(np.unique(conv)) > 20
    assert (("conv" in m._nhwc) and ("mul" in m._nhwc)) == channels_last
    lut = oracle.lut(conv, table)
    ms = oracle.mulshift_int8(conv, 90, 6)
    assert np.array_equal(m.get_tensor("lut"), lut)
    assert np.array_equal(m.get_tensor("ms"), ms)
    assert np.array_equal(m.get_tensor("mul"), oracle.mul_int8(lut, ms, 5, 7, do_relu=True, out_dt=oracle.DT_U8))


def _matmul_graph(attrs, weights_extra=None, w_shape=(64, 24), zp=0):
    rng = np.random.default_rng(12)
    tens = {"input": dict(shape=[5, 64], dtype="f32"), "q": dict(shape=[5, 64], dtype="i8", scale=0.05, zp=0),
            "fc": dict(shape=[5, 24], dtype="i8", scale=0.2, zp=zp), "out": dict(shape=[5, 24], dtype="f32")}
    ops = [dict(type="tpu.Cast", name="q", inputs=["input"]),
           dict(type="tpu.MatMul", name="fc", inputs=["q"], attrs=dict(do_relu=False, **attrs)),
           dict(type="tpu.Cast", name="out", inputs=["fc"])]
    weights = {"fc_filter": rng.integers(-127, 128, w_shape, dtype=np.int8), "fc_bias": rng.integers(-500, 500, 24, dtype=np.int32)}
    weights.update(weights_extra or {})
    return dict(inputs=["input"], outputs=["out"], tensors=tens, ops=ops), weights


@pytest.mark.parametrize("case", ["tflite", "tflite_lshift", "right_transpose", "fuse_rq", "zero_points"])
def test_executor_matmul_honours_its_attributes(case, tmp_path):
    """tpu.MatMul through the executor with the attributes a lowered model can carry (MatMul.cpp:636-728): TFLite
    requantisation, a right operand stored [N, K], per-channel multipliers with a common shift; the graph goes through
    the .mlir text on the way, and every tensor is compared with the oracle walk."""
    import oracle_graph
    from tpu_mlir_b200 import mlir_text as MT
    from tpu_mlir_b200.module import module
    rng = np.random.default_rng(13)
    if case in ("tflite", "tflite_lshift"):
        g, w = _matmul_graph(dict(quant_mode="TFLite" if case == "tflite" else "TFLite_LShift", multipliers=[1518500250], rshifts=[9]), zp=3)
    elif case == "zero_points":
        g, w = _matmul_graph(dict(quant_mode="MultiplierShift", input_zp=4, right_zp=-3, multipliers=[777], rshifts=[14]))
    elif case == "right_transpose":
        g, w = _matmul_graph(dict(quant_mode="MultiplierShift", right_transpose=True, multipliers=[777], rshifts=[14]), w_shape=(24, 64))
    else:
        multi = rng.integers(300, 900, 24).astype(np.float32)
        g, w = _matmul_graph(dict(quant_mode="MultiplierShift", fuse_rq=True, multipliers=[1] * 24, rshifts=[14] * 24), {"fc_multi": multi})
    (tmp_path / "m.mlir").write_text(MT.emit_module(g, w, weight_file="w.npz"))
    np.savez(tmp_path / "w.npz", **w)
    x = rng.standard_normal((5, 64)).astype(np.float32)
    want = oracle_graph.run(g, w, {"input": x})
    for src in ((g, w), (str(tmp_path / "m.mlir"), None)):
        m = module()
        m.load(*src)
        m.set_tensor("input", x)
        m.invoke(fixed_to_float=False)
        assert np.array_equal(m.get_tensor("fc"), want["fc"]) and want["fc"].any()


@pytest.mark.parametrize("lt,ot", [(True, False), (False, True), (True, True)])
def test_executor_matmul_transposed_operands(lt, ot):
    """left_transpose: the input tensor is stored [K, M]; output_transpose: the output tensor is stored [N, M]
    (MatMul.cpp:24-135, lib/Support/Dnnl/MatMul.cpp:182-186,:229-238)."""
    import oracle_graph
    from tpu_mlir_b200.module import module
    rng = np.random.default_rng(21)
    M, K, N = 37, 64, 24
    in_shape, out_shape = ([K, M] if lt else [M, K]), ([N, M] if ot else [M, N])
    tens = {"input": dict(shape=in_shape, dtype="f32"), "q": dict(shape=in_shape, dtype="i8", scale=0.05, zp=0),
            "fc": dict(shape=out_shape, dtype="i8", scale=0.2, zp=0), "out": dict(shape=out_shape, dtype="f32")}
    ops = [dict(type="tpu.Cast", name="q", inputs=["input"]),
           dict(type="tpu.MatMul", name="fc", inputs=["q"], attrs=dict(do_relu=False, quant_mode="MultiplierShift", multipliers=[777],
                                                                       rshifts=[14], left_transpose=lt, output_transpose=ot)),
           dict(type="tpu.Cast", name="out", inputs=["fc"])]
    g = dict(inputs=["input"], outputs=["out"], tensors=tens, ops=ops)
    w = {"fc_filter": rng.integers(-127, 128, (K, N), dtype=np.int8), "fc_bias": rng.integers(-500, 500, N, dtype=np.int32)}
    x = rng.standard_normal(in_shape).astype(np.float32)
    want = oracle_graph.run(g, w, {"input": x})
    m = module()
    m.load(g, w)
    m.set_tensor("input", x)
    m.invoke(fixed_to_float=False)
    assert list(want["fc"].shape) == out_shape and len(np.unique(want["fc"])) > 30
    assert np.array_equal(m.get_tensor("fc"), want["fc"])
    assert np.array_equal(m.get_tensor("out"), want["out"])


def test_executor_refuses_matmul_attributes_it_does_not_honour():
    from tpu_mlir_b200.module import module
    for bad in (dict(hdim_is_batch=True), dict(quant_mode="OnlyScale")):
        attrs = dict(quant_mode="MultiplierShift", multipliers=[77], rshifts=[12])
        attrs.update(bad)
        g, w = _matmul_graph(attrs)
        with pytest.raises(L.B200QError) as ei:
            module().load(g, w)
        assert ei.value.code == L.ERR_UNSUPPORTED


def test_executor_invoke_surface():
    """invoke(fixed_to_float), invoke_at, invoke_from and fake_quant_weight of pymlir.module
    (pymlir.cpp:108-112, ModuleInterpreter.cpp:583-612,:992-1011,:1210-1253)."""
    import oracle_graph
    from test_mlir_text import small_graph
    from tpu_mlir_b200.module import module
    graph, weights = small_graph()
    x = np.random.default_rng(3).standard_normal((2, 3, 8, 8)).astype(np.float32)
    want = oracle_graph.run(graph, weights, {"input": x})
    m = module()
    m.load(graph, weights)
    m.set_tensor("input", x)
    # fixed_to_float (the default): get_tensor returns the expressed values (q - zp) * scale
    m.invoke()
    sc = np.float32(graph["tensors"]["conv"]["scale"])
    assert np.array_equal(m.get_tensor("conv"), want["conv"].astype(np.float32) * sc)
    assert np.array_equal(m.get_raw_tensor("conv"), want["conv"])
    m.invoke(fixed_to_float=False)
    assert np.array_equal(m.get_tensor("conv"), want["conv"])
    # invoke_at: one op with its hooks, result as stored
    seen = []
    m.before_invoke(lambda n: seen.append(("b", n)))
    m.after_invoke(lambda n: seen.append(("a", n)))
    assert np.array_equal(m.invoke_at("pool"), want["pool"]) and seen == [("b", "pool"), ("a", "pool")]
    # invoke_from: overwrite an intermediate tensor, run the rest
    seen.clear()
    m.tensors["pool"].zero_()
    m.invoke_from("sum")
    assert [n for k, n in seen if k == "a"] == ["sum", "flat", "fc", "output"]
    assert not m.get_tensor("sum").any()
    m.clear_hooks()
    m.invoke(fixed_to_float=False)
    assert np.array_equal(m.get_tensor("fc"), want["fc"])
    # fake_quant_weight: filters rounded to 127 levels of their own maximum, biases untouched; the ops follow
    w2 = {k: v.copy() for k, v in weights.items()}
    w2["conv_filter"] = (w2["conv_filter"].astype(np.int32) // 3).astype(np.int8)      # maximum 42: the rounding changes values
    m2 = module()
    m2.load(graph, w2)
    m2.fake_quant_weight()
    fq = {}
    for k, v in w2.items():
        if k.endswith("_bias"):
            fq[k] = v
        else:
            f = v.astype(np.float32)
            mx = np.abs(f).max()
            fq[k] = (np.round(f * 127 / mx) * mx / 127).astype(v.dtype)
    want2 = oracle_graph.run(graph, fq, {"input": x})
    m2.set_tensor("input", x)
    m2.invoke(fixed_to_float=False)
    assert np.array_equal(m2.get_tensor("fc"), want2["fc"])
    assert m2.parser.get_next_op_by_op_name("pool") == ["sum"]
