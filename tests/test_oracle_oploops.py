"""The oracle's operator loops against the reference's OWN loops.

`make -C oracle ref_oploops` cuts the loops between the fp32 accumulator and the quantised output out of the reference
checkout (Conv2D.cpp:311-340, MatMul.cpp:637-728, Add.cpp:180-206, Pool2D.cpp:179-198, A16MatMul.cpp:190-197,
RequantIntAxis.cpp:18-120, RequantInt.cpp:18-71, CastUtils.cpp:15-47, MathUtils.cpp:849-872) and compiles them behind
a shim of accessors.  Every test feeds both sides the same seeded values, the reference side as the float buffers the
interpreter holds, and asks for identical results."""
import ctypes as C

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.skipif(not oracle.ref_oploops_available(), reason="compiled reference operator loops not present")

DT = {oracle.DT_I8: (8, 0), oracle.DT_U8: (8, 1), oracle.DT_I16: (16, 0), oracle.DT_I32: (32, 0)}


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _i64(a):
    return np.ascontiguousarray(a, dtype=np.int64)


def test_saturate():
    R = oracle.ref_oploops()
    vals = [0, 1, -1, 127, 128, -128, -129, 255, 256, 32767, 32768, -32768, -32769, 2**31 - 1, 2**31, -2**31, -2**31 - 1, 2**40, -2**40]
    for dt, (w, u) in DT.items():
        for v in vals:
            assert oracle.saturate(v, dt) == R.ref_saturate_i64(v, w, u), (v, dt)


def _conv_acc(rng, n, ic, hw, oc, k):
    """Integer accumulators of a small random convolution (exact, int64) and their float image."""
    x = rng.integers(-128, 128, (n, ic, hw, hw), dtype=np.int64)
    w = rng.integers(-127, 128, (oc, ic, k, k), dtype=np.int64)
    oh = hw - k + 1
    acc = np.zeros((n, oc, oh, oh), dtype=np.int64)
    for fy in range(k):
        for fx in range(k):
            acc += np.einsum("nchw,oc->nohw", x[:, :, fy:fy + oh, fx:fx + oh], w[:, :, fy, fx])
    return x.astype(np.int8), w.astype(np.int8), acc


@pytest.mark.parametrize("qmode,cv18xx", [(oracle.QM_MULTIPLIER_SHIFT, 0), (oracle.QM_QDM, 1), (oracle.QM_QDM, 0),
                                          (oracle.QM_TFLITE, 0), (oracle.QM_TFLITE_LSHIFT, 0), (oracle.QM_ONLY_SHIFT, 0)])
@pytest.mark.parametrize("per_axis", [True, False])
@pytest.mark.parametrize("do_relu,out_dt,zp", [(False, oracle.DT_I8, 0), (True, oracle.DT_U8, 0), (True, oracle.DT_I8, -5), (False, oracle.DT_I8, 3)])
def test_conv2d_requant(qmode, cv18xx, per_axis, do_relu, out_dt, zp):
    """Conv2D.cpp:311-340: float accumulator + int32 bias, applyMultiplierAndRShift with the dialect's rounding, zero
    point, ReLU as a floor at the zero point, saturate."""
    R = oracle.ref_oploops()
    rng = np.random.default_rng(hash((qmode, cv18xx, per_axis, do_relu, zp)) % 2**32)
    x, w, acc = _conv_acc(rng, 2, 8, 6, 5, 3)
    oc = 5
    bias = rng.integers(-2**12, 2**12, oc).astype(np.int32)
    cnt = oc if per_axis else 1
    if qmode == oracle.QM_MULTIPLIER_SHIFT:
        mult, rshift = rng.integers(2000, 30000, cnt), rng.integers(14, 24, cnt)
    elif qmode == oracle.QM_ONLY_SHIFT:
        mult, rshift = np.ones(cnt, np.int64), rng.integers(6, 12, cnt)
    else:
        mult = rng.integers(2**30, 2**31, cnt)
        rshift = rng.integers(8, 16, cnt) if cv18xx else -rng.integers(8, 16, cnt)   # BM168x: positive attribute = left shift
    got = oracle.conv2d_int8(x, w, bias, do_relu=do_relu, qmode=qmode, is_cv18xx=bool(cv18xx), mult=mult, rshift=rshift,
                             out_zp=zp, out_dt=out_dt)
    buf = np.ascontiguousarray(acc, dtype=np.float32)
    assert np.array_equal(buf.astype(np.int64), acc)   # inside the exact-float domain
    n, _, oh, ow = acc.shape
    width, uns = DT[out_dt]
    R.ref_conv2d_requant(_p(buf), n, oc, oh * ow, _p(_i64(rshift)), cnt, _p(_i64(mult)), cnt, _p(bias), qmode, int(do_relu), zp,
                         width, uns, cv18xx)
    assert np.array_equal(buf.astype(np.int64), got.astype(np.int64))
    # the oracle's other entry (float accumulators in, used by the CPU baseline) agrees as well
    got2 = np.empty(acc.shape, dtype=got.dtype)
    oracle.lib().orc_conv_requant_from_f32(_p(np.ascontiguousarray(acc, dtype=np.float32)), _p(bias), n, oc, oh * ow, int(do_relu),
                                           qmode, cv18xx, _p(_i64(mult)), _p(_i64(rshift)), cnt, zp, out_dt, _p(got2))
    assert np.array_equal(got2, got)


MATMUL_CASES = [
    dict(qmode=oracle.QM_MULTIPLIER_SHIFT, fuse_rq=False), dict(qmode=oracle.QM_MULTIPLIER_SHIFT, fuse_rq=True),
    dict(qmode=oracle.QM_TFLITE, fuse_rq=False), dict(qmode=oracle.QM_TFLITE_LSHIFT, fuse_rq=False),
    dict(qmode=oracle.QM_ONLY_SCALE, fuse_rq=False), dict(qmode=oracle.QM_QDM, cv18xx=True, batch=3),
    dict(qmode=oracle.QM_MULTIPLIER_SHIFT, cv18xx=True, batch=2),
]


@pytest.mark.parametrize("case", MATMUL_CASES)
@pytest.mark.parametrize("do_relu,out_dt,zp", [(False, oracle.DT_I8, 0), (True, oracle.DT_U8, 0), (False, oracle.DT_I8, 4)])
def test_matmul_requant(case, do_relu, out_dt, zp):
    """MatMul.cpp:637-728: bias and ReLU belong to the fp32 GEMM, then the dialect's requantisation (per batch on
    cv18xx, per channel with fuse_rq, per tensor otherwise), zero point, saturate."""
    R = oracle.ref_oploops()
    qmode, fuse_rq, cv, batch = case["qmode"], case.get("fuse_rq", False), case.get("cv18xx", False), case.get("batch", 1)
    if cv and zp != 0:
        pytest.skip("the cv18xx branch adds no zero point (MatMul.cpp:655-661)")
    rng = np.random.default_rng(hash((qmode, fuse_rq, cv, do_relu, zp)) % 2**32)
    M, K, N = 7, 48, 11
    A = rng.integers(-128, 128, (batch, M, K)).astype(np.int8)
    B = rng.integers(-128, 128, (batch, K, N) if batch > 1 else (K, N)).astype(np.int8)
    bias = rng.integers(-2**12, 2**12, N).astype(np.int32)
    scale = 0.0
    if cv:
        mult = rng.integers(2**30, 2**31, batch) if qmode == oracle.QM_QDM else rng.integers(500, 2000, batch)
        rshift = rng.integers(8, 14, batch)
    elif qmode == oracle.QM_MULTIPLIER_SHIFT and fuse_rq:
        mult, rshift = rng.integers(2000, 30000, N), np.array([int(rng.integers(16, 22))])
    elif qmode == oracle.QM_MULTIPLIER_SHIFT:
        mult, rshift = np.array([int(rng.integers(2000, 30000))]), np.array([int(rng.integers(16, 22))])
    elif qmode == oracle.QM_ONLY_SCALE:
        mult, rshift, scale = np.array([1]), np.array([0]), 0.00371
    else:
        mult, rshift = np.array([int(rng.integers(2**30, 2**31))]), np.array([int(rng.integers(8, 14))])
    got = oracle.matmul_int8(A if batch > 1 else A[0], B, bias, do_relu=do_relu, qmode=qmode, is_cv18xx=cv, fuse_rq=fuse_rq,
                             mult=mult, rshift=rshift, only_scale=scale, out_zp=zp, out_dt=out_dt)
    acc = np.einsum("bmk,bkn->bmn", A.astype(np.int64), (B if batch > 1 else B[None]).astype(np.int64)) + bias.astype(np.int64)
    if do_relu:
        acc = np.maximum(acc, 0)
    buf = np.ascontiguousarray(acc, dtype=np.float32)
    multi_operand = np.ascontiguousarray(mult, dtype=np.float32) if fuse_rq else None
    width, uns = DT[out_dt]
    # attribute arrays as MatMul.cpp:668-671 expects them: per batch on cv18xx; N entries with fuse_rq (only the first
    # shift is used and the multipliers come from the operand); one value otherwise
    n_mult = 0 if fuse_rq else len(mult)
    rshift_attr = np.repeat(rshift, N) if fuse_rq else rshift
    R.ref_matmul_requant(_p(buf), batch, M, N, _p(_i64(rshift_attr)), len(rshift_attr), _p(_i64(mult)), n_mult,
                         _p(multi_operand), qmode, int(fuse_rq), float(scale), zp, width, uns, int(cv), 1)
    assert np.array_equal(buf.reshape(got.shape).astype(np.int64), got.astype(np.int64))


@pytest.mark.parametrize("do_relu,out_dt", [(False, oracle.DT_I8), (True, oracle.DT_U8), (True, oracle.DT_I8)])
def test_add_int8(do_relu, out_dt):
    """Add.cpp:180-206: each input through applyMultiplierAndRShift (half up), fp32 add (+ReLU), saturate."""
    R = oracle.ref_oploops()
    rng = np.random.default_rng(5)
    a = rng.integers(-128, 128, 4096).astype(np.int8)
    b = rng.integers(0, 256, 4096).astype(np.uint8)
    for m0, s0, m1, s1 in [(77, 6, 101, 7), (126, 0, 1, 0), (3, 30, 120, 5), (64, 7, 64, 7)]:
        got = oracle.add_int8(a, b, m0, s0, m1, s1, do_relu=do_relu, out_dt=out_dt)
        out = np.zeros(4096, dtype=np.float32)
        width, uns = DT[out_dt]
        R.ref_add_int8(_p(a.astype(np.float32)), _p(b.astype(np.float32)), _p(out), 4096, m0, s0, m1, s1, int(do_relu), width, uns)
        assert np.array_equal(out.astype(np.int64), got.astype(np.int64)), (m0, s0, m1, s1)


def test_avgpool_window_sum_round_trip():
    """Pool2D.cpp:186 recovers the integer window sum from the pooling primitive's fp32 average as
    to_int(avg * kh * kw, half away).  The oracle (and the kernels) use the exact sum; the two agree as long as that
    round trip is the identity, which is checked here exhaustively for every window up to 8 x 8 and every sum an 8-bit
    input can produce, for both ways a primitive can form the average (division, multiplication by the reciprocal)."""
    R = oracle.ref_oploops()
    for kh in range(1, 9):
        for kw in range(1, 9):
            n = kh * kw
            s = np.arange(-255 * n, 255 * n + 1, dtype=np.int64)
            for avg in (s.astype(np.float32) / np.float32(n), s.astype(np.float32) * np.float32(1.0 / n)):
                buf = np.ascontiguousarray(avg, dtype=np.float32)
                R.ref_avgpool_int8(_p(buf), buf.size, kh, kw, 1, 1, 1, 0, 0, 32, 0, 0)   # multiplier 1, shift 0, 32-bit range
                assert np.array_equal(buf.astype(np.int64), s), (kh, kw)


@pytest.mark.parametrize("kernel,do_relu", [((7, 7), False), ((3, 3), True), ((2, 2), False)])
def test_avgpool_int8(kernel, do_relu):
    R = oracle.ref_oploops()
    rng = np.random.default_rng(9)
    kh, kw = kernel
    x = rng.integers(-128, 128, (2, 6, kh * 2, kw * 2)).astype(np.int8)
    multi, rshift = 83, 12
    got = oracle.pool2d_int8(x, kernel, kernel, (0, 0, 0, 0), mode="avg", multi=multi, rshift=rshift, do_relu=do_relu)
    sums = x.astype(np.int64).reshape(2, 6, 2, kh, 2, kw).sum(axis=(3, 5))
    avg = np.ascontiguousarray(sums.astype(np.float32) / np.float32(kh * kw))
    R.ref_avgpool_int8(_p(avg), avg.size, kh, kw, 1, multi, 1, rshift, int(do_relu), 8, 0, 0)
    assert np.array_equal(avg.astype(np.int64), got.astype(np.int64))


def test_a16_dequant_w4():
    """A16MatMul.cpp:190-197: flat index i, group i / q_group_size, low nibble first, (q - zp) * scale in fp32."""
    R = oracle.ref_oploops()
    rng = np.random.default_rng(2)
    for N, K, g in [(6, 128, 64), (5, 256, 128), (3, 64, 32)]:
        wq = rng.integers(0, 256, (N, K // 2)).astype(np.uint8)
        scale_bits = oracle.f32_to_bf16_bits_fast(rng.uniform(0.001, 0.02, N * K // g).astype(np.float32))
        zp = rng.integers(0, 16, N * K // g).astype(np.uint8)
        got = oracle.a16_dequant_w4(wq, scale_bits, zp, group=g)
        out = np.zeros((N, K), dtype=np.float32)
        R.ref_a16_dequant_w4(_p(wq.astype(np.float32)), _p(oracle.bf16_bits_to_f32(scale_bits)), _p(zp.astype(np.float32)), N, K, g, _p(out))
        assert out.tobytes() == got.tobytes()


@pytest.mark.parametrize("qmode,rmode", [(oracle.QM_MULTIPLIER_SHIFT, oracle.RM_HALF_UP), (oracle.QM_MULTIPLIER_SHIFT, oracle.RM_HALF_AWAY),
                                         (oracle.QM_TFLITE, oracle.RM_HALF_AWAY), (oracle.QM_TFLITE_LSHIFT, oracle.RM_HALF_UP)])
@pytest.mark.parametrize("fuse_axis", [False, True])
@pytest.mark.parametrize("words", [3, 2])
def test_requant_int_axis(qmode, rmode, fuse_axis, words):
    """RequantIntAxis.cpp:18-120 with both layouts of the quant operand: three words per channel {multiplier, shift,
    zero point} on BM1684X, two elsewhere {multiplier, shift in the low byte | zero point in the high half-word}."""
    if fuse_axis and qmode != oracle.QM_MULTIPLIER_SHIFT:
        pytest.skip("fuse_rq_axis exists for MultiplierShift only")
    R = oracle.ref_oploops()
    rng = np.random.default_rng(hash((qmode, rmode, fuse_axis, words)) % 2**32)
    Cn = 6
    shape = (3, 5, Cn) if fuse_axis else (3, Cn, 5, 2)
    x = rng.integers(-2**20, 2**20, shape).astype(np.int32)
    if qmode == oracle.QM_MULTIPLIER_SHIFT:
        mult = rng.integers(2000, 30000, Cn)
        shift = rng.integers(8, 24, Cn) if fuse_axis else -rng.integers(8, 24, Cn)   # stored negated unless fused (:103)
    else:
        mult, shift = rng.integers(2**30, 2**31, Cn), -rng.integers(6, 20, Cn)
    # the packed word travels through a float buffer: a non-negative zero point keeps it below 2^24, i.e. exact
    zp = rng.integers(0, 100, Cn) if words == 2 else rng.integers(-10, 10, Cn)
    if words == 2 and qmode != oracle.QM_MULTIPLIER_SHIFT:
        # a float operand keeps 24 bits: the two-word layout reads the multiplier through the same float
        mult = oracle.through_f32(mult)
    quant3 = np.stack([oracle.through_f32(mult), shift, zp], axis=1)
    got = oracle.requant_int_axis(x, quant3, qmode=qmode, rmode=rmode, fuse_rq_axis=fuse_axis, out_dt=oracle.DT_I8)
    if words == 3:
        q = quant3.astype(np.float32)
    else:
        packed = (shift.astype(np.int64) & 0xFF) | ((zp.astype(np.int64) & 0xFFFF) << 16)
        q = np.stack([mult.astype(np.float32), packed.astype(np.float32)], axis=1)
        # the packed word must survive its trip through the float buffer for the layout to mean anything
        if not np.array_equal(q[:, 1].astype(np.int64), packed):
            pytest.skip("this (shift, zero point) pair is not representable in a float-stored packed word")
    out = np.zeros(x.shape, dtype=np.float32)
    shp = _i64(shape)
    R.ref_requant_int_axis(_p(np.ascontiguousarray(x, dtype=np.float32)), _p(np.ascontiguousarray(q)), _p(out), _p(shp), len(shape),
                           qmode, rmode, int(fuse_axis), int(words == 3), 0, 0, 8, 0)
    assert np.array_equal(out.astype(np.int64), got.astype(np.int64))


@pytest.mark.parametrize("qmode,rmode", [(oracle.QM_MULTIPLIER_SHIFT, oracle.RM_HALF_UP), (oracle.QM_MULTIPLIER_SHIFT, oracle.RM_HALF_AWAY),
                                         (oracle.QM_TFLITE, oracle.RM_HALF_AWAY), (oracle.QM_TFLITE_LSHIFT, oracle.RM_HALF_UP)])
def test_requant_int(qmode, rmode):
    R = oracle.ref_oploops()
    rng = np.random.default_rng(hash((qmode, rmode)) % 2**32)
    shape = (2, 4, 9)
    x = rng.integers(-2**20, 2**20, shape).astype(np.int32)
    if qmode == oracle.QM_MULTIPLIER_SHIFT:
        multi, rshift = int(rng.integers(2000, 30000)), int(rng.integers(8, 24))
    else:
        multi, rshift = int(rng.integers(2**30, 2**31)), int(rng.integers(6, 20))
    for out_zp in (0, -7):
        got = oracle.requant_int(x, multi, rshift, qmode=qmode, rmode=rmode, out_zp=out_zp, out_dt=oracle.DT_I8)
        out = np.zeros(shape, dtype=np.float32)
        R.ref_requant_int(_p(np.ascontiguousarray(x, dtype=np.float32)), _p(out), _p(_i64(shape)), 3, multi, rshift, qmode, rmode, 0, 0,
                          out_zp, 8, 0)
        assert np.array_equal(out.astype(np.int64), got.astype(np.int64))


def test_cast_requant_dequant():
    """CastUtils.cpp:15-47 (f32 expressed type): round(x * (float)(1 / scale)) + zp before Cast.cpp's saturate, and
    (float)scale * (q - zp)."""
    R = oracle.ref_oploops()
    rng = np.random.default_rng(4)
    x = np.concatenate([rng.standard_normal(3000).astype(np.float32) * 3, np.array([0.5, -0.5, 1.5, 2.5, -2.5, 1e9, -1e9], np.float32)])
    for scale, zp, dt in [(0.0235, 0, oracle.DT_I8), (0.0371, 3, oracle.DT_I8), (0.011, 0, oracle.DT_U8)]:
        got = oracle.cast_f32_to_q8(x, scale, zp, out_dt=dt)
        width, uns = DT[dt]
        want = np.array([R.ref_saturate_f32(R.ref_cast_requant(float(v), scale, zp, 0), width, uns, oracle.RM_HALF_AWAY) for v in x])
        assert np.array_equal(got.astype(np.int64), want)
        back = oracle.cast_q8_to_f32(got, scale, zp)
        want_back = np.array([R.ref_cast_dequant(float(q), scale, zp, 0) for q in got], dtype=np.float32)
        assert back.tobytes() == want_back.tobytes()
