"""INT8 Conv2D parity on the GPU against the CPU oracle (bit exact), through both faces of the C ABI."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import tpu_mlir_b200._lib as L
from tpu_mlir_b200 import synth
from tpu_mlir_b200.ops import Conv2DOp, InferenceParameter

from gpu_util import Guarded, dev, dt_of, empty_dev, ptr

pytestmark = pytest.mark.gpu


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def oracle_conv(c, *, stride=(1, 1), pads=(1, 1, 1, 1), dilation=(1, 1), groups=1, qmode, is_cv18xx=False,
                do_relu=True, out_dt=oracle.DT_I8, out_zp=0, per_axis=True, rshift_sign=1):
    mult = c["mult"] if per_axis else c["mult"][:1]
    rshift = (c["rshift"] if per_axis else c["rshift"][:1]) * rshift_sign
    # oracle pads are (top, bottom, left, right); the op attribute is (top, left, bottom, right)
    out, viol = oracle.conv2d_int8(c["x"], c["w"], c["bias"], stride=stride, pads=(pads[0], pads[2], pads[1], pads[3]),
                                   dilation=dilation, groups=groups, do_relu=do_relu, qmode=qmode,
                                   is_cv18xx=is_cv18xx, mult=mult, rshift=rshift, out_zp=out_zp, out_dt=out_dt,
                                   return_violations=True)
    assert viol == 0, "inputs leave the domain where the reference's fp32 accumulation is exact"
    return out, mult, rshift


def run_operator_face(c, *, strides=(1, 1), pads=(1, 1, 1, 1), dilations=(1, 1), group=1, qmode, is_cv18xx=False,
                      do_relu=True, out_dt=L.DT_I8, out_zp=0, mult, rshift, algo=L.ALGO_AUTO):
    x, w = c["x"], c["w"]
    op = Conv2DOp(input_shape=x.shape, oc=w.shape[0], kernel_shape=w.shape[2:], strides=strides, dilations=dilations,
                  pads=pads, group=group, do_relu=do_relu, input_dtype=dt_of(x), out_dtype=out_dt, quant_mode=qmode,
                  is_cv18xx=is_cv18xx, out_zp=out_zp, multiplier=mult, rshift=rshift, algo=algo)
    out = np.full(op.out_shape, -777, np.float32)
    bias_buf = f32(c["bias"])
    p = InferenceParameter(inputs=[f32(x), f32(w), bias_buf], outputs=[out])
    op.init(p)
    op.inference(p)
    first = out.copy()
    out[...] = -777
    op.inference(p)     # resident weights, reused bordered buffer
    op.deinit(p)
    assert np.array_equal(first, out)
    assert np.array_equal(bias_buf, f32(c["bias"])), "the caller's bias buffer must not be modified"
    return out


@pytest.mark.parametrize("algo", [L.ALGO_TENSOR_CORE, L.ALGO_CUDA_CORE])
def test_operator_face_follows_weight_version(algo):
    """The interpreter rewrites filters in place (setTensor, fake_quant_weight: ModuleInterpreter.cpp:583-612).  The
    handle keeps its device copy until the descriptor's weight_version changes: the same version returns the cached
    result, a bumped version the result of the new filter and bias."""
    c = synth.conv2d_int8(seed=41, N=2, C=128, H=10, W=10, OC=32)
    c2 = synth.conv2d_int8(seed=42, N=2, C=128, H=10, W=10, OC=32)
    want1, mult, rshift = oracle_conv(c, qmode=oracle.QM_MULTIPLIER_SHIFT)
    want2, _, _ = oracle_conv(dict(c, w=c2["w"], bias=c2["bias"]), qmode=oracle.QM_MULTIPLIER_SHIFT)
    assert not np.array_equal(want1, want2)
    op = Conv2DOp(input_shape=c["x"].shape, oc=32, kernel_shape=(3, 3), pads=(1, 1, 1, 1), do_relu=True,
                  quant_mode=L.QM_MULTIPLIER_SHIFT, multiplier=mult, rshift=rshift, algo=algo)
    w_buf, b_buf = f32(c["w"]), f32(c["bias"])
    out = np.zeros(op.out_shape, np.float32)
    p = InferenceParameter(inputs=[f32(c["x"]), w_buf, b_buf], outputs=[out])
    op.init(p)
    op.inference(p)
    assert np.array_equal(out, want1.astype(np.float32))
    w_buf[...] = c2["w"]          # rewritten in place, version not bumped: the resident copy still answers
    b_buf[...] = c2["bias"]
    op.inference(p)
    assert np.array_equal(out, want1.astype(np.float32))
    op.invalidate_weights()
    op.inference(p)
    assert np.array_equal(out, want2.astype(np.float32))
    op.inference(p)
    assert np.array_equal(out, want2.astype(np.float32))
    op.deinit(p)


@pytest.mark.parametrize("algo", [L.ALGO_TENSOR_CORE, L.ALGO_CUDA_CORE])
def test_conv3x3_qdm_small(algo):
    """Shape family of BASELINE config 1 at a size the oracle finishes quickly: 3x3, stride 1, pad 1, ReLU, QDM."""
    c = synth.conv2d_int8(seed=21, N=3, C=128, H=13, W=11, OC=72)
    # BASELINE's form RSR(RSR(acc*M,31), rshift, half away) is QDM with the CV18xx shift-sign convention
    want, mult, rshift = oracle_conv(c, qmode=oracle.QM_QDM, is_cv18xx=True)
    got = run_operator_face(c, qmode=L.QM_QDM, is_cv18xx=True, mult=mult, rshift=rshift, algo=algo)
    assert np.array_equal(got, want.astype(np.float32))


@pytest.mark.parametrize("case", [
    dict(N=2, C=256, H=9, W=9, OC=256, k=3, pads=(1, 1, 1, 1)),            # two K blocks per tap, full N tile
    dict(N=1, C=128, H=8, W=20, OC=40, k=3, pads=(0, 0, 0, 0)),            # "valid" convolution
    dict(N=2, C=128, H=7, W=7, OC=130, k=3, pads=(1, 0, 0, 1)),            # asymmetric pads
    dict(N=2, C=64, H=14, W=14, OC=256, k=1, pads=(0, 0, 0, 0)),           # 1x1, K < 128
    dict(N=1, C=48, H=5, W=6, OC=24, k=1, pads=(0, 0, 0, 0)),              # 1x1, K multiple of 16 only
    dict(N=1, C=128, H=6, W=6, OC=8, k=5, pads=(2, 2, 2, 2)),              # 5x5
    # larger images: CTA-pair tiles, several channel tiles, odd sizes
    dict(N=3, C=128, H=13, W=28, OC=300, k=3, pads=(1, 1, 1, 1)),          # two channel tiles, odd height
    dict(N=2, C=256, H=30, W=17, OC=136, k=3, pads=(1, 1, 1, 1)),          # odd width
    dict(N=5, C=128, H=11, W=64, OC=96, k=3, pads=(1, 1, 0, 2)),           # asymmetric pads
    dict(N=2, C=80, H=16, W=16, OC=512, k=1, pads=(0, 0, 0, 0)),           # 1x1 with a ragged K block
    # 64 channels: horizontally adjacent taps are paired into one 128-byte K block
    dict(N=3, C=64, H=12, W=20, OC=64, k=3, pads=(1, 1, 1, 1)),            # 3x3: the third tap pairs with zeros
    dict(N=2, C=64, H=9, W=11, OC=200, k=3, pads=(0, 0, 0, 0)),            # no border: the last pixel is data
    dict(N=1, C=64, H=10, W=10, OC=32, k=2, pads=(0, 1, 1, 0)),            # even filter width
    dict(N=1, C=64, H=8, W=9, OC=16, k=5, pads=(2, 2, 2, 2)),              # 5x5
])
def test_conv_tensor_core_shapes(case):
    c = synth.conv2d_int8(seed=case["C"] + case["OC"], N=case["N"], C=case["C"], H=case["H"], W=case["W"],
                          OC=case["OC"], KH=case["k"], KW=case["k"], unsigned_input=True)
    c["w"] = np.clip(c["w"] // 2, -127, 127).astype(np.int8)   # u8 activations: keep |acc| < 2^24
    c["mult"] = np.random.default_rng(1).integers(5000, 30000, size=case["OC"])
    c["rshift"] = np.random.default_rng(2).integers(18, 26, size=case["OC"])
    want, mult, rshift = oracle_conv(c, pads=case["pads"], qmode=oracle.QM_MULTIPLIER_SHIFT, out_dt=oracle.DT_U8)
    got = run_operator_face(c, pads=case["pads"], qmode=L.QM_MULTIPLIER_SHIFT, out_dt=L.DT_U8, mult=mult, rshift=rshift,
                            algo=L.ALGO_TENSOR_CORE)
    assert np.array_equal(got, want.astype(np.float32))


@pytest.mark.parametrize("case", [
    dict(N=2, C=3, H=32, W=32, OC=16, k=7, stride=(2, 2), pads=(3, 3, 3, 3), group=1, dil=(1, 1)),   # ResNet stem
    dict(N=1, C=16, H=12, W=12, OC=16, k=3, stride=(1, 1), pads=(1, 1, 1, 1), group=16, dil=(1, 1)),  # depthwise
    dict(N=1, C=8, H=15, W=15, OC=12, k=3, stride=(2, 1), pads=(2, 2, 2, 2), group=2, dil=(2, 2)),    # dilation, groups
    # depthwise shapes of the patch kernel: 4-row and 2-row patches, ragged edges, both strides and filter sizes, uneven pads
    dict(N=2, C=24, H=28, W=28, OC=24, k=3, stride=(1, 1), pads=(1, 1, 1, 1), group=24, dil=(1, 1)),
    dict(N=2, C=10, H=29, W=31, OC=10, k=3, stride=(2, 2), pads=(0, 1, 1, 0), group=10, dil=(1, 1)),
    dict(N=3, C=7, H=7, W=7, OC=7, k=3, stride=(1, 1), pads=(1, 1, 1, 1), group=7, dil=(1, 1)),
    dict(N=1, C=5, H=17, W=13, OC=5, k=5, stride=(1, 1), pads=(2, 2, 2, 2), group=5, dil=(1, 1)),
    dict(N=2, C=6, H=14, W=14, OC=6, k=5, stride=(2, 2), pads=(2, 1, 1, 2), group=6, dil=(1, 1)),
    dict(N=1, C=4, H=3, W=2, OC=4, k=3, stride=(1, 1), pads=(1, 1, 1, 1), group=4, dil=(1, 1)),
    # eight-column patches (output width a multiple of 8, or rounding up the same way as to 4), a one-patch plane
    dict(N=2, C=9, H=13, W=16, OC=9, k=3, stride=(1, 1), pads=(1, 1, 1, 1), group=9, dil=(1, 1)),
    dict(N=1, C=6, H=27, W=47, OC=6, k=3, stride=(2, 2), pads=(1, 1, 0, 1), group=6, dil=(1, 1)),
    dict(N=2, C=3, H=56, W=56, OC=3, k=3, stride=(1, 1), pads=(1, 1, 1, 1), group=3, dil=(1, 1)),
    dict(N=3, C=300, H=2, W=2, OC=300, k=3, stride=(1, 1), pads=(1, 1, 1, 1), group=300, dil=(1, 1)),
])
def test_conv_cuda_core_shapes(case):
    rng = np.random.default_rng(77)
    x = rng.integers(-128, 128, size=(case["N"], case["C"], case["H"], case["W"]), dtype=np.int8)
    w = rng.integers(-127, 128, size=(case["OC"], case["C"] // case["group"], case["k"], case["k"]), dtype=np.int8)
    c = dict(x=x, w=w, bias=rng.integers(-500, 500, size=case["OC"], dtype=np.int32),
             mult=rng.integers(100, 20000, size=case["OC"]), rshift=rng.integers(10, 20, size=case["OC"]))
    for qmode, per_axis in ((oracle.QM_MULTIPLIER_SHIFT, True), (oracle.QM_ONLY_SHIFT, False), (oracle.QM_TFLITE, True)):
        sign = -1 if qmode == oracle.QM_TFLITE else 1    # BM168x TFLite: positive shift attribute = left shift
        want, mult, rshift = oracle_conv(c, stride=case["stride"], pads=case["pads"], dilation=case["dil"],
                                         groups=case["group"], qmode=qmode, per_axis=per_axis, out_zp=-4,
                                         do_relu=(qmode != oracle.QM_ONLY_SHIFT), rshift_sign=sign)
        got = run_operator_face(c, strides=case["stride"], pads=case["pads"], dilations=case["dil"], group=case["group"],
                                qmode=qmode, mult=mult, rshift=rshift, out_zp=-4,
                                do_relu=(qmode != oracle.QM_ONLY_SHIFT))
        assert np.array_equal(got, want.astype(np.float32)), (case, qmode)


@pytest.mark.parametrize("u8_in", [False, True])
def test_depthwise_requant_forms(u8_in):
    """The depthwise kernel's three MultiplierShift forms: shifts of 32 and more with 31-bit multipliers, small multipliers
    under a short shift (scaled to a 32-bit binary point) and multipliers too large for that; signed and unsigned inputs,
    a non-zero output zero point with ReLU."""
    rng = np.random.default_rng(78)
    C_ = 12
    x = rng.integers(0, 256, size=(2, C_, 19, 23)).astype(np.uint8) if u8_in else rng.integers(-128, 128, size=(2, C_, 19, 23), dtype=np.int8)
    w = rng.integers(-127, 128, size=(C_, 1, 3, 3), dtype=np.int8)
    mult = np.array([2**30 + 12345, -(2**30) + 999, 1_500_000_000, 900_000_000, 37, 500, 20000, 19999, 3, 1, 65535, 2**20], dtype=np.int64)
    rshift = np.array([44, 45, 46, 32, 8, 12, 11, 15, 2, 1, 20, 30], dtype=np.int64)
    c = dict(x=x, w=w, bias=rng.integers(-3000, 3000, size=C_, dtype=np.int32), mult=mult, rshift=rshift)
    want, m_, s_ = oracle_conv(c, groups=C_, qmode=oracle.QM_MULTIPLIER_SHIFT, out_zp=5, do_relu=True)
    got = run_operator_face(c, group=C_, qmode=L.QM_MULTIPLIER_SHIFT, mult=m_, rshift=s_, out_zp=5, do_relu=True)
    assert np.array_equal(got, want.astype(np.float32)) and len(np.unique(want)) > 40


def test_conv_device_face_matches_operator_face():
    c = synth.conv2d_int8(seed=8, N=4, C=128, H=10, W=10, OC=64)
    want, mult, rshift = oracle_conv(c, qmode=oracle.QM_QDM, is_cv18xx=True)
    d = Conv2DOp(input_shape=c["x"].shape, oc=64, kernel_shape=(3, 3), pads=(1, 1, 1, 1), do_relu=True,
                 quant_mode=L.QM_QDM, is_cv18xx=True, multiplier=mult, rshift=rshift).desc
    w_d, b_d, x_d = dev(c["w"]), dev(c["bias"]), dev(c["x"])
    y_d = empty_dev(want.shape, L.DT_I8)
    h = C.c_void_p()
    lib = L.lib()
    L.check(lib.b200q_conv2d_dev_create(C.byref(d), ptr(w_d), ptr(b_d), C.byref(h)))
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(3):
            L.check(lib.b200q_conv2d_dev_run(h, ptr(x_d), ptr(y_d), C.c_void_p(stream.cuda_stream)))
    L.check(lib.b200q_conv2d_dev_status(h, C.c_void_p(stream.cuda_stream)))
    lib.b200q_conv2d_dev_destroy(C.byref(h))
    assert np.array_equal(y_d.cpu().numpy(), want)


@pytest.mark.parametrize("misalign", [0, 1, 3])
def test_depthwise_device_face_pad_value_and_misaligned_input(misalign):
    """The depthwise kernel through the device face: unsigned input padded with its zero point (the byte masks' fill value), and
    an input tensor that does not start on a 4-byte boundary (every patch then takes the byte-wise loop)."""
    rng = np.random.default_rng(79)
    C_, H, W = 20, 17, 22
    x = rng.integers(0, 256, size=(3, C_, H, W)).astype(np.uint8)
    w = rng.integers(-127, 128, size=(C_, 1, 3, 3), dtype=np.int8)
    bias = rng.integers(-3000, 3000, size=C_, dtype=np.int32)
    mult, rshift = rng.integers(2000, 9000, size=C_), rng.integers(17, 21, size=C_)
    want = oracle.conv2d_int8(x, w, bias, pads=(1, 1, 1, 1), groups=C_, pad_value=131, do_relu=True, qmode=oracle.QM_MULTIPLIER_SHIFT,
                              mult=mult, rshift=rshift, out_zp=-3)
    d = Conv2DOp(input_shape=x.shape, oc=C_, kernel_shape=(3, 3), pads=(1, 1, 1, 1), group=C_, pad_value=131, do_relu=True,
                 input_dtype=L.DT_U8, quant_mode=L.QM_MULTIPLIER_SHIFT, multiplier=mult, rshift=rshift, out_zp=-3).desc
    buf = torch.zeros(x.size + 8, dtype=torch.uint8, device="cuda")
    x_d = buf[misalign:misalign + x.size]
    x_d.copy_(torch.from_numpy(x.reshape(-1)).cuda())
    assert x_d.data_ptr() % 4 == misalign % 4
    w_d, b_d = dev(w), dev(bias)
    y_d = empty_dev(want.shape, L.DT_I8)
    h = C.c_void_p()
    lib = L.lib()
    L.check(lib.b200q_conv2d_dev_create(C.byref(d), ptr(w_d), ptr(b_d), C.byref(h)))
    L.check(lib.b200q_conv2d_dev_run(h, ptr(x_d), ptr(y_d), None))
    L.check(lib.b200q_conv2d_dev_status(h, None))
    lib.b200q_conv2d_dev_destroy(C.byref(h))
    assert np.array_equal(y_d.cpu().numpy(), want) and len(np.unique(want)) > 40


@pytest.mark.parametrize("case", [
    dict(N=2, C=64, H=14, W=14, OC=256, k=1, stride=(1, 1), pads=(0, 0, 0, 0)),     # 1x1: x is read in place
    dict(N=3, C=128, H=13, W=11, OC=80, k=3, stride=(1, 1), pads=(1, 1, 1, 1)),     # 3x3 through the bordered image
    dict(N=2, C=64, H=12, W=20, OC=64, k=3, stride=(1, 1), pads=(1, 1, 1, 1)),      # 64 channels: paired taps
    dict(N=2, C=128, H=9, W=8, OC=48, k=3, stride=(1, 1), pads=(0, 0, 0, 0)),       # "valid" 3x3 read in place
    dict(N=2, C=128, H=14, W=14, OC=128, k=3, stride=(2, 2), pads=(1, 1, 1, 1)),    # strided 3x3: im2col rows
    dict(N=2, C=256, H=14, W=14, OC=512, k=1, stride=(2, 2), pads=(0, 0, 0, 0)),    # strided 1x1 (a downsample branch)
    dict(N=1, C=32, H=7, W=9, OC=272, k=1, stride=(1, 1), pads=(0, 0, 0, 0)),       # ragged channel tile
    # output channels a multiple of 128: the transposed product (rows = channels, per-row requantisation constants)
    dict(N=3, C=128, H=9, W=7, OC=128, k=1, stride=(1, 1), pads=(0, 0, 0, 0)),      # one row tile, ragged pixel tile
    dict(N=2, C=48, H=20, W=20, OC=384, k=1, stride=(1, 1), pads=(0, 0, 0, 0)),     # three row tiles
    dict(N=40, C=64, H=28, W=28, OC=256, k=1, stride=(1, 1), pads=(0, 0, 0, 0)),    # enough tiles for CTA pairs
])
@pytest.mark.parametrize("layouts", [(1, 1), (0, 1), (1, 0)])
def test_conv_device_face_channels_last(case, layouts):
    """b200q_conv2d_dev_run_layout: the same values as the NCHW run, for every mix of input and output layout."""
    c = synth.conv2d_int8(seed=case["C"] + case["OC"] + case["H"], N=case["N"], C=case["C"], H=case["H"], W=case["W"],
                          OC=case["OC"], KH=case["k"], KW=case["k"], unsigned_input=True)
    c["w"] = np.clip(c["w"] // 2, -127, 127).astype(np.int8)
    c["mult"] = np.random.default_rng(1).integers(5000, 30000, size=case["OC"])
    c["rshift"] = np.random.default_rng(2).integers(18, 26, size=case["OC"])
    want, mult, rshift = oracle_conv(c, stride=case["stride"], pads=case["pads"], qmode=oracle.QM_MULTIPLIER_SHIFT,
                                     out_dt=oracle.DT_U8)
    d = Conv2DOp(input_shape=c["x"].shape, oc=case["OC"], kernel_shape=(case["k"], case["k"]), strides=case["stride"],
                 pads=case["pads"], do_relu=True, input_dtype=L.DT_U8, out_dtype=L.DT_U8, quant_mode=L.QM_MULTIPLIER_SHIFT,
                 multiplier=mult, rshift=rshift).desc
    xl, yl = layouts
    x = c["x"].transpose(0, 2, 3, 1) if xl else c["x"]
    w_d, b_d, x_d = dev(c["w"]), dev(c["bias"]), dev(np.ascontiguousarray(x))
    y_shape = (want.shape[0], want.shape[2], want.shape[3], want.shape[1]) if yl else want.shape
    guard = Guarded(y_shape, torch.uint8, fill=77)     # canary bytes around the output (ragged pixel and channel tiles)
    y_d = guard.view
    h = C.c_void_p()
    lib = L.lib()
    L.check(lib.b200q_conv2d_dev_create(C.byref(d), ptr(w_d), ptr(b_d), C.byref(h)))
    for _ in range(2):
        L.check(lib.b200q_conv2d_dev_run_layout(h, ptr(x_d), xl, ptr(y_d), yl, None))
    L.check(lib.b200q_conv2d_dev_status(h, None))
    lib.b200q_conv2d_dev_destroy(C.byref(h))
    guard.check()
    got = y_d.cpu().numpy()
    assert np.array_equal(got.transpose(0, 3, 1, 2) if yl else got, want)


def test_conv_channels_last_needs_a_tensor_core_route():
    rng = np.random.default_rng(5)
    w = rng.integers(-127, 128, size=(16, 1, 3, 3), dtype=np.int8)
    d = Conv2DOp(input_shape=(1, 16, 8, 8), oc=16, kernel_shape=(3, 3), pads=(1, 1, 1, 1), group=16,
                 quant_mode=L.QM_MULTIPLIER_SHIFT, multiplier=[1000] * 16, rshift=[12] * 16, with_bias=False).desc
    w_d = dev(w)
    x_d, y_d = torch.zeros(1, 8, 8, 16, dtype=torch.int8, device="cuda"), torch.zeros(1, 8, 8, 16, dtype=torch.int8, device="cuda")
    h = C.c_void_p()
    lib = L.lib()
    L.check(lib.b200q_conv2d_dev_create(C.byref(d), ptr(w_d), None, C.byref(h)))
    assert lib.b200q_conv2d_dev_run_layout(h, ptr(x_d), 1, ptr(y_d), 1, None) == L.ERR_UNSUPPORTED
    assert lib.b200q_conv2d_dev_run_layout(h, ptr(x_d), 7, ptr(y_d), 0, None) == L.ERR_INVALID
    lib.b200q_conv2d_dev_destroy(C.byref(h))


def test_conv_back_to_back_runs_read_fresh_inputs():
    """The convolution kernel launches as a programmatic dependent of its layout kernel (it becomes resident while the
    layout kernel drains and waits for it before reading the image): alternating inputs queued without any
    synchronisation must each produce their own result."""
    ca = synth.conv2d_int8(seed=91, N=8, C=128, H=28, W=28, OC=128)
    cb = dict(ca)
    cb["x"] = np.random.default_rng(92).integers(-128, 128, size=ca["x"].shape, dtype=np.int8)
    want_a, mult, rshift = oracle_conv(ca, qmode=oracle.QM_QDM, is_cv18xx=True)
    want_b, _, _ = oracle_conv(cb, qmode=oracle.QM_QDM, is_cv18xx=True)
    d = Conv2DOp(input_shape=ca["x"].shape, oc=128, kernel_shape=(3, 3), pads=(1, 1, 1, 1), do_relu=True,
                 quant_mode=L.QM_QDM, is_cv18xx=True, multiplier=mult, rshift=rshift).desc
    w_d, b_d, xa_d, xb_d = dev(ca["w"]), dev(ca["bias"]), dev(ca["x"]), dev(cb["x"])
    ya_d, yb_d = empty_dev(want_a.shape, L.DT_I8), empty_dev(want_a.shape, L.DT_I8)
    h = C.c_void_p()
    lib = L.lib()
    L.check(lib.b200q_conv2d_dev_create(C.byref(d), ptr(w_d), ptr(b_d), C.byref(h)))
    for _ in range(25):
        L.check(lib.b200q_conv2d_dev_run(h, ptr(xa_d), ptr(ya_d), None))
        L.check(lib.b200q_conv2d_dev_run(h, ptr(xb_d), ptr(yb_d), None))
    L.check(lib.b200q_conv2d_dev_status(h, None))
    lib.b200q_conv2d_dev_destroy(C.byref(h))
    assert np.array_equal(ya_d.cpu().numpy(), want_a)
    assert np.array_equal(yb_d.cpu().numpy(), want_b)


def test_config1_full_size():
    """BASELINE config 1 at full size: N=32, C=256, 56x56, OC=256, 3x3, stride 1, pad 1, fused ReLU, QDM requant."""
    c = synth.conv2d_int8(seed=1)
    want, mult, rshift = oracle_conv(c, qmode=oracle.QM_QDM, is_cv18xx=True)
    got = run_operator_face(c, qmode=L.QM_QDM, is_cv18xx=True, mult=mult, rshift=rshift, algo=L.ALGO_TENSOR_CORE)
    assert np.array_equal(got, want.astype(np.float32))


@pytest.mark.parametrize("case", [
    dict(N=2, C=64, H=12, W=20, OC=256, k=1, do_relu=False),     # 1x1, channels a multiple of 128: transposed product
    dict(N=3, C=128, H=9, W=7, OC=80, k=1, do_relu=False),       # pixel-major, ragged channel tile
    dict(N=2, C=128, H=13, W=11, OC=96, k=3, do_relu=True),      # 3x3 through the bordered image
    dict(N=2, C=256, H=14, W=14, OC=512, k=1, stride=(2, 2), do_relu=False),   # strided 1x1 (downsample branch): im2col rows
    dict(N=40, C=64, H=28, W=28, OC=256, k=1, do_relu=False),    # enough tiles for CTA pairs
])
@pytest.mark.parametrize("layout", [1, 0])
@pytest.mark.parametrize("res_unsigned,add_relu", [(True, True), (False, False)])
def test_conv_with_fused_residual_add(case, layout, res_unsigned, add_relu):
    """b200q_conv2d_dev_run_add: the convolution followed by tpu.Add (Add.cpp:177-207) in one kernel equals the oracle's
    convolution followed by the oracle's Add, in both layouts, with the convolution as either kind of operand."""
    stride = case.get("stride", (1, 1))
    pads = (1, 1, 1, 1) if case["k"] == 3 else (0, 0, 0, 0)
    c = synth.conv2d_int8(seed=case["C"] + case["OC"], N=case["N"], C=case["C"], H=case["H"], W=case["W"], OC=case["OC"],
                          KH=case["k"], KW=case["k"], unsigned_input=True)
    c["w"] = np.clip(c["w"] // 2, -127, 127).astype(np.int8)
    c["mult"] = np.random.default_rng(1).integers(5000, 30000, size=case["OC"])
    c["rshift"] = np.random.default_rng(2).integers(18, 24, size=case["OC"])
    conv_dt = oracle.DT_U8 if case["do_relu"] else oracle.DT_I8
    conv_out, mult, rshift = oracle_conv(c, stride=stride, pads=pads, qmode=oracle.QM_MULTIPLIER_SHIFT, do_relu=case["do_relu"],
                                         out_dt=conv_dt)
    rng = np.random.default_rng(9)
    res = rng.integers(0, 256, conv_out.shape).astype(np.uint8) if res_unsigned else rng.integers(-128, 128, conv_out.shape).astype(np.int8)
    m_c, s_c, m_r, s_r = 19001, 14, 23456, 15
    out_dt = oracle.DT_U8 if add_relu else oracle.DT_I8
    want = oracle.add_int8(conv_out, res, m_c, s_c, m_r, s_r, do_relu=add_relu, out_dt=out_dt)
    assert len(np.unique(want)) > 50
    d = Conv2DOp(input_shape=c["x"].shape, oc=case["OC"], kernel_shape=(case["k"], case["k"]), strides=stride, pads=pads,
                 do_relu=case["do_relu"], input_dtype=L.DT_U8, out_dtype=L.DT_U8 if case["do_relu"] else L.DT_I8,
                 quant_mode=L.QM_MULTIPLIER_SHIFT, multiplier=mult, rshift=rshift).desc
    to_l = (lambda t: np.ascontiguousarray(t.transpose(0, 2, 3, 1))) if layout else (lambda t: np.ascontiguousarray(t))
    w_d, b_d, x_d, r_d = dev(c["w"]), dev(c["bias"]), dev(to_l(c["x"])), dev(to_l(res))
    guard = Guarded(to_l(want).shape, torch.uint8 if add_relu else torch.int8, fill=77)
    h = C.c_void_p()
    lib = L.lib()
    L.check(lib.b200q_conv2d_dev_create(C.byref(d), ptr(w_d), ptr(b_d), C.byref(h)))
    assert lib.b200q_conv2d_dev_route(h) in (1, 2)
    fa = L.FusedAdd(residual=r_d.data_ptr(), residual_dtype=L.DT_U8 if res_unsigned else L.DT_I8, conv_multiplier=m_c,
                    conv_rshift=s_c, residual_multiplier=m_r, residual_rshift=s_r, do_relu=int(add_relu),
                    out_dtype=L.DT_U8 if add_relu else L.DT_I8)
    for _ in range(2):
        L.check(lib.b200q_conv2d_dev_run_add(h, ptr(x_d), layout, ptr(guard.view), layout, C.byref(fa), None))
    L.check(lib.b200q_conv2d_dev_status(h, None))
    lib.b200q_conv2d_dev_destroy(C.byref(h))
    guard.check()
    got = guard.view.cpu().numpy()
    assert np.array_equal(got.transpose(0, 3, 1, 2) if layout else got, want)


def test_fused_add_refusals():
    c = synth.conv2d_int8(seed=3, N=1, C=32, H=8, W=8, OC=32, KH=3, KW=3)
    d = Conv2DOp(input_shape=c["x"].shape, oc=32, kernel_shape=(3, 3), pads=(1, 1, 1, 1), quant_mode=L.QM_MULTIPLIER_SHIFT,
                 multiplier=[3], rshift=[9]).desc
    w_d, b_d, x_d = dev(c["w"]), dev(c["bias"]), dev(c["x"])
    y = empty_dev((1, 32, 8, 8), L.DT_I8)
    h = C.c_void_p()
    lib = L.lib()
    L.check(lib.b200q_conv2d_dev_create(C.byref(d), ptr(w_d), ptr(b_d), C.byref(h)))
    fa = L.FusedAdd(residual=y.data_ptr(), residual_dtype=L.DT_I8, conv_multiplier=1 << 24, conv_rshift=3,
                    residual_multiplier=5, residual_rshift=3, do_relu=0, out_dtype=L.DT_I8)
    assert lib.b200q_conv2d_dev_run_add(h, ptr(x_d), 0, ptr(y), 0, C.byref(fa), None) == L.ERR_UNSUPPORTED   # multiplier too wide
    fa.conv_multiplier, fa.residual_dtype = 7, L.DT_I32
    assert lib.b200q_conv2d_dev_run_add(h, ptr(x_d), 0, ptr(y), 0, C.byref(fa), None) == L.ERR_INVALID
    lib.b200q_conv2d_dev_destroy(C.byref(h))
