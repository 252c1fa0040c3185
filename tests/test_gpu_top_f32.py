"""fp32 Top-dialect forward kernels on the GPU against the oracle's restatement of top::ConvOp / Pool / Add / Relu /
MatMul (tolerance: the reference's oneDNN does not define a summation order; the kernels keep full fp32 products and
sums, so the bound is a few ulps of the accumulated magnitude: |y - ref| <= 1e-5 * sum_k |x_k * w_k| + 1e-6)."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import oracle  # noqa: E402
from tpu_mlir_b200 import _lib as L  # noqa: E402
from tpu_mlir_b200 import resnet50  # noqa: E402
from tpu_mlir_b200.ops import InferenceParameter, TopConvOp  # noqa: E402


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def conv_bound(x, w, **kw):
    """1e-5 * sum |x| * |w| per output + 1e-6."""
    mag = oracle.top_conv2d_f32(np.abs(x), np.abs(w), None, **{k: v for k, v in kw.items() if k in ("stride", "pads", "dilation", "groups")})
    return 1e-5 * mag + 1e-6


CASES = [
    dict(n=2, ic=64, hw=(56, 56), oc=256, k=(1, 1)),                                   # ResNet 1x1 expand
    dict(n=2, ic=64, hw=(56, 56), oc=64, k=(3, 3), pads=(1, 1, 1, 1)),                 # 64-channel tile
    dict(n=3, ic=3, hw=(224, 224), oc=64, k=(7, 7), stride=(2, 2), pads=(3, 3, 3, 3)), # stem
    dict(n=2, ic=256, hw=(14, 14), oc=512, k=(3, 3), stride=(2, 2), pads=(1, 1, 1, 1)),# 7 x 7 output: scalar stores
    dict(n=1, ic=20, hw=(9, 11), oc=50, k=(3, 2), stride=(2, 1), pads=(1, 0, 2, 1), dilation=(1, 2)),  # ragged everything
    dict(n=2, ic=16, hw=(12, 12), oc=24, k=(3, 3), pads=(1, 1, 1, 1), groups=4),       # grouped
    dict(n=2, ic=32, hw=(10, 10), oc=32, k=(3, 3), pads=(1, 1, 1, 1), groups=32),      # depthwise
    dict(n=1, ic=7, hw=(5, 5), oc=3, k=(5, 5)),                                        # one output pixel
    dict(n=5, ic=130, hw=(6, 6), oc=131, k=(1, 1)),                                    # channel counts off the vector width
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("relu", [False, True])
def test_conv_device_face(case, relu):
    rng = np.random.default_rng(3)
    n, ic, (ih, iw), oc, (kh, kw) = case["n"], case["ic"], case["hw"], case["oc"], case["k"]
    stride, pads, dil, groups = case.get("stride", (1, 1)), case.get("pads", (0, 0, 0, 0)), case.get("dilation", (1, 1)), case.get("groups", 1)
    x = rng.standard_normal((n, ic, ih, iw)).astype(np.float32)
    w = (rng.standard_normal((oc, ic // groups, kh, kw)) / np.sqrt(ic // groups * kh * kw)).astype(np.float32)
    b = rng.standard_normal(oc).astype(np.float32)
    limit = 0.75 if relu else -1.0
    ref = oracle.top_conv2d_f32(x, w, b, stride=stride, pads=pads, dilation=dil, groups=groups, do_relu=relu, relu_limit=limit)
    d = L.TopConvDesc(n=n, ic=ic, ih=ih, iw=iw, oc=oc, kh=kh, kw=kw, sh=stride[0], sw=stride[1], dh=dil[0], dw=dil[1], pht=pads[0],
                      phb=pads[1], pwl=pads[2], pwr=pads[3], groups=groups, with_bias=1, do_relu=int(relu), relu_limit=limit)
    xd, wd, bd = dev(x), dev(w), dev(b)
    h = C.c_void_p()
    L.check(L.lib().b200q_top_conv2d_dev_create(C.byref(d), ptr(wd), ptr(bd), C.byref(h)))
    y = torch.full(ref.shape, float("nan"), dtype=torch.float32, device="cuda")
    L.check(L.lib().b200q_top_conv2d_dev_run(h, ptr(xd), ptr(y), n, None))
    torch.cuda.synchronize()
    L.lib().b200q_top_conv2d_dev_destroy(C.byref(h))
    got = y.cpu().numpy()
    bound = conv_bound(x, w, stride=stride, pads=pads, dilation=dil, groups=groups)
    assert np.all(np.abs(got - ref) <= bound), float(np.abs(got - ref).max())


def test_conv_operator_face():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((2, 8, 13, 13)).astype(np.float32)
    w = rng.standard_normal((10, 8, 3, 3)).astype(np.float32) * 0.1
    b = rng.standard_normal(10).astype(np.float32)
    op = TopConvOp(input_shape=x.shape, oc=10, kernel_shape=(3, 3), strides=(2, 2), pads=(1, 1, 0, 0), do_relu=True)
    out = np.zeros(op.out_shape, np.float32)
    p = InferenceParameter(inputs=[x, w, b], outputs=[out])
    with pytest.raises(L.B200QError):
        op.inference(p)                       # no init: the reference fails the same way (Conv.cpp:223-225)
    op.init(p)
    op.inference(p)
    op.deinit(p)
    ref = oracle.top_conv2d_f32(x, w, b, stride=(2, 2), pads=(1, 0, 1, 0), do_relu=True)
    assert out.shape == ref.shape
    assert np.all(np.abs(out - ref) <= conv_bound(x, w, stride=(2, 2), pads=(1, 0, 1, 0)))


@pytest.mark.parametrize("M,K,N", [(64, 2048, 1000), (1, 7, 3), (130, 96, 257), (5, 513, 130)])
def test_matmul(M, K, N):
    rng = np.random.default_rng(7)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    ref = (x.astype(np.float64) @ w.astype(np.float64) + b).astype(np.float32)
    y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    xd, wd, bd = dev(x), dev(w), dev(b)
    L.check(L.lib().b200q_top_matmul_f32_dev(ptr(xd), ptr(wd), ptr(bd), ptr(y), M, K, N, 0, -1.0, None))
    torch.cuda.synchronize()
    bound = 1e-5 * (np.abs(x).astype(np.float64) @ np.abs(w).astype(np.float64)) + 1e-6
    assert np.all(np.abs(y.cpu().numpy() - ref) <= bound)


@pytest.mark.parametrize("case", [dict(k=(3, 3), s=(2, 2), p=(1, 1, 1, 1), is_max=True), dict(k=(7, 7), s=(7, 7), p=(0, 0, 0, 0), is_max=False),
                                  dict(k=(3, 2), s=(1, 2), p=(1, 0, 0, 1), is_max=False, cip=True),
                                  dict(k=(3, 3), s=(2, 2), p=(1, 1, 1, 1), is_max=False, cip=False, relu=True),
                                  dict(k=(2, 2), s=(2, 2), p=(0, 0, 0, 0), is_max=True, relu=True)])
def test_pool(case):
    rng = np.random.default_rng(9)
    x = rng.standard_normal((3, 5, 14, 14)).astype(np.float32)
    k, s, p = case["k"], case["s"], case["p"]
    ref = oracle.top_pool2d_f32(x, kernel=k, stride=s, pads=p, is_max=case["is_max"], count_include_pad=case.get("cip", False),
                                do_relu=case.get("relu", False), relu_limit=0.5 if case.get("relu") else -1.0)
    y = torch.full(ref.shape, float("nan"), dtype=torch.float32, device="cuda")
    xd = dev(x)
    L.check(L.lib().b200q_top_pool2d_f32_dev(ptr(xd), ptr(y), 15, 14, 14, k[0], k[1], s[0], s[1], p[0], p[1], p[2], p[3],
                                             int(case["is_max"]), int(case.get("cip", False)), int(case.get("relu", False)),
                                             0.5 if case.get("relu") else -1.0, None))
    torch.cuda.synchronize()
    got = y.cpu().numpy()
    if case["is_max"]:
        assert np.array_equal(got, ref)
    else:
        assert np.allclose(got, ref, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("n", [1, 3, 4, 1001, 1 << 20])
def test_add_and_relu(n):
    rng = np.random.default_rng(11)
    a, b = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    ad, bd = dev(a), dev(b)
    y = torch.empty(n, dtype=torch.float32, device="cuda")
    L.check(L.lib().b200q_top_add_f32_dev(ptr(ad), ptr(bd), ptr(y), n, 1, 1.5, None))
    assert np.array_equal(y.cpu().numpy(), np.clip(a + b, 0, 1.5))
    L.check(L.lib().b200q_top_add_f32_dev(ptr(ad), ptr(bd), ptr(y), n, 0, -1.0, None))
    assert np.array_equal(y.cpu().numpy(), a + b)
    L.check(L.lib().b200q_top_relu_f32_dev(ptr(ad), ptr(y), n, -1.0, None))
    assert np.array_equal(y.cpu().numpy(), np.maximum(a, 0))


def test_resnet50_forward_against_onednn():
    """Every activation of the fused fp32 graph against torch's CPU operators (oneDNN, the library behind the
    reference's Top dialect): relative to each tensor's rms."""
    ops = resnet50.build_fp32()
    x = np.random.default_rng(1).standard_normal((2, 3, 224, 224)).astype(np.float32)
    got = resnet50.Fp32Forward(ops, torch.device("cuda"))(torch.from_numpy(x).cuda())
    ref = resnet50.fp32_forward_torch(ops, torch.from_numpy(x))
    for op in ops:
        g, r = got[op["name"]].cpu().numpy().reshape(-1), ref[op["name"]].numpy().reshape(-1)
        assert g.shape == r.shape, op["name"]
        rms = float(np.sqrt(np.mean(r.astype(np.float64) ** 2))) + 1e-12
        assert float(np.abs(g - r).max()) <= 2e-4 * rms, (op["name"], float(np.abs(g - r).max()), rms)


def test_conv_split_k_is_deterministic_and_matches():
    """A layer with few output tiles and a long K (ResNet-50 layer4: 512 -> 512, 3x3 on 7x7) runs as several K splits
    whose partial sums are added in a fixed order: two runs give the same bits, and the values meet the bound."""
    rng = np.random.default_rng(13)
    n, ic, hw, oc = 8, 512, 7, 512
    x = rng.standard_normal((n, ic, hw, hw)).astype(np.float32)
    w = (rng.standard_normal((oc, ic, 3, 3)) / np.sqrt(ic * 9)).astype(np.float32)
    b = rng.standard_normal(oc).astype(np.float32)
    ref = oracle.top_conv2d_f32(x, w, b, pads=(1, 1, 1, 1), do_relu=True)
    d = L.TopConvDesc(n=n, ic=ic, ih=hw, iw=hw, oc=oc, kh=3, kw=3, sh=1, sw=1, dh=1, dw=1, pht=1, phb=1, pwl=1, pwr=1, groups=1,
                      with_bias=1, do_relu=1, relu_limit=-1.0)
    xd, wd, bd = dev(x), dev(w), dev(b)
    h = C.c_void_p()
    L.check(L.lib().b200q_top_conv2d_dev_create(C.byref(d), ptr(wd), ptr(bd), C.byref(h)))
    outs = []
    for _ in range(2):
        y = torch.full(ref.shape, float("nan"), dtype=torch.float32, device="cuda")
        L.check(L.lib().b200q_top_conv2d_dev_run(h, ptr(xd), ptr(y), n, None))
        torch.cuda.synchronize()
        outs.append(y.cpu().numpy())
    L.lib().b200q_top_conv2d_dev_destroy(C.byref(h))
    assert np.array_equal(outs[0], outs[1])
    assert np.all(np.abs(outs[0] - ref) <= conv_bound(x, w, pads=(1, 1, 1, 1)))


def test_empty_and_invalid_arguments():
    """Zero-sized work returns OK without launching; bad attributes and null pointers are reported, never computed."""
    lib = L.lib()
    y = torch.zeros(4, dtype=torch.float32, device="cuda")
    assert lib.b200q_top_add_f32_dev(ptr(y), ptr(y), ptr(y), 0, 0, -1.0, None) == L.OK
    assert lib.b200q_top_relu_f32_dev(ptr(y), ptr(y), 0, -1.0, None) == L.OK
    assert lib.b200q_top_eltwise_f32_dev(L.TOP_GELU, ptr(y), None, 0.0, ptr(y), 0, 0, -1.0, None) == L.OK
    assert lib.b200q_top_eltwise_f32_dev(99, ptr(y), None, 0.0, ptr(y), 4, 0, -1.0, None) == L.ERR_INVALID
    assert lib.b200q_top_eltwise_f32_dev(L.TOP_MUL, ptr(y), None, 0.0, ptr(y), 4, 0, -1.0, None) == L.ERR_INVALID   # no second operand
    assert lib.b200q_top_fake_quant_f32_dev(ptr(y), ptr(y), 4, 0.0, None) == L.ERR_INVALID                          # threshold must be positive
    assert lib.b200q_top_pool2d_f32_dev(ptr(y), ptr(y), 1, 2, 2, 3, 3, 1, 1, 0, 0, 0, 0, 1, 0, 0, -1.0, None) == L.ERR_INVALID  # empty output
    assert lib.b200q_top_matmul_f32_dev(ptr(y), ptr(y), None, ptr(y), 0, 2, 2, 0, -1.0, None) == L.OK
    d = L.TopConvDesc(n=1, ic=3, ih=4, iw=4, oc=4, kh=5, kw=5, sh=1, sw=1, dh=1, dw=1, pht=0, phb=0, pwl=0, pwr=0, groups=1,
                      with_bias=0, do_relu=0, relu_limit=-1.0)
    h = C.c_void_p()
    assert lib.b200q_top_conv2d_dev_create(C.byref(d), ptr(y), None, C.byref(h)) == L.ERR_INVALID                    # filter larger than the image
    d2 = L.TopConvDesc(n=1, ic=3, ih=4, iw=4, oc=4, kh=1, kw=1, sh=1, sw=1, dh=1, dw=1, pht=0, phb=0, pwl=0, pwr=0, groups=2,
                       with_bias=0, do_relu=0, relu_limit=-1.0)
    assert lib.b200q_top_conv2d_dev_create(C.byref(d2), ptr(y), None, C.byref(h)) == L.ERR_INVALID                   # channels do not divide into groups
    # a batch of zero images through a valid handle
    d3 = L.TopConvDesc(n=1, ic=2, ih=3, iw=3, oc=2, kh=1, kw=1, sh=1, sw=1, dh=1, dw=1, pht=0, phb=0, pwl=0, pwr=0, groups=1,
                       with_bias=0, do_relu=0, relu_limit=-1.0)
    w = torch.ones(4, dtype=torch.float32, device="cuda")
    L.check(lib.b200q_top_conv2d_dev_create(C.byref(d3), ptr(w), None, C.byref(h)))
    assert lib.b200q_top_conv2d_dev_run(h, ptr(y), ptr(y), 0, None) == L.OK
    lib.b200q_top_conv2d_dev_destroy(C.byref(h))
    assert h.value is None
