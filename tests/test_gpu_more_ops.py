"""Further ops of the py_cuda set in the executor: the Top dialect's elementwise float ops and Scale, and the data-movement
ops (Slice, Permute, Tile, Upsample, Pad, Concat, Squeeze, Unsqueeze) of both dialects, against numpy restatements of
the reference's inference loops (lib/Dialect/Top/Interfaces/<Op>.cpp)."""
import math

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from tpu_mlir_b200 import _lib as L  # noqa: E402
from tpu_mlir_b200.module import module  # noqa: E402
from op_restatements import active_table, d2s_ref, grid_sampler_ref, interp_ref  # noqa: E402


def run_graph(tensors, ops, weights, feeds, **kw):
    g = dict(inputs=list(feeds), outputs=[ops[-1]["name"]], tensors=tensors, ops=ops, state="TOP_F32")
    m = module(**kw)
    m.load(g, weights)
    for k, v in feeds.items():
        m.set_tensor(k, v)
    m.invoke(fixed_to_float=False)
    return m


def f32(shape):
    return {"shape": list(shape), "dtype": "f32"}


def test_top_elementwise_ops():
    rng = np.random.default_rng(0)
    x = (rng.standard_normal((2, 3, 5, 7)) * 3).astype(np.float32)
    y2 = (rng.standard_normal((2, 3, 5, 7)) + 2.5).astype(np.float32)
    sh = x.shape
    ops = [dict(type="top.AddConst", name="addc", inputs=["x"], attrs=dict(const_val=1.7, do_relu=True, relu_limit=3.0)),
           dict(type="top.SubConst", name="subc", inputs=["x"], attrs=dict(const_val=0.3)),
           dict(type="top.SubConst", name="rsubc", inputs=["x"], attrs=dict(const_val=0.3, is_reverse=True)),
           dict(type="top.MulConst", name="mulc", inputs=["x"], attrs=dict(const_val=0.1)),
           dict(type="top.MaxConst", name="maxc", inputs=["x"], attrs=dict(const_val=-0.5)),
           dict(type="top.MinConst", name="minc", inputs=["x"], attrs=dict(const_val=0.5)),
           dict(type="top.Mul", name="mul", inputs=["x", "y"], attrs=dict(do_relu=True)),
           dict(type="top.Sub", name="sub", inputs=["x", "y"], attrs={}),
           dict(type="top.Sub", name="rsub", inputs=["x", "y"], attrs=dict(is_reverse=True)),
           dict(type="top.Div", name="div", inputs=["x", "y"], attrs={}),
           dict(type="top.Sigmoid", name="sig", inputs=["x"], attrs={}),
           dict(type="top.Sigmoid", name="lsig", inputs=["x"], attrs=dict(log=True)),
           dict(type="top.SiLU", name="silu", inputs=["x"], attrs={}),
           dict(type="top.GELU", name="gelu", inputs=["x"], attrs={}),
           dict(type="top.Floor", name="floor", inputs=["x"], attrs={}),
           dict(type="top.Scale", name="scale", inputs=["x"], attrs=dict(do_relu=True))]
    tensors = {"x": f32(sh), "y": f32(sh)}
    tensors.update({o["name"]: f32(sh) for o in ops})
    sc, bi = rng.standard_normal(3).astype(np.float32), rng.standard_normal(3).astype(np.float32)
    m = run_graph(tensors, ops, {"scale_scale": sc, "scale_bias": bi}, {"x": x, "y": y2})
    g = m.get_tensor
    one = np.float32(1)
    assert np.array_equal(g("addc"), np.clip(x + np.float32(1.7), 0, 3))
    assert np.array_equal(g("subc"), x - np.float32(0.3))
    assert np.array_equal(g("rsubc"), np.float32(0.3) - x)
    assert np.array_equal(g("mulc"), (x.astype(np.float64) * 0.1).astype(np.float32))          # float * double, rounded once
    assert np.array_equal(g("maxc"), np.maximum(x, np.float32(-0.5)))
    assert np.array_equal(g("minc"), np.minimum(x, np.float32(0.5)))
    assert np.array_equal(g("mul"), np.maximum(x * y2, 0))
    assert np.array_equal(g("sub"), x - y2)
    assert np.array_equal(g("rsub"), y2 - x)
    assert np.array_equal(g("div"), x / y2)
    sig = one / (one + np.exp(-x))
    assert np.allclose(g("sig"), sig, rtol=3e-7, atol=1e-7)                                      # expf: a few ulps between libraries
    assert np.allclose(g("lsig"), np.log(sig), rtol=1e-5, atol=1e-6)
    assert np.allclose(g("silu"), x / (one + np.exp(-x)), rtol=3e-7, atol=1e-7)
    gelu = np.array([0.5 * float(v) * (1.0 + math.erf(float(v) / math.sqrt(2.0))) for v in x.ravel()]).astype(np.float32).reshape(sh)
    assert np.allclose(g("gelu"), gelu, rtol=1e-6, atol=1e-7)
    assert np.array_equal(g("floor"), np.floor(x))
    assert np.array_equal(g("scale"), np.maximum(x * sc.reshape(1, 3, 1, 1) + bi.reshape(1, 3, 1, 1), 0))


def movement_ops(dt):
    return [dict(type=f"{dt}.Slice", name="slice", inputs=["x"], attrs=dict(offset=[0, 1, 2, -5], steps=[1, 2, 1, 2])),
            dict(type=f"{dt}.Permute", name="perm", inputs=["x"], attrs=dict(order=[0, 2, 3, 1])),
            dict(type=f"{dt}.Tile", name="tile", inputs=["x"], attrs=dict(tile=[2, 1, 1, 3])),
            dict(type=f"{dt}.Upsample", name="up", inputs=["x"], attrs=dict(scale_h=2, scale_w=3)),
            dict(type=f"{dt}.Pad", name="pad", inputs=["x"], attrs=dict(paddings=[0, 1, 2, 0, 0, 0, 1, 3], val=-3.0, mode="constant")),
            dict(type=f"{dt}.Pad", name="crop", inputs=["x"], attrs=dict(paddings=[0, 0, -1, 1, 0, -1, 0, 0], val=0.0)),
            dict(type=f"{dt}.Concat", name="cat", inputs=["x", "perm2", "x"], attrs=dict(axis=1)),
            dict(type=f"{dt}.Unsqueeze", name="unsq", inputs=["x"], attrs=dict(axes=[1])),
            dict(type=f"{dt}.Squeeze", name="sq", inputs=["unsq"], attrs=dict(axes=[1]))]


def movement_expect(x, p2):
    return dict(slice=x[:, 1::2, 2:, 2::2], perm=np.transpose(x, (0, 2, 3, 1)), tile=np.tile(x, (2, 1, 1, 3)),
                up=np.repeat(np.repeat(x, 2, axis=2), 3, axis=3),
                pad=np.pad(x, ((0, 0), (1, 0), (2, 1), (0, 3)), constant_values=-3),
                crop=np.pad(x[:, :-1, 1:, :], ((0, 0), (0, 0), (0, 0), (1, 0)), constant_values=0),
                cat=np.concatenate([x, p2, x], axis=1), unsq=x[:, None], sq=x)


@pytest.mark.parametrize("dtype", ["f32", "i8"])
def test_data_movement_ops(dtype):
    rng = np.random.default_rng(1)
    sh = (2, 4, 6, 7)
    if dtype == "f32":
        x = rng.standard_normal(sh).astype(np.float32)
        p2 = rng.standard_normal((2, 3, 6, 7)).astype(np.float32)
        dt = "top"
    else:
        x = rng.integers(-128, 128, sh).astype(np.int8)
        p2 = rng.integers(-128, 128, (2, 3, 6, 7)).astype(np.int8)
        dt = "tpu"
    ops = movement_ops(dt)
    want = movement_expect(x, p2)
    ti = lambda shape: {"shape": list(shape), "dtype": dtype, "scale": 1.0, "zp": 0}  # noqa: E731
    tensors = {"x": ti(sh), "perm2": ti(p2.shape)}
    tensors.update({o["name"]: ti(want[o["name"]].shape) for o in ops})
    m = run_graph(tensors, ops, {}, {"x": x, "perm2": p2})
    for o in ops:
        got = m.get_raw_tensor(o["name"])
        assert got.shape == want[o["name"]].shape, o["name"]
        assert np.array_equal(got, want[o["name"]].astype(got.dtype)), o["name"]


def test_concat_relu_and_refusals():
    x = np.random.default_rng(2).standard_normal((1, 2, 3, 3)).astype(np.float32)
    ops = [dict(type="top.Concat", name="cat", inputs=["x", "x"], attrs=dict(axis=-3, do_relu=True, relu_limit=0.5))]
    m = run_graph({"x": f32(x.shape), "cat": f32((1, 4, 3, 3))}, ops, {}, {"x": x})
    assert np.array_equal(m.get_tensor("cat"), np.clip(np.concatenate([x, x], axis=1), 0, 0.5))
    with pytest.raises(L.B200QError):
        run_graph({"x": f32(x.shape), "p": f32((1, 2, 5, 5))}, [dict(type="top.Pad", name="p", inputs=["x"], attrs=dict(paddings=[0, 0, 1, 1, 0, 0, 1, 1], mode="symmetric"))],
                  {}, {"x": x})


def test_softmax_and_layernorm():
    rng = np.random.default_rng(3)
    x = (rng.standard_normal((3, 10, 4, 5)) * 2).astype(np.float32)
    w, b = rng.standard_normal(20).astype(np.float32), rng.standard_normal(20).astype(np.float32)
    ops = [dict(type="top.Softmax", name="sm1", inputs=["x"], attrs=dict(axis=1)),
           dict(type="top.Softmax", name="sm3", inputs=["x"], attrs=dict(axis=-1, log=True)),
           dict(type="top.LayerNorm", name="ln", inputs=["x"], attrs=dict(axis=2, eps=1e-5)),
           dict(type="top.LayerNorm", name="ln0", inputs=["x"], attrs=dict(axis=-1, eps=1e-3))]
    tensors = {"x": f32(x.shape)}
    tensors.update({o["name"]: f32(x.shape) for o in ops})
    m = run_graph(tensors, ops, {"ln_weight": w, "ln_bias": b}, {"x": x})
    x64 = x.astype(np.float64)
    e = np.exp(x64 - x64.max(axis=1, keepdims=True))
    assert np.allclose(m.get_tensor("sm1"), e / e.sum(axis=1, keepdims=True), rtol=1e-5, atol=1e-7)
    d = x64 - x64.max(axis=-1, keepdims=True)
    assert np.allclose(m.get_tensor("sm3"), d - np.log(np.exp(d).sum(axis=-1, keepdims=True)), rtol=1e-5, atol=1e-5)
    r = x64.reshape(30, 20)
    ln = (r - r.mean(axis=1, keepdims=True)) / np.sqrt(r.var(axis=1, keepdims=True) + 1e-5) * w + b
    assert np.allclose(m.get_tensor("ln"), ln.reshape(x.shape), rtol=1e-4, atol=1e-5)
    r = x64.reshape(120, 5)
    ln0 = (r - r.mean(axis=1, keepdims=True)) / np.sqrt(r.var(axis=1, keepdims=True) + 1e-3)
    assert np.allclose(m.get_tensor("ln0"), ln0.reshape(x.shape), rtol=1e-4, atol=1e-5)


def test_tpu_addconst_and_mulconst_int8():
    """tpu.AddConst (AddConst.cpp:26-47) and the symmetric tpu.MulConst (MulConst.cpp:50-62) on int8 / uint8 tensors."""
    rng = np.random.default_rng(4)
    x = rng.integers(-128, 128, (3, 5, 7)).astype(np.int8)
    ops = [dict(type="tpu.AddConst", name="ac", inputs=["x"], attrs=dict(multiplier=77, rshift=6, const_val=-300.0, do_relu=False)),
           dict(type="tpu.AddConst", name="acr", inputs=["x"], attrs=dict(multiplier=5, rshift=0, const_val=17.0, do_relu=True)),
           dict(type="tpu.MulConst", name="mc", inputs=["x"], attrs=dict(multiplier=-93, rshift=7, do_relu=True))]
    tensors = {"x": {"shape": list(x.shape), "dtype": "i8", "scale": 1.0, "zp": 0}, "ac": {"shape": list(x.shape), "dtype": "i8", "scale": 1.0, "zp": 0},
               "acr": {"shape": list(x.shape), "dtype": "u8", "scale": 1.0, "zp": 0}, "mc": {"shape": list(x.shape), "dtype": "u8", "scale": 1.0, "zp": 0}}
    m = run_graph(tensors, ops, {}, {"x": x})

    def rsr(v, s):
        return (v + (1 << (s - 1))) >> s if s > 0 else v

    xi = x.astype(np.int64)
    ac = np.clip(np.vectorize(lambda v: rsr(int(v) * 77 - 300, 6))(xi), -128, 127)
    acr = np.clip(np.maximum(np.vectorize(lambda v: rsr(int(v) * 5 + 17, 0))(xi), 0), 0, 255)
    mc = np.clip(np.maximum(np.vectorize(lambda v: rsr(int(v) * -93, 7))(xi), 0), 0, 255)
    assert np.array_equal(m.get_raw_tensor("ac").astype(np.int64), ac)
    assert np.array_equal(m.get_raw_tensor("acr").astype(np.int64), acr)
    assert np.array_equal(m.get_raw_tensor("mc").astype(np.int64), mc)


def test_reduce_and_tpu_relu():
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((2, 3, 4, 5)) + 0.5).astype(np.float32)
    cases = [("ReduceMean", [2, 3]), ("ReduceSum", [1]), ("ReduceMax", [-1]), ("ReduceMin", [0, 1]), ("ReduceProd", [2]), ("ReduceL2", [3]), ("ReduceL1", [1, 2])]
    ops, tensors = [], {"x": f32(x.shape)}
    for i, (mode, axes) in enumerate(cases):
        ax = [v % 4 for v in axes]
        shape = [1 if d in ax else x.shape[d] for d in range(4)]
        ops.append(dict(type="top.Reduce", name=f"r{i}", inputs=["x"], attrs=dict(mode=mode, axes=axes, keepdims=True)))
        tensors[f"r{i}"] = f32(shape)
    m = run_graph(tensors, ops, {}, {"x": x})
    fns = dict(ReduceMean=np.mean, ReduceSum=np.sum, ReduceMax=np.max, ReduceMin=np.min, ReduceProd=np.prod,
               ReduceL2=lambda v, axis, keepdims: np.sqrt(np.sum(v * v, axis=axis, keepdims=keepdims)),
               ReduceL1=lambda v, axis, keepdims: np.sum(np.abs(v), axis=axis, keepdims=keepdims))
    for i, (mode, axes) in enumerate(cases):
        want = fns[mode](x.astype(np.float64), axis=tuple(v % 4 for v in axes), keepdims=True)
        assert np.allclose(m.get_tensor(f"r{i}"), want, rtol=2e-6, atol=1e-6), mode
    xi = rng.integers(-128, 128, (4, 9)).astype(np.int8)
    t = {"x": {"shape": [4, 9], "dtype": "i8", "scale": 1.0, "zp": 0}, "r": {"shape": [4, 9], "dtype": "i8", "scale": 1.0, "zp": 0}}
    m2 = run_graph(t, [dict(type="tpu.Relu", name="r", inputs=["x"], attrs={})], {}, {"x": xi})
    assert np.array_equal(m2.get_raw_tensor("r"), np.maximum(xi, 0))


@pytest.mark.parametrize("cfg", [dict(crd=False, inv=False, in_nchw=True, out_nchw=True, swap=False), dict(crd=True, inv=False, in_nchw=True, out_nchw=True, swap=True),
                                 dict(crd=False, inv=True, in_nchw=True, out_nchw=True, swap=False), dict(crd=True, inv=False, in_nchw=False, out_nchw=True, swap=False),
                                 dict(crd=False, inv=True, in_nchw=True, out_nchw=False, swap=True)])
def test_depth2space(cfg):
    rng = np.random.default_rng(6)
    bh, bw, c, h, w = 2, 3, 4, 3, 2
    deep_nchw, shallow_nchw = (2, c * bh * bw, h, w), (2, c, h * bh, w * bw)
    to_layout = lambda shp, f: shp if f else (shp[0], shp[2], shp[3], shp[1])  # noqa: E731
    if cfg["inv"]:
        in_shape, out_shape = to_layout(shallow_nchw, cfg["in_nchw"]), to_layout(deep_nchw, cfg["out_nchw"])
    else:
        in_shape, out_shape = to_layout(deep_nchw, cfg["in_nchw"]), to_layout(shallow_nchw, cfg["out_nchw"])
    x = rng.standard_normal(in_shape).astype(np.float32)
    want = d2s_ref(x, out_shape, bh, bw, cfg["crd"], cfg["inv"], cfg["in_nchw"], cfg["out_nchw"], cfg["swap"])
    ops = [dict(type="top.Depth2Space", name="d", inputs=["x"], attrs=dict(block_h=bh, block_w=bw, is_CRD=cfg["crd"], is_inversed=cfg["inv"],
                                                                         in_is_NCHW=cfg["in_nchw"], out_is_NCHW=cfg["out_nchw"], swap_cr=cfg["swap"]))]
    m = run_graph({"x": f32(in_shape), "d": f32(out_shape)}, ops, {}, {"x": x})
    assert np.array_equal(m.get_tensor("d"), want)


def test_tpu_active_modes():
    """tpu::ActiveOp on f32 tensors against the function table of lib/Support/ActiveUtils.cpp:16-181 evaluated in Python doubles
    (one float ulp of slack, plus a few double ulps of the input's size where 1 + erf or 1 + tanh cancels: the device's double
    functions and the C library's may differ in their last bit)."""
    rng = np.random.default_rng(8)
    x = np.concatenate([(rng.standard_normal(4000) * 2).astype(np.float32), np.float32([0, -0.0, 1, -1, 25, -25, 0.5])]).reshape(1, -1)
    pos = np.abs(x) + np.float32(0.01)
    unit = np.clip(x / 4, -0.99, 0.99).astype(np.float32)
    table = {mode: ({'x': x, 'pos': pos, 'unit': unit}[dom], fn, coeffs) for mode, (dom, fn, coeffs) in active_table().items()}
    for mode, (inp, fn, coeffs) in table.items():
        ops = [dict(type="tpu.Active", name="y", inputs=["x"], attrs=dict(mode=mode, coeffs=coeffs))]
        m = run_graph({"x": f32(inp.shape), "y": f32(inp.shape)}, ops, {}, {"x": inp})
        want = np.array([fn(float(v)) for v in inp.ravel()], dtype=np.float64).astype(np.float32).reshape(inp.shape)
        got = m.get_tensor("y")
        exact = mode in ("SQUARE", "ABSVAL", "ROUND", "CEIL", "FLOOR", "SIGN", "HSWISH", "HSIGMOID", "SOFT_SIGN", "SQRT")
        if exact:
            assert np.array_equal(got, want), mode
        else:
            assert np.all(np.abs(got.astype(np.float64) - want) <= np.spacing(np.abs(want)).astype(np.float64) + 1e-14 * (1 + np.abs(inp))), mode
    # MISH works in float in the reference (GenericCpuFunc.cpp:25-33): a float restatement, a few ulps for exp/log
    f = np.float32
    sp = np.log(np.exp(x) + f(1))
    want = x * (f(2) / (f(1) + np.exp(f(-2) * sp)) - f(1))
    m = run_graph({"x": f32(x.shape), "y": f32(x.shape)}, [dict(type="tpu.Active", name="y", inputs=["x"], attrs=dict(mode="MISH"))], {}, {"x": x})
    np.testing.assert_allclose(m.get_tensor("y"), want, rtol=2e-6, atol=1e-6)
    with pytest.raises(L.B200QError):
        run_graph({"x": f32(x.shape), "y": f32(x.shape)}, [dict(type="tpu.Active", name="y", inputs=["x"], attrs=dict(mode="ARCSIN"))], {}, {"x": x})


def test_tpu_float_mode_ops_follow_top():
    """F32-mode Tpu ops that share the Top op's arithmetic, and tpu.Reduce's mean (sum * float(1 / n), Reduce.cpp:132-138)."""
    rng = np.random.default_rng(9)
    x = (rng.standard_normal((2, 7, 5)) * 3).astype(np.float32)
    y2 = (rng.standard_normal((2, 7, 5)) + 2.5).astype(np.float32)
    sh = x.shape
    ops = [dict(type="tpu.Sub", name="sub", inputs=["x", "y"], attrs=dict(is_reverse=True, do_relu=True)),
           dict(type="tpu.Div", name="div", inputs=["x", "y"], attrs={}),
           dict(type="tpu.MaxConst", name="maxc", inputs=["x"], attrs=dict(const_val=-0.5)),
           dict(type="tpu.MinConst", name="minc", inputs=["x"], attrs=dict(const_val=0.5)),
           dict(type="tpu.SubConst", name="subc", inputs=["x"], attrs=dict(const_val=0.3, is_reverse=True)),
           dict(type="tpu.Softmax", name="sm", inputs=["x"], attrs=dict(axis=1)),
           dict(type="tpu.LayerNorm", name="ln", inputs=["x"], attrs=dict(axis=2, eps=1e-5, normalized_shape=[5])),
           dict(type="tpu.Reduce", name="mean", inputs=["x"], attrs=dict(axes=[1], keepdims=False, mode="ReduceMean")),
           dict(type="top.Reduce", name="tmean", inputs=["x"], attrs=dict(axes=[1], keepdims=False, mode="ReduceMean"))]
    tensors = {"x": f32(sh), "y": f32(sh), "mean": f32((2, 5)), "tmean": f32((2, 5))}
    tensors.update({o["name"]: f32(sh) for o in ops if o["name"] not in tensors})
    lw, lb = rng.standard_normal(5).astype(np.float32), rng.standard_normal(5).astype(np.float32)
    m = run_graph(tensors, ops, {"ln_weight": lw, "ln_bias": lb}, {"x": x, "y": y2})
    g = m.get_tensor
    assert np.array_equal(g("sub"), np.maximum(y2 - x, 0))
    assert np.array_equal(g("div"), x / y2)
    assert np.array_equal(g("maxc"), np.maximum(x, np.float32(-0.5)))
    assert np.array_equal(g("minc"), np.minimum(x, np.float32(0.5)))
    assert np.array_equal(g("subc"), np.float32(0.3) - x)
    e = np.exp(x - x.max(axis=1, keepdims=True))
    np.testing.assert_allclose(g("sm"), e / e.sum(axis=1, keepdims=True), rtol=1e-6)
    mu = x.mean(axis=2, keepdims=True)
    np.testing.assert_allclose(g("ln"), (x - mu) / np.sqrt(((x - mu) ** 2).mean(axis=2, keepdims=True) + 1e-5) * lw + lb, rtol=1e-4, atol=1e-5)
    s = np.zeros((2, 5), np.float32)
    for a_ in range(7):
        s = s + x[:, a_, :]
    assert np.array_equal(g("mean"), s * np.float32(1.0 / 7))
    assert np.array_equal(g("tmean"), s / np.float32(7))


def test_gather_and_gather_elements():
    rng = np.random.default_rng(10)
    x = rng.standard_normal((3, 6, 4)).astype(np.float32)
    idx = np.float32([[5, 0, -1], [2, 2, -6]])                      # float-stored indices, negatives count from the end
    ops = [dict(type="top.Gather", name="g", inputs=["x", "i"], attrs=dict(axis=1))]
    m = run_graph({"x": f32(x.shape), "i": f32(idx.shape), "g": f32((3, 2, 3, 4))}, ops, {}, {"x": x, "i": idx})
    assert np.array_equal(m.get_tensor("g"), np.take(x, idx.astype(np.int64), axis=1))
    # indices as a weight, int32; an int8 tensor through the Tpu op
    q = rng.integers(-128, 128, (5, 7), dtype=np.int8)
    ops = [dict(type="tpu.Gather", name="g", inputs=["x"], attrs=dict(axis=0))]
    m = run_graph({"x": dict(shape=[5, 7], dtype="i8", scale=0.1, zp=0), "g": dict(shape=[3, 7], dtype="i8", scale=0.1, zp=0)}, ops,
                  {"g_indices": np.int32([4, -5, 2])}, {"x": q})
    assert np.array_equal(m.get_raw_tensor("g"), q[[4, 0, 2]])
    # GatherElements: indices smaller than the source off the axis
    src = rng.standard_normal((4, 5, 6)).astype(np.float32)
    ind = rng.integers(0, 5, (3, 2, 6)).astype(np.float32)
    ops = [dict(type="top.GatherElements", name="ge", inputs=["x", "i"], attrs=dict(axis=1))]
    m = run_graph({"x": f32(src.shape), "i": f32(ind.shape), "ge": f32(ind.shape)}, ops, {}, {"x": src, "i": ind})
    want = np.zeros(ind.shape, np.float32)
    for a_ in range(3):
        for b_ in range(2):
            for c_ in range(6):
                want[a_, b_, c_] = src[a_, int(ind[a_, b_, c_]), c_]
    assert np.array_equal(m.get_tensor("ge"), want)
    ops = [dict(type="tpu.GatherElements", name="ge", inputs=["x", "i"], attrs=dict(axis=-1))]
    ind2 = rng.integers(0, 6, (4, 5, 2)).astype(np.int32)
    m = run_graph({"x": f32(src.shape), "i": dict(shape=list(ind2.shape), dtype="i32"), "ge": f32(ind2.shape)}, ops, {}, {"x": src, "i": ind2})
    assert np.array_equal(m.get_tensor("ge"), np.take_along_axis(src, ind2.astype(np.int64), axis=2))


def test_swap_dim_inner():
    rng = np.random.default_rng(11)
    x = rng.standard_normal((2, 5, 6, 7)).astype(np.float32)
    for offs in ([0, 0, 2, 0], [0, 3, 0, 4], [0, 0, 0, 7]):
        ops = [dict(type="top.SwapDimInner", name="s", inputs=["x"], attrs=dict(offset=offs))]
        m = run_graph({"x": f32(x.shape), "s": f32(x.shape)}, ops, {}, {"x": x})
        want = x
        for ax, o in enumerate(offs):
            if o:
                want = np.roll(want, -o, axis=ax)      # out[b] = in[(b + offset) % dim]
        assert np.array_equal(m.get_tensor("s"), want), offs


def test_tpu_prelu():
    rng = np.random.default_rng(12)
    x = rng.standard_normal((2, 3, 4, 5)).astype(np.float32)
    sl = np.float32([0.1, -0.25, 0.5]).reshape(1, 3, 1, 1)
    ops = [dict(type="tpu.PRelu", name="p", inputs=["x"], attrs={})]
    m = run_graph({"x": f32(x.shape), "p": f32(x.shape)}, ops, {"p_slope": sl}, {"x": x})
    assert np.array_equal(m.get_tensor("p"), np.where(x > 0, x, x * sl))
    q = rng.integers(-128, 128, (2, 3, 4, 5), dtype=np.int8)
    qs = np.int8([13, -7, 100]).reshape(1, 3, 1, 1)
    qi = dict(shape=list(q.shape), dtype="i8", scale=0.05, zp=0)
    m = run_graph({"x": qi, "p": dict(qi)}, [dict(type="tpu.PRelu", name="p", inputs=["x"], attrs=dict(rshift=5))], {"p_slope": qs}, {"x": q})
    prod = q.astype(np.int64) * qs
    neg = np.clip((prod + 16) >> 5, -128, 127)                                    # round half up
    assert np.array_equal(m.get_raw_tensor("p"), np.where(q < 0, neg, q).astype(np.int8))


def _rsr(v, s, half_away):
    """RightShiftRound on Python integers: half up, or half away from zero."""
    if s <= 0:
        return v << (-s)
    val, mant, half = v >> s, v & ((1 << s) - 1), 1 << (s - 1)
    if half_away:
        return val + (1 if (mant >= half if v >= 0 else mant > half) else 0)
    return val + (1 if mant >= half else 0)


def test_tpu_requant_fp_and_int_axis():
    rng = np.random.default_rng(13)
    acc = rng.integers(-60000, 60000, (2, 4, 3, 5), dtype=np.int32)
    acc.ravel()[:4] = [250, -250, 750, -750]                          # ties at scale 0.002 * ... below
    i32 = dict(shape=list(acc.shape), dtype="i32")
    # RequantFp, MultiplierShift: to_int(float(x) * scale + offset), half away from zero
    sc, of = 0.002, 0.5
    out = dict(shape=list(acc.shape), dtype="i8", scale=1.0, zp=0)
    m = run_graph({"x": i32, "y": out}, [dict(type="tpu.RequantFp", name="y", inputs=["x"], attrs=dict(scale=sc, offset=of, quant_mode="MultiplierShift"))],
                  {}, {"x": acc})
    f = acc.astype(np.float32) * np.float32(sc) + np.float32(of)
    want = np.clip(np.sign(f) * np.floor(np.abs(f) + np.float32(0.5)), -128, 127).astype(np.int8)
    assert np.array_equal(m.get_raw_tensor("y"), want)
    # RequantFp, TFLite: to_int(x * scale) + zp, half to even, uint8 output
    out = dict(shape=list(acc.shape), dtype="u8", scale=1.0, zp=7)
    m = run_graph({"x": i32, "y": out}, [dict(type="tpu.RequantFp", name="y", inputs=["x"], attrs=dict(scale=sc, quant_mode="TFLite", round_mode="HalfToEven"))],
                  {}, {"x": acc})
    want = np.clip(np.rint(acc.astype(np.float32) * np.float32(sc)).astype(np.int64) + 7, 0, 255).astype(np.uint8)
    assert np.array_equal(m.get_raw_tensor("y"), want)
    # RequantIntAxis, MultiplierShift per channel: zp + RSR(x * m, -shift), half away from zero by default
    table = np.int32([[3, -9, 2], [17, -12, -3], [1, -5, 0], [-5, -10, 1]])
    out = dict(shape=list(acc.shape), dtype="i8", scale=1.0, zp=0)
    m = run_graph({"x": i32, "y": out}, [dict(type="tpu.RequantIntAxis", name="y", inputs=["x"], attrs=dict(quant_mode="MultiplierShift"))],
                  {"y_quant": table}, {"x": acc})
    want = np.zeros(acc.shape, np.int8)
    for idx in np.ndindex(*acc.shape):
        mu, sh, zp = (int(v) for v in table[idx[1]])
        want[idx] = max(-128, min(127, zp + _rsr(int(acc[idx]) * mu, -sh, True)))
    assert np.array_equal(m.get_raw_tensor("y"), want)
    # fused along the last dimension, half up, shift as it stands
    table = np.int32([[3, 9, 2], [17, 12, -3], [1, 5, 0], [-5, 10, 1], [7, 11, 4]])
    m = run_graph({"x": i32, "y": out}, [dict(type="tpu.RequantIntAxis", name="y", inputs=["x"],
                                              attrs=dict(quant_mode="MultiplierShift", fuse_rq_axis=True, round_mode="HalfUp"))],
                  {"y_quant": table}, {"x": acc})
    for idx in np.ndindex(*acc.shape):
        mu, sh, zp = (int(v) for v in table[idx[3]])
        want[idx] = max(-128, min(127, zp + _rsr(int(acc[idx]) * mu, sh, False)))
    assert np.array_equal(m.get_raw_tensor("y"), want)
    # TFLite: zp + MultiplyByQuantizedMultiplier(x, m, shift): RSR(x * m, 31, half up), then RSR by -shift (half away from zero)
    table = np.int32([[1518500250, -7, 3], [1073741824, -9, -2], [2000000000, -6, 0], [1300000000, -8, 5]])
    m = run_graph({"x": i32, "y": out}, [dict(type="tpu.RequantIntAxis", name="y", inputs=["x"], attrs=dict(quant_mode="TFLite"))],
                  {"y_quant": table}, {"x": acc})
    for idx in np.ndindex(*acc.shape):
        mu, sh, zp = (int(v) for v in table[idx[1]])
        want[idx] = max(-128, min(127, zp + _rsr(_rsr(int(acc[idx]) * mu, 31, False), -sh, True)))
    assert np.array_equal(m.get_raw_tensor("y"), want)


def test_arg_and_top_cast():
    rng = np.random.default_rng(14)
    x = rng.integers(-3, 4, (3, 9, 5)).astype(np.float32)             # many ties
    for mode, last in (("ArgMax", True), ("ArgMax", False), ("ArgMin", True), ("ArgMin", False)):
        ops = [dict(type="top.Arg", name="idx", values="val", inputs=["x"], attrs=dict(axis=1, keepdims=True, mode=mode, select_last_index=last))]
        m = run_graph({"x": f32(x.shape), "idx": f32((3, 1, 5)), "val": f32((3, 1, 5))}, ops, {}, {"x": x})
        ext = x.max(axis=1) if mode == "ArgMax" else x.min(axis=1)
        hit = x == ext[:, None, :]
        first = hit.argmax(axis=1)
        want = (x.shape[1] - 1 - hit[:, ::-1, :].argmax(axis=1)) if last else first
        assert np.array_equal(m.get_tensor("idx").reshape(3, 5), want.astype(np.float32)), (mode, last)
        assert np.array_equal(m.get_tensor("val").reshape(3, 5), ext)
    ops = [dict(type="tpu.Arg", name="idx", inputs=["x"], attrs=dict(axis=-1, keepdims=False, mode="ArgMin", select_last_index=False))]
    m = run_graph({"x": f32(x.shape), "idx": dict(shape=[3, 9], dtype="i32")}, ops, {}, {"x": x})
    assert np.array_equal(m.get_raw_tensor("idx"), x.argmin(axis=2).astype(np.int32))
    v = np.float32([-300.5, -128.5, -2.5, -1.5, -0.5, 0.5, 1.5, 2.5, 126.5, 127.5, 255.5, 300.2, 40000.7, -40000.7]).reshape(1, -1)
    away = np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))
    cases = [("INT8", "HalfAwayFromZero", np.clip(away, -128, 127)), ("UINT8", "HalfToEven", np.clip(np.rint(v), 0, 255)),
             ("INT16", "Down", np.clip(np.floor(v), -32768, 32767)), ("UINT16", "Up", np.clip(np.ceil(v), 0, 65535)),
             ("INT32", "TowardsZero", np.trunc(v)), ("F32", "HalfAwayFromZero", v)]
    for to, rm, want in cases:
        ops = [dict(type="top.Cast", name="y", inputs=["x"], attrs=dict(to=to, round_mode=rm))]
        m = run_graph({"x": f32(v.shape), "y": f32(v.shape)}, ops, {}, {"x": v})
        assert np.array_equal(m.get_tensor("y"), want.astype(np.float32)), to
    m = run_graph({"x": f32(v.shape), "y": dict(shape=list(v.shape), dtype="i8", scale=1.0, zp=0)},
                  [dict(type="top.Cast", name="y", inputs=["x"], attrs=dict(to="INT8"))], {}, {"x": v})
    assert np.array_equal(m.get_raw_tensor("y"), np.clip(away, -128, 127).astype(np.int8))


@pytest.mark.parametrize("mode,padding,align", [(0, 0, False), (0, 1, True), (0, 2, False), (0, 2, True), (1, 0, True), (1, 2, False)])
def test_grid_sampler(mode, padding, align):
    rng = np.random.default_rng(15)
    x = rng.standard_normal((2, 3, 5, 7)).astype(np.float32)
    grid = (rng.random((2, 4, 6, 2)) * 3 - 1.5).astype(np.float32)          # some samples fall outside [-1, 1]
    grid[0, 0, 0] = [-1, 1]
    grid[0, 0, 1] = [0, 0]
    ops = [dict(type="top.GridSampler", name="y", inputs=["x", "g"], attrs=dict(mode=mode, padding_mode=padding, align_corners=align))]
    m = run_graph({"x": f32(x.shape), "g": f32(grid.shape), "y": f32((2, 3, 4, 6))}, ops, {}, {"x": x, "g": grid})
    assert np.array_equal(m.get_tensor("y"), grid_sampler_ref(x, grid, mode, padding, align))


@pytest.mark.parametrize("mode,coord,platform,osz", [("linear", "half_pixel", "ONNX", (9, 11)), ("linear", "align_corners", "ONNX", (9, 11)),
                                                     ("linear", "asymmetric", "TORCH", (3, 4)), ("linear", "pytorch_half_pixel", "CAFFE", (10, 14)),
                                                     ("nearest", "asymmetric", "ONNX", (10, 14)), ("nearest", "half_pixel", "ONNX", (9, 11)),
                                                     ("nearest", "half_pixel", "TORCH", (7, 5)), ("nearest", "align_corners", "TFLITE", (8, 13)),
                                                     ("nearest", "half_pixel", "CAFFE", (1, 1))])
def test_interp(mode, coord, platform, osz):
    rng = np.random.default_rng(16)
    x = rng.standard_normal((2, 3, 5, 7)).astype(np.float32)
    for tname in ("top.Interp", "tpu.Interp"):
        ops = [dict(type=tname, name="y", inputs=["x"], attrs=dict(mode=mode, coord_mode=coord, platform=platform, scale_h=osz[0] / 5, scale_w=osz[1] / 7))]
        m = run_graph({"x": f32(x.shape), "y": f32((2, 3) + osz)}, ops, {}, {"x": x})
        assert np.array_equal(m.get_tensor("y"), interp_ref(x, osz[0], osz[1], mode, coord, platform)), tname


def deconv_ref(x, w, b, izp, strides, dil, pads, opad, mult, rshift, ozp, relu, groups=1):
    """tpu.Deconv as the reference computes it (Deconv.cpp:95-150): without an input zero point the scatter form of a transposed
    convolution; with one, the spread input padded with the zero point and correlated with the rotated filter
    (lib/Support/Dnnl/Deconv.cpp:17-110, MathUtils.cpp:673-705).  Then RSR(acc * m, s, half up) + zp, saturated to int8."""
    n, ic, ih, iw = x.shape
    oc, icg, kh, kw = w.shape
    sh, sw = strides
    dh, dw = dil
    pt, pl, pb, pr = pads
    oh = (ih - 1) * sh + 1 + dh * (kh - 1) - pt - pb + opad[0]
    ow = (iw - 1) * sw + 1 + dw * (kw - 1) - pl - pr + opad[1]
    acc = np.zeros((n, oc, oh, ow), np.int64)
    ocg = oc // groups
    if izp == 0:
        full = np.zeros((n, oc, (ih - 1) * sh + dh * (kh - 1) + 1 + opad[0] + pt + pb, (iw - 1) * sw + dw * (kw - 1) + 1 + opad[1] + pl + pr), np.int64)
        for o in range(oc):
            g = o // ocg
            for c in range(icg):
                for i in range(kh):
                    for j in range(kw):
                        full[:, o, i * dh:i * dh + (ih - 1) * sh + 1:sh, j * dw:j * dw + (iw - 1) * sw + 1:sw] += \
                            x[:, g * icg + c].astype(np.int64) * int(w[o, c, i, j])
        acc = full[:, :, pt:pt + oh, pl:pl + ow].copy()
    else:
        hs, ws = oh + kh - 1, ow + kw - 1
        st = np.full((n, ic, hs, ws), izp, np.int64)
        st[:, :, kh - 1 - pt:kh - 1 - pt + (ih - 1) * sh + 1:sh, kw - 1 - pl:kw - 1 - pl + (iw - 1) * sw + 1:sw] = x
        wr = w[:, :, ::-1, ::-1].astype(np.int64)
        for o in range(oc):
            g = o // ocg
            for i in range(kh):
                for j in range(kw):
                    acc[:, o] += (st[:, g * icg:(g + 1) * icg, i:i + oh, j:j + ow] * wr[o, :, i, j][None, :, None, None]).sum(axis=1)
    if b is not None:
        acc += b.astype(np.int64)[None, :, None, None]
    if relu:
        acc = np.maximum(acc, 0)
    m_ = np.asarray(mult, np.int64).reshape(1, -1, 1, 1)
    s_ = np.asarray(rshift, np.int64).reshape(1, -1, 1, 1)
    v = ((acc * m_ + (1 << (s_ - 1))) >> s_) + ozp
    return np.clip(v, -128, 127).astype(np.int8)


@pytest.mark.parametrize("cfg", [dict(ic=16, oc=32, k=(2, 2), s=(2, 2), pads=(0, 0, 0, 0)), dict(ic=8, oc=16, k=(3, 3), s=(2, 2), pads=(1, 1, 1, 1), opad=(1, 1), relu=True),
                                 dict(ic=16, oc=16, k=(4, 4), s=(2, 2), pads=(1, 1, 1, 1), izp=-5, ozp=3), dict(ic=8, oc=8, k=(3, 2), s=(1, 3), pads=(0, 1, 2, 0), dil=(2, 1)),
                                 dict(ic=8, oc=12, k=(3, 3), s=(2, 1), pads=(1, 0, 0, 1), groups=4, izp=7)])
def test_tpu_deconv(cfg):
    rng = np.random.default_rng(17)
    ic, oc, (kh, kw), groups = cfg["ic"], cfg["oc"], cfg["k"], cfg.get("groups", 1)
    strides, dil, pads, opad = cfg["s"], cfg.get("dil", (1, 1)), cfg["pads"], cfg.get("opad", (0, 0))
    izp, ozp, relu = cfg.get("izp", 0), cfg.get("ozp", 0), cfg.get("relu", False)
    x = rng.integers(-128, 128, (2, ic, 5, 6), dtype=np.int8)
    w = rng.integers(-128, 128, (oc, ic // groups, kh, kw), dtype=np.int8)
    b = rng.integers(-5000, 5000, oc, dtype=np.int32)
    mult = rng.integers(1000, 20000, oc).tolist()
    rshift = rng.integers(18, 22, oc).tolist()
    want = deconv_ref(x, w, b, izp, strides, dil, pads, opad, mult, rshift, ozp, relu, groups)
    ops = [dict(type="tpu.Deconv", name="y", inputs=["x"], attrs=dict(kernel_shape=[kh, kw], strides=list(strides), dilations=list(dil), pads=list(pads),
                                                                     output_padding=list(opad), group=groups, do_relu=relu, multiplier=mult, rshift=rshift,
                                                                     quant_mode="MultiplierShift"))]
    tensors = {"x": dict(shape=list(x.shape), dtype="i8", scale=0.1, zp=izp), "y": dict(shape=list(want.shape), dtype="i8", scale=0.1, zp=ozp)}
    m = run_graph(tensors, ops, {"y_filter": w, "y_bias": b}, {"x": x})
    m.check_status()
    assert np.array_equal(m.get_raw_tensor("y"), want)


def test_binary_ops_broadcast():
    """Operands of different shapes (numpy broadcasting): per-channel and scalar second operands, a broadcast first operand."""
    rng = np.random.default_rng(18)
    x = rng.standard_normal((2, 3, 4, 5)).astype(np.float32)
    c = (rng.standard_normal((1, 3, 1, 1)) + 2).astype(np.float32)
    row = rng.standard_normal((5,)).astype(np.float32)
    ops = [dict(type="top.Add", name="add", inputs=["x", "c"], attrs=dict(do_relu=True)),
           dict(type="top.Mul", name="mul", inputs=["x", "row"], attrs={}),
           dict(type="top.Sub", name="sub", inputs=["c", "x"], attrs={}),
           dict(type="top.Div", name="div", inputs=["x", "c"], attrs={}),
           dict(type="tpu.Sub", name="tsub", inputs=["x", "c"], attrs=dict(is_reverse=True))]
    tensors = {"x": f32(x.shape), "c": f32(c.shape), "row": f32(row.shape)}
    tensors.update({o["name"]: f32(x.shape) for o in ops})
    m = run_graph(tensors, ops, {}, {"x": x, "c": c, "row": row})
    g = m.get_tensor
    assert np.array_equal(g("add"), np.maximum(x + c, 0))
    assert np.array_equal(g("mul"), x * row)
    assert np.array_equal(g("sub"), c - x)
    assert np.array_equal(g("div"), x / c)
    assert np.array_equal(g("tsub"), c - x)
    # 8-bit: tpu.Mul and tpu.Add with a per-channel operand
    q = rng.integers(-128, 128, (2, 3, 4, 5), dtype=np.int8)
    qc = rng.integers(-128, 128, (1, 3, 1, 1), dtype=np.int8)
    qi = lambda shp: dict(shape=list(shp), dtype="i8", scale=0.05, zp=0)  # noqa: E731
    ops = [dict(type="tpu.Mul", name="mul", inputs=["x", "c"], attrs=dict(multiplier=77, rshift=12)),
           dict(type="tpu.Add", name="add", inputs=["c", "x"], attrs=dict(multipliers=[90, 70], rshifts=[7, 7], do_relu=True))]
    m = run_graph({"x": qi(q.shape), "c": qi(qc.shape), "mul": qi(q.shape), "add": qi(q.shape)}, ops, {}, {"x": q, "c": qc})
    prod = q.astype(np.int64) * qc
    assert np.array_equal(m.get_raw_tensor("mul"), np.clip((prod * 77 + (1 << 11)) >> 12, -128, 127).astype(np.int8))
    m2 = run_graph({"x": qi(q.shape), "c": qi(qc.shape), "sub": qi(q.shape)},
                   [dict(type="tpu.Sub", name="sub", inputs=["x", "c"], attrs=dict(multipliers=[90, 70], rshifts=[7, 6]))], {}, {"x": q, "c": qc})
    diff = ((q.astype(np.int64) * 90 + 64) >> 7) - ((qc.astype(np.int64) * 70 + 32) >> 6)
    assert np.array_equal(m2.get_raw_tensor("sub"), np.clip(diff, -128, 127).astype(np.int8))
    ssum = ((qc.astype(np.int64) * 90 + 64) >> 7) + ((q.astype(np.int64) * 70 + 64) >> 7)
    assert np.array_equal(m.get_raw_tensor("add"), np.clip(np.maximum(ssum, 0), -128, 127).astype(np.int8))


def test_tpu_const_ops_8bit():
    """tpu.MaxConst / MinConst / SubConst on 8-bit tensors, in the reference's mix of float and integer steps."""
    rng = np.random.default_rng(19)
    q = rng.integers(-128, 128, (2, 3, 4, 5), dtype=np.int8)
    qi = lambda zp=0: dict(shape=list(q.shape), dtype="i8", scale=0.05, zp=zp)  # noqa: E731

    def rsr(v, s):
        return (v + (1 << (s - 1))) >> s if s > 0 else v
    # MaxConst with an input zero point: max(float((x - zp) * m), float(c)) -> int toward zero -> RSR
    m = run_graph({"x": qi(3), "y": qi()}, [dict(type="tpu.MaxConst", name="y", inputs=["x"], attrs=dict(const_val=-150.7, multiplier=9, rshift=3))],
                  {}, {"x": q})
    pf = np.maximum(((q.astype(np.int64) - 3) * 9).astype(np.float32), np.float32(-150.7))
    assert np.array_equal(m.get_raw_tensor("y"), np.clip(rsr(np.trunc(pf).astype(np.int64), 3), -128, 127).astype(np.int8))
    m = run_graph({"x": qi(), "y": qi()}, [dict(type="tpu.MinConst", name="y", inputs=["x"], attrs=dict(const_val=200.25, multiplier=7, rshift=2,
                                                                                                       do_relu=True))], {}, {"x": q})
    pf = np.minimum((q.astype(np.int64) * 7).astype(np.float32), np.float32(200.25))
    assert np.array_equal(m.get_raw_tensor("y"), np.clip(np.maximum(rsr(np.trunc(pf).astype(np.int64), 2), 0), -128, 127).astype(np.int8))
    for rev in (False, True):
        m = run_graph({"x": qi(), "y": qi()}, [dict(type="tpu.SubConst", name="y", inputs=["x"],
                                                    attrs=dict(const_val=33.5, multiplier=11, rshift=4, is_reverse=rev))], {}, {"x": q})
        prod = (q.astype(np.int64) * 11).astype(np.float64)
        f = (33.5 - prod if rev else prod - 33.5).astype(np.float32)
        assert np.array_equal(m.get_raw_tensor("y"), np.clip(rsr(np.trunc(f).astype(np.int64), 4), -128, 127).astype(np.int8)), rev


def test_tpu_concat_requant_is_cv18xx_only():
    """tpu.Concat's multipliers / rshifts are applied by the CV18xx interpreter alone (Concat.cpp:43-60)."""
    rng = np.random.default_rng(20)
    a_ = rng.integers(-128, 128, (2, 3, 4), dtype=np.int8)
    b_ = rng.integers(-128, 128, (2, 5, 4), dtype=np.int8)
    qi = lambda shp: dict(shape=list(shp), dtype="i8", scale=0.05, zp=0)  # noqa: E731
    ops = [dict(type="tpu.Concat", name="y", inputs=["a", "b"], attrs=dict(axis=1, multipliers=[1, 3], rshifts=[0, 2]))]
    for chip in ("bm1684x", "cv183x"):
        g = dict(inputs=["a", "b"], outputs=["y"], tensors={"a": qi(a_.shape), "b": qi(b_.shape), "y": qi((2, 8, 4))}, ops=ops, chip=chip)
        m = module()
        m.load(g, {})
        m.set_tensor("a", a_)
        m.set_tensor("b", b_)
        m.invoke(fixed_to_float=False)
        second = np.clip((b_.astype(np.int64) * 3 + 2) >> 2, -128, 127).astype(np.int8) if chip.startswith("cv18") else b_
        assert np.array_equal(m.get_raw_tensor("y"), np.concatenate([a_, second], axis=1)), chip


@pytest.mark.parametrize("mode", ["reflect", "edge"])
def test_pad_reflect_and_edge(mode):
    rng = np.random.default_rng(21)
    x = rng.standard_normal((2, 3, 5, 6)).astype(np.float32)
    pads = [0, 0, 2, 1, 0, 0, 3, 4]
    ops = [dict(type="top.Pad", name="y", inputs=["x"], attrs=dict(paddings=pads, mode=mode))]
    m = run_graph({"x": f32(x.shape), "y": f32((2, 3, 10, 11))}, ops, {}, {"x": x})
    assert np.array_equal(m.get_tensor("y"), np.pad(x, ((0, 0), (0, 0), (2, 3), (1, 4)), mode=mode))
    q = rng.integers(-128, 128, (1, 2, 4, 4), dtype=np.int8)
    qi = lambda shp: dict(shape=list(shp), dtype="i8", scale=0.05, zp=0)  # noqa: E731
    m = run_graph({"x": qi(q.shape), "y": qi((1, 2, 6, 7))}, [dict(type="tpu.Pad", name="y", inputs=["x"],
                                                                 attrs=dict(paddings=[0, 0, 1, 3, 0, 0, 1, 0], mode=mode))], {}, {"x": q})
    assert np.array_equal(m.get_raw_tensor("y"), np.pad(q, ((0, 0), (0, 0), (1, 1), (3, 0)), mode=mode))


def test_tpu_reduce_8bit():
    rng = np.random.default_rng(22)
    q = rng.integers(-128, 128, (2, 7, 3, 5), dtype=np.int8)
    qi = lambda shp: dict(shape=list(shp), dtype="i8", scale=0.05, zp=0)  # noqa: E731
    m = run_graph({"x": qi(q.shape), "y": qi((2, 3, 5))}, [dict(type="tpu.Reduce", name="y", inputs=["x"],
                                                               attrs=dict(axes=[1], keepdims=False, mode="ReduceMean", multiplier=[77], rshift=[6]))], {}, {"x": q})
    ssum = np.zeros((2, 3, 5), np.float32)
    for a_ in range(7):
        ssum = ssum + q[:, a_].astype(np.float32)
    mean = np.trunc(ssum * np.float32(1.0 / 7)).astype(np.int64)
    assert np.array_equal(m.get_raw_tensor("y"), np.clip((mean * 77 + 32) >> 6, -128, 127).astype(np.int8))
    m = run_graph({"x": qi(q.shape), "y": qi((2, 7))}, [dict(type="tpu.Reduce", name="y", inputs=["x"],
                                                           attrs=dict(axes=[2, 3], keepdims=False, mode="ReduceMax", multiplier=[1], rshift=[0]))], {}, {"x": q})
    assert np.array_equal(m.get_raw_tensor("y"), q.max(axis=(2, 3)))


def test_inverted_residual_block_against_the_oracle():
    """A MobileNetV2 block through the executor, every tensor against the oracle's op walk: 1x1 expansion (tensor cores),
    depthwise 3x3 (the CUDA-core patch kernel), 1x1 projection, residual Add; then a stride-2 depthwise into an Upsample,
    a channel Concat and a PRelu."""
    import oracle
    rng = np.random.default_rng(23)
    N, Cin, Cexp, H = 2, 32, 96, 14
    x = rng.integers(-128, 128, (N, Cin, H, H), dtype=np.int8)

    def conv_w(oc, icg, k):
        return (rng.integers(-127, 128, (oc, icg, k, k), dtype=np.int8), rng.integers(-2000, 2000, oc, dtype=np.int32),
                rng.integers(8000, 20000, oc).tolist(), rng.integers(19, 23, oc).tolist())
    w1, b1, m1, s1 = conv_w(Cexp, Cin, 1)
    wd, bd, md, sd = conv_w(Cexp, 1, 3)
    w2, b2, m2, s2 = conv_w(Cin, Cexp, 1)
    wd2, bd2, md2, sd2 = conv_w(Cin, 1, 3)
    slope = rng.integers(-60, 60, 2 * Cin).astype(np.int8).reshape(1, -1, 1, 1)
    qi = lambda shp: dict(shape=list(shp), dtype="i8", scale=0.05, zp=0)  # noqa: E731
    conv = lambda name, src, k, pads, stride=1, group=1, relu=True, m=None, s=None: dict(  # noqa: E731
        type="tpu.Conv2D", name=name, inputs=[src], attrs=dict(kernel_shape=[k, k], strides=[stride, stride], pads=list(pads), group=group,
                                                                do_relu=relu, multiplier=m, rshift=s, quant_mode="MultiplierShift"))
    ops = [conv("exp", "x", 1, (0, 0, 0, 0), m=m1, s=s1), conv("dw", "exp", 3, (1, 1, 1, 1), group=Cexp, m=md, s=sd),
           conv("proj", "dw", 1, (0, 0, 0, 0), relu=False, m=m2, s=s2),
           dict(type="tpu.Add", name="res", inputs=["x", "proj"], attrs=dict(multipliers=[64, 70], rshifts=[6, 7])),
           conv("down", "res", 3, (1, 1, 1, 1), stride=2, group=Cin, m=md2, s=sd2),
           dict(type="tpu.Upsample", name="up", inputs=["down"], attrs=dict(scale_h=2, scale_w=2)),
           dict(type="tpu.Concat", name="cat", inputs=["res", "up"], attrs=dict(axis=1)),
           dict(type="tpu.PRelu", name="out", inputs=["cat"], attrs=dict(rshift=6))]
    tensors = {"x": qi(x.shape), "exp": qi((N, Cexp, H, H)), "dw": qi((N, Cexp, H, H)), "proj": qi(x.shape), "res": qi(x.shape),
               "down": qi((N, Cin, H // 2, H // 2)), "up": qi(x.shape), "cat": qi((N, 2 * Cin, H, H)), "out": qi((N, 2 * Cin, H, H))}
    weights = {"exp_filter": w1, "exp_bias": b1, "dw_filter": wd, "dw_bias": bd, "proj_filter": w2, "proj_bias": b2, "down_filter": wd2,
               "down_bias": bd2, "out_slope": slope}
    oc_ = lambda t, w, b, mu, sh, **kw: oracle.conv2d_int8(t, w, b, mult=mu, rshift=sh, **kw)  # noqa: E731
    want = {"exp": oc_(x, w1, b1, m1, s1, do_relu=True)}
    want["dw"] = oc_(want["exp"], wd, bd, md, sd, pads=(1, 1, 1, 1), groups=Cexp, do_relu=True)
    want["proj"] = oc_(want["dw"], w2, b2, m2, s2)
    want["res"] = oracle.add_int8(x, want["proj"], 64, 6, 70, 7)
    want["down"] = oc_(want["res"], wd2, bd2, md2, sd2, stride=(2, 2), pads=(1, 1, 1, 1), groups=Cin, do_relu=True)
    want["up"] = np.repeat(np.repeat(want["down"], 2, axis=2), 2, axis=3)
    want["cat"] = np.concatenate([want["res"], want["up"]], axis=1)
    prod = want["cat"].astype(np.int64) * slope
    want["out"] = np.where(want["cat"] < 0, np.clip((prod + 32) >> 6, -128, 127), want["cat"]).astype(np.int8)
    assert len(np.unique(want["out"])) > 50
    # NCHW executor, and the channels-last one (which keeps what the depthwise kernels, Concat's consumer and PRelu read in NCHW)
    for cl in (False, True):
        m = run_graph(tensors, ops, weights, {"x": x}, channels_last=cl)
        m.check_status()
        for name, w_ in want.items():
            assert np.array_equal(m.get_raw_tensor(name), w_), (name, cl)


def test_top_matmul_forms():
    """top.MatMul with a transposed weight, with a second activation (batched over heads, as in attention), and with a
    transposed second activation."""
    rng = np.random.default_rng(24)
    x = rng.standard_normal((2, 3, 5, 16)).astype(np.float32)
    wt = rng.standard_normal((24, 16)).astype(np.float32)
    bias = rng.standard_normal(24).astype(np.float32)
    k_ = rng.standard_normal((2, 3, 7, 16)).astype(np.float32)       # [.., N, K]: scores = x @ k^T
    v_ = rng.standard_normal((2, 3, 16, 9)).astype(np.float32)       # [.., K, N]
    ops = [dict(type="top.MatMul", name="fc", inputs=["x"], attrs=dict(right_transpose=True, do_relu=True)),
           dict(type="top.MatMul", name="qk", inputs=["x", "k"], attrs=dict(right_transpose=True)),
           dict(type="top.MatMul", name="xv", inputs=["x", "v"], attrs={})]
    tensors = {"x": f32(x.shape), "k": f32(k_.shape), "v": f32(v_.shape), "fc": f32((2, 3, 5, 24)), "qk": f32((2, 3, 5, 7)), "xv": f32((2, 3, 5, 9))}
    g = dict(inputs=["x", "k", "v"], outputs=["fc", "qk", "xv"], tensors=tensors, ops=ops)
    m = module()
    m.load(g, {"fc_filter": wt, "fc_bias": bias})
    for n_, v in (("x", x), ("k", k_), ("v", v_)):
        m.set_tensor(n_, v)
    m.invoke(fixed_to_float=False)
    d = lambda a_: a_.astype(np.float64)  # noqa: E731
    np.testing.assert_allclose(m.get_tensor("fc"), np.maximum(d(x) @ d(wt).T + bias, 0), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(m.get_tensor("qk"), d(x) @ d(k_).transpose(0, 1, 3, 2), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(m.get_tensor("xv"), d(x) @ d(v_), rtol=1e-5, atol=1e-5)


def test_float_attention_block():
    """A ViT-style attention block in the Top dialect through the executor (LayerNorm, weight and activation MatMuls, Reshape,
    Permute, MulConst, Softmax, Add, GELU) against numpy in float64: the float graph a calibration of such a model runs."""
    rng = np.random.default_rng(25)
    B, T, D, Hh = 2, 10, 32, 4
    dh = D // Hh
    x = rng.standard_normal((B, T, D)).astype(np.float32)
    W = {k: (rng.standard_normal((D, D)) * 0.2).astype(np.float32) for k in "qkvo"}
    lw, lb = (rng.standard_normal(D) * 0.1 + 1).astype(np.float32), (rng.standard_normal(D) * 0.1).astype(np.float32)
    heads = lambda n_: [dict(type="top.Reshape", name=n_ + "r", inputs=[n_], attrs={}),  # noqa: E731
                        dict(type="top.Permute", name=n_ + "h", inputs=[n_ + "r"], attrs=dict(order=[0, 2, 1, 3]))]
    ops = [dict(type="top.LayerNorm", name="ln", inputs=["x"], attrs=dict(axis=2, eps=1e-5)),
           dict(type="top.MatMul", name="q", inputs=["ln"], attrs={}), dict(type="top.MatMul", name="k", inputs=["ln"], attrs={}),
           dict(type="top.MatMul", name="v", inputs=["ln"], attrs={})] + heads("q") + heads("k") + heads("v") + [
           dict(type="top.MatMul", name="s", inputs=["qh", "kh"], attrs=dict(right_transpose=True)),
           dict(type="top.MulConst", name="ss", inputs=["s"], attrs=dict(const_val=1.0 / math.sqrt(dh))),
           dict(type="top.Softmax", name="p", inputs=["ss"], attrs=dict(axis=3)),
           dict(type="top.MatMul", name="a", inputs=["p", "vh"], attrs={}),
           dict(type="top.Permute", name="ap", inputs=["a"], attrs=dict(order=[0, 2, 1, 3])),
           dict(type="top.Reshape", name="ar", inputs=["ap"], attrs={}),
           dict(type="top.MatMul", name="o", inputs=["ar"], attrs={}),
           dict(type="top.Add", name="res", inputs=["x", "o"], attrs={}),
           dict(type="top.GELU", name="y", inputs=["res"], attrs={})]
    t3, t4, th = f32((B, T, D)), f32((B, T, Hh, dh)), f32((B, Hh, T, dh))
    tensors = {"x": t3, "ln": t3, "q": t3, "k": t3, "v": t3, "qr": t4, "kr": t4, "vr": t4, "qh": th, "kh": th, "vh": th, "s": f32((B, Hh, T, T)),
               "ss": f32((B, Hh, T, T)), "p": f32((B, Hh, T, T)), "a": th, "ap": t4, "ar": t3, "o": t3, "res": t3, "y": t3}
    weights = {"ln_weight": lw, "ln_bias": lb, "q_filter": W["q"], "k_filter": W["k"], "v_filter": W["v"], "o_filter": W["o"]}
    m = run_graph(tensors, ops, weights, {"x": x})
    d = lambda a_: np.asarray(a_, dtype=np.float64)  # noqa: E731
    xd = d(x)
    mu = xd.mean(axis=2, keepdims=True)
    ln = (xd - mu) / np.sqrt(((xd - mu) ** 2).mean(axis=2, keepdims=True) + 1e-5) * d(lw) + d(lb)
    split = lambda t: t.reshape(B, T, Hh, dh).transpose(0, 2, 1, 3)  # noqa: E731
    q_, k_, v_ = (split(ln @ d(W[c])) for c in "qkv")
    sc = q_ @ k_.transpose(0, 1, 3, 2) / math.sqrt(dh)
    e_ = np.exp(sc - sc.max(axis=3, keepdims=True))
    p_ = e_ / e_.sum(axis=3, keepdims=True)
    o_ = (p_ @ v_).transpose(0, 2, 1, 3).reshape(B, T, D) @ d(W["o"])
    res = xd + o_
    want = 0.5 * res * (1 + np.vectorize(math.erf)(res / math.sqrt(2.0)))
    np.testing.assert_allclose(m.get_tensor("p"), p_, rtol=2e-4, atol=1e-6)
    np.testing.assert_allclose(m.get_tensor("y"), want, rtol=2e-4, atol=2e-5)


def test_run_calibration_on_a_float_graph(tmp_path):
    """run_calibration (the reference's tool flow) on a small float graph: table written in the reference's format, thresholds
    within (0, abs max], the min / max columns equal to numpy's over the same samples, tuning only ever raises a threshold."""
    from tpu_mlir_b200.cali_table import read_cali_table
    from tpu_mlir_b200.run_calibration import run_calibration
    rng = np.random.default_rng(26)
    B, Cc, H = 4, 8, 6
    w1 = (rng.standard_normal((16, Cc, 3, 3)) * 0.2).astype(np.float32)
    ops = [dict(type="top.Conv", name="c1", inputs=["x"], attrs=dict(kernel_shape=[3, 3], pads=[1, 1, 1, 1], do_relu=True)),
           dict(type="top.MaxPool", name="p1", inputs=["c1"], attrs=dict(kernel_shape=[2, 2], strides=[2, 2])),
           dict(type="top.Sigmoid", name="s1", inputs=["p1"], attrs={})]
    tensors = {"x": f32((B, Cc, H, H)), "c1": f32((B, 16, H, H)), "p1": f32((B, 16, 3, 3)), "s1": f32((B, 16, 3, 3))}
    g = dict(inputs=["x"], outputs=["s1"], tensors=tensors, ops=ops)
    samples = rng.standard_normal((16, Cc, H, H)).astype(np.float32)
    path = str(tmp_path / "cali_table")
    th = run_calibration(g, {"c1_filter": w1}, samples, out_table=path)
    table = read_cali_table(path)
    assert set(th) == {"x", "c1", "p1", "s1"} and list(table.int8) == ["x", "c1", "p1", "s1"]
    assert all(0 < v for v in th.values()) and th["x"] <= float(np.abs(samples).max()) + 1e-6
    assert abs(table.int8["x"][1] - float(samples.min())) < 1e-5 and abs(table.int8["x"][2] - float(samples.max())) < 1e-5
    assert all(abs(table.int8[n][0] - th[n]) < 1e-6 for n in th)
    assert table.int8["s1"][1] >= 0.5 - 1e-6 and table.int8["s1"][2] <= 1.0 + 1e-6          # a sigmoid of ReLU'd values
    tuned = run_calibration(g, {"c1_filter": w1}, samples, tune_num=2)
    assert all(tuned[n] >= th[n] - 1e-7 for n in th)
