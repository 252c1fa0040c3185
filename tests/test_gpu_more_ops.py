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
        run_graph({"x": f32(x.shape), "p": f32((1, 2, 5, 5))}, [dict(type="top.Pad", name="p", inputs=["x"], attrs=dict(paddings=[0, 0, 1, 1, 0, 0, 1, 1], mode="reflect"))],
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
