"""Reader / writer of the MLIR text subset of a lowered model."""
import os

import numpy as np
import pytest

from tpu_mlir_b200 import mlir_text as MT

# a checkout of the reference, when there is one (TPU_MLIR_REFERENCE overrides the default location)
REF_SAMPLE = os.path.join(os.environ.get("TPU_MLIR_REFERENCE", "/root/reference"), "test/Transforms/Parallel/Conv.mlir")


def test_types():
    t = MT.parse_type("tensor<1x256x14x14xf32>")
    assert (t.shape, t.dtype, t.scale) == ([1, 256, 14, 14], "f32", None)
    t = MT.parse_type("tensor<1x256x14x14x!quant.uniform<i8:f32, 0.064606035433070863>>")
    assert (t.shape, t.dtype, t.zp) == ([1, 256, 14, 14], "i8", 0) and t.scale == 0.064606035433070863
    t = MT.parse_type("tensor<1x25088x!quant.uniform<u8:f32, 0.051140184251968507:128>, 4362649600 : i64>")
    assert (t.shape, t.dtype, t.zp, t.address) == ([1, 25088], "u8", 128, 4362649600)
    t = MT.parse_type("tensor<1x16x512x!quant.calibrated<f32<-0.92979659999999997:0.92979659999999997>>, 4459302912 : i64>")
    assert (t.shape, t.dtype, t.scale) == ([1, 16, 512], "f32", None)
    assert MT.parse_type("none").dtype == "none"
    for txt in ("tensor<2x3xsi8>", "tensor<4x!quant.uniform<u8:f32, 0.5:3>>", "tensor<7x1x!quant.uniform<i8:f32, 0.25>>"):
        assert MT.format_type(MT.parse_type(txt)) == txt


def test_attributes():
    a = MT.parse_attr_dict('{coeff_merged = false, dilations = [1, 1], group = 1 : i64, quant_mode = #tpu<rq_mode MultiplierShift>, '
                           'relu_limit = -1.000000e+00 : f64, name = "a, b}", multiplier = [123, -4], pool_mode = #tpu<pool_mode Avg>, '
                           'next_index = array<i32: -1, 2>, flag}')
    assert a == dict(coeff_merged=False, dilations=[1, 1], group=1, quant_mode="MultiplierShift", relu_limit=-1.0,
                     name="a, b}", multiplier=[123, -4], pool_mode="Avg", next_index=[-1, 2], flag=True)


@pytest.mark.skipif(not os.path.isfile(REF_SAMPLE), reason="the reference tree is not present on this machine")
def test_reference_sample_parses():
    mod = MT.parse_module(open(REF_SAMPLE).read())
    assert mod.name == "Conv2d_2" and mod.attrs["module.chip"] == "bm1688" and mod.attrs["module.cores"] == 8
    assert [a[2] for a in mod.args] == ["input"]
    types = [o.type for o in mod.ops]
    assert types == ["top.Weight", "top.Weight", "tpu.Conv2D"]
    conv = mod.ops[2]
    assert conv.loc == "output_Conv" and conv.attrs["kernel_shape"] == [3, 3] and conv.attrs["quant_mode"] == "MultiplierShift"
    assert conv.attrs["with_bias"] is True and conv.out_types[0].shape == [4, 65, 100, 100]
    assert [mod.ops[0].loc, mod.ops[1].loc] == ["weight", "bias"]
    assert mod.returns == [conv.results[0]]


def small_graph():
    rng = np.random.default_rng(0)
    tensors = {"input": dict(shape=[2, 3, 8, 8], dtype="f32"),
               "input_q": dict(shape=[2, 3, 8, 8], dtype="i8", scale=0.03125, zp=0),
               "conv": dict(shape=[2, 16, 8, 8], dtype="u8", scale=0.0625, zp=0),
               "pool": dict(shape=[2, 16, 4, 4], dtype="u8", scale=0.0625, zp=0),
               "sum": dict(shape=[2, 16, 4, 4], dtype="i8", scale=0.125, zp=0),
               "flat": dict(shape=[2, 256], dtype="i8", scale=0.125, zp=0),
               "fc": dict(shape=[2, 10], dtype="i8", scale=0.5, zp=0),
               "output": dict(shape=[2, 10], dtype="f32")}
    ops = [dict(type="tpu.Cast", name="input_q", inputs=["input"]),
           dict(type="tpu.Conv2D", name="conv", inputs=["input_q"],
                attrs=dict(kernel_shape=[3, 3], strides=[1, 1], dilations=[1, 1], pads=[1, 1, 1, 1], group=1, do_relu=True,
                           quant_mode="MultiplierShift", multiplier=[int(v) for v in rng.integers(100, 2000, 16)],
                           rshift=[int(v) for v in rng.integers(8, 14, 16)])),
           dict(type="tpu.Pool2D", name="pool", inputs=["conv"],
                attrs=dict(pool_mode="Max", kernel_shape=[2, 2], strides=[2, 2], pads=[0, 0, 0, 0], do_relu=False)),
           dict(type="tpu.Add", name="sum", inputs=["pool", "pool"], attrs=dict(do_relu=False, multipliers=[64, 64], rshifts=[7, 7])),
           dict(type="tpu.Reshape", name="flat", inputs=["sum"]),
           dict(type="tpu.MatMul", name="fc", inputs=["flat"], attrs=dict(do_relu=False, quant_mode="MultiplierShift",
                                                                         multipliers=[77], rshifts=[12])),
           dict(type="tpu.Cast", name="output", inputs=["fc"])]
    weights = {"conv_filter": rng.integers(-127, 128, (16, 3, 3, 3), dtype=np.int8),
               "conv_bias": rng.integers(-100, 100, 16, dtype=np.int32),
               "fc_filter": rng.integers(-127, 128, (256, 10), dtype=np.int8)}     # no bias: a top.None operand
    return dict(inputs=["input"], outputs=["output"], tensors=tensors, ops=ops), weights


def test_emit_then_load_round_trip(tmp_path):
    graph, weights = small_graph()
    text = MT.emit_module(graph, weights, weight_file="w.npz")
    (tmp_path / "m.mlir").write_text(text)
    np.savez(tmp_path / "w.npz", **weights)
    g2, w2 = MT.load_mlir(str(tmp_path / "m.mlir"))
    assert g2["inputs"] == graph["inputs"] and g2["outputs"] == graph["outputs"]
    assert [(o["type"], o["name"], o["inputs"]) for o in g2["ops"]] == [(o["type"], o["name"], o["inputs"]) for o in graph["ops"]]
    for o, o2 in zip(graph["ops"], g2["ops"]):
        assert o.get("attrs", {}) == o2.get("attrs", {}), o["name"]
    for n, t in graph["tensors"].items():
        t2 = g2["tensors"][n]
        assert t2["shape"] == t["shape"] and t2["dtype"] == t["dtype"] and t2.get("scale") == t.get("scale")
    assert set(w2) == set(weights)
    for k in weights:
        assert np.array_equal(w2[k], weights[k]) and w2[k].dtype == weights[k].dtype


def test_divided_modules_are_rejected():
    text = 'module @m attributes {module.state = "TPU_DIVIDED"} {\n  func.func @main(%arg0: tensor<1xf32> loc("i")) -> tensor<1xf32> {\n' \
           '    %0 = "func.call"(%arg0) : (tensor<1xf32>) -> tensor<1xf32> loc(#loc)\n    return %0 : tensor<1xf32> loc(#loc)\n  }\n}\n'
    with pytest.raises(MT.MlirTextError):
        MT.parse_module(text)


def test_elementwise_ops_round_trip(tmp_path):
    """tpu.Lut (with its table as a weight operand), tpu.MulShift and tpu.Mul survive emit -> load."""
    rng = np.random.default_rng(1)
    shp = [1, 16, 4, 4]
    tensors = {"input": dict(shape=shp, dtype="f32"),
               "q": dict(shape=shp, dtype="i8", scale=0.25, zp=0),
               "lut": dict(shape=shp, dtype="i8", scale=0.25, zp=0),
               "ms": dict(shape=shp, dtype="u8", scale=0.5, zp=3),
               "mul": dict(shape=shp, dtype="i8", scale=0.125, zp=0)}
    ops = [dict(type="tpu.Cast", name="q", inputs=["input"]),
           dict(type="tpu.Lut", name="lut", inputs=["q"]),
           dict(type="tpu.MulShift", name="ms", inputs=["q"], attrs=dict(multiplier=90, rshift=6)),
           dict(type="tpu.Mul", name="mul", inputs=["lut", "ms"], attrs=dict(multiplier=5, rshift=7, do_relu=True))]
    graph = dict(inputs=["input"], outputs=["mul"], tensors=tensors, ops=ops)
    weights = {"lut_table": rng.integers(-128, 128, 256).astype(np.int8)}
    (tmp_path / "m.mlir").write_text(MT.emit_module(graph, weights, weight_file="w.npz"))
    np.savez(tmp_path / "w.npz", **weights)
    g2, w2 = MT.load_mlir(str(tmp_path / "m.mlir"))
    assert [(o["type"], o["name"], o["inputs"], o.get("attrs", {})) for o in g2["ops"]] == \
           [(o["type"], o["name"], o["inputs"], o.get("attrs", {})) for o in ops]
    assert np.array_equal(w2["lut_table"].reshape(-1), weights["lut_table"])
    assert g2["tensors"]["ms"]["zp"] == 3 and g2["tensors"]["ms"]["dtype"] == "u8"
