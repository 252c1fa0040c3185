"""Host logic of the executor's channels-last residency: which tensors of a graph are stored as [N][H][W][C]."""
import pytest

from tpu_mlir_b200 import _lib as L
from tpu_mlir_b200.module import module


def _graph(ops, shapes, dtypes=None):
    dtypes = dtypes or {}
    return {"inputs": ["input"], "outputs": [ops[-1]["name"]],
            "tensors": {n: {"shape": s, "dtype": dtypes.get(n, "i8"), "scale": 1.0, "zp": 0} for n, s in shapes.items()},
            "ops": ops}


def test_bottleneck_block_is_channels_last_behind_the_stem():
    ops = [dict(type="tpu.Cast", name="q", inputs=["input"]),
           dict(type="tpu.Conv2D", name="stem", inputs=["q"], attrs=dict(group=1)),
           dict(type="tpu.Pool2D", name="pool", inputs=["stem"], attrs={}),
           dict(type="tpu.Conv2D", name="c1", inputs=["pool"], attrs=dict(group=1)),
           dict(type="tpu.Conv2D", name="ds", inputs=["pool"], attrs=dict(group=1)),
           dict(type="tpu.Add", name="add", inputs=["c1", "ds"], attrs={}),
           dict(type="tpu.Pool2D", name="gap", inputs=["add"], attrs={}),
           dict(type="tpu.Reshape", name="flat", inputs=["gap"]),
           dict(type="tpu.MatMul", name="fc", inputs=["flat"], attrs={}),
           dict(type="tpu.Cast", name="out", inputs=["fc"])]
    shapes = dict(input=[2, 3, 32, 32], q=[2, 3, 32, 32], stem=[2, 64, 16, 16], pool=[2, 64, 8, 8], c1=[2, 256, 8, 8],
                  ds=[2, 256, 8, 8], add=[2, 256, 8, 8], gap=[2, 256, 1, 1], flat=[2, 256], fc=[2, 10], out=[2, 10])
    g = _graph(ops, shapes, dict(input="f32", out="f32"))
    nhwc = module._assign_layouts(g, {})
    # the quantised 3-channel input stays NCHW (the stem gathers its rows from it); everything 4-D behind it is NHWC
    assert nhwc == {"stem", "pool", "c1", "ds", "add", "gap"}


def test_channel_count_and_groups_decide():
    ops = [dict(type="tpu.Conv2D", name="a", inputs=["input"], attrs=dict(group=1)),      # 24 output channels: not % 16
           dict(type="tpu.Conv2D", name="b", inputs=["a"], attrs=dict(group=1)),           # NCHW in, NHWC out
           dict(type="tpu.Conv2D", name="c", inputs=["b"], attrs=dict(group=32))]          # grouped: cannot read NHWC
    shapes = dict(input=[1, 16, 8, 8], a=[1, 24, 8, 8], b=[1, 32, 8, 8], c=[1, 32, 8, 8])
    g = _graph(ops[:2], shapes)
    assert module._assign_layouts(g, {}) == {"b"}
    # a grouped convolution reads NCHW: its producer then writes NCHW instead of the graph being refused
    assert module._assign_layouts(_graph(ops, shapes), {}) == set()


def test_add_of_mixed_layouts_keeps_both_operands_nchw():
    ops = [dict(type="tpu.Conv2D", name="a", inputs=["input"], attrs=dict(group=1)),
           dict(type="tpu.Add", name="s", inputs=["a", "input"], attrs={})]
    shapes = dict(input=[1, 32, 4, 4], a=[1, 32, 4, 4], s=[1, 32, 4, 4])
    assert module._assign_layouts(_graph(ops, shapes), {}) == set()
