"""Host logic of the channels-last executor: which tensors are stored [N][H][W][C] (module._assign_layouts)."""
from tpu_mlir_b200.module import module


def qi(shape):
    return dict(shape=list(shape), dtype="i8", scale=0.05, zp=0)


def conv(name, src, oc_unused=None, group=1):
    return dict(type="tpu.Conv2D", name=name, inputs=[src], attrs=dict(kernel_shape=[1, 1], group=group, multiplier=[1], rshift=[0]))


def test_residual_chain_stays_channels_last():
    t = {n: qi((2, 64, 8, 8)) for n in ("x", "a", "b", "sum", "pool")}
    ops = [conv("a", "x"), conv("b", "a"), dict(type="tpu.Add", name="sum", inputs=["a", "b"], attrs={}),
           dict(type="tpu.Pool2D", name="pool", inputs=["sum"], attrs={})]
    assert module._assign_layouts(dict(tensors=t, ops=ops), {}) == {"a", "b", "sum", "pool"}


def test_an_nchw_only_consumer_pins_its_input_and_what_feeds_it_elementwise():
    t = {n: qi((2, 64, 8, 8)) for n in ("x", "a", "b", "sum", "dw", "c", "pr")}
    ops = [conv("a", "x"), conv("b", "a"), dict(type="tpu.Add", name="sum", inputs=["a", "b"], attrs={}),
           conv("dw", "sum", group=64),              # depthwise: reads NCHW, so the Add writes NCHW, so both its operands are NCHW
           conv("c", "dw"),                          # a dense convolution after it is channels-last again
           dict(type="tpu.PRelu", name="pr", inputs=["c"], attrs={})]       # ... unless its consumer reads NCHW only
    assert module._assign_layouts(dict(tensors=t, ops=ops), {}) == set()
    ops[-1] = dict(type="tpu.Pool2D", name="pr", inputs=["c"], attrs={})
    assert module._assign_layouts(dict(tensors=t, ops=ops), {}) == {"c", "pr"}


def test_broadcasting_add_keeps_its_operands_nchw():
    t = {"x": qi((2, 64, 8, 8)), "a": qi((2, 64, 8, 8)), "s": qi((1, 64, 1, 1)), "y": qi((2, 64, 8, 8))}
    ops = [conv("a", "x"), dict(type="tpu.Add", name="y", inputs=["a", "s"], attrs={})]
    assert module._assign_layouts(dict(tensors=t, ops=ops), {}) == set()
