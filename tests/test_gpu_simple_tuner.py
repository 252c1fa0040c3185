"""The threshold tuner on the GPU against a host restatement of the reference's SimpleTuner
(python/calibration/simple_tunner.py:334-507) that evaluates the ops with the oracle's fp32 kernels."""
import copy

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import oracle  # noqa: E402
from tpu_mlir_b200 import resnet50  # noqa: E402
from tpu_mlir_b200.module import module  # noqa: E402
from tpu_mlir_b200.simple_tuner import SimpleTuner, import_quant_bias  # noqa: E402


def small_graph(rng, batch=2):
    tensors = {"input": {"shape": [batch, 4, 10, 10], "dtype": "f32"}, "c1": {"shape": [batch, 8, 10, 10], "dtype": "f32"},
               "c2": {"shape": [batch, 8, 10, 10], "dtype": "f32"}, "sum": {"shape": [batch, 8, 10, 10], "dtype": "f32"},
               "pool": {"shape": [batch, 8, 5, 5], "dtype": "f32"}, "c3": {"shape": [batch, 6, 5, 5], "dtype": "f32"}}
    ops = [dict(type="top.Conv", name="c1", inputs=["input"], attrs=dict(kernel_shape=[3, 3], pads=[1, 1, 1, 1], do_relu=True)),
           dict(type="top.Conv", name="c2", inputs=["c1"], attrs=dict(kernel_shape=[1, 1])),
           dict(type="top.Add", name="sum", inputs=["c1", "c2"], attrs=dict(do_relu=True)),
           dict(type="top.MaxPool", name="pool", inputs=["sum"], attrs=dict(kernel_shape=[2, 2], strides=[2, 2])),
           dict(type="top.Conv", name="c3", inputs=["pool"], attrs=dict(kernel_shape=[3, 3], pads=[1, 1, 1, 1]))]
    w = {"c1_filter": rng.standard_normal((8, 4, 3, 3)).astype(np.float32) * 0.3, "c1_bias": rng.standard_normal(8).astype(np.float32) * 0.1,
         "c2_filter": rng.standard_normal((8, 8, 1, 1)).astype(np.float32) * 0.4, "c2_bias": rng.standard_normal(8).astype(np.float32) * 0.1,
         "c3_filter": rng.standard_normal((6, 8, 3, 3)).astype(np.float32) * 0.2, "c3_bias": rng.standard_normal(6).astype(np.float32) * 0.1}
    return dict(inputs=["input"], outputs=["c3"], tensors=tensors, ops=ops, state="TOP_F32"), w


def host_eval(op, ins, w):
    a, t = op.get("attrs", {}), op["type"]
    if t == "top.Conv":
        p = a.get("pads", [0, 0, 0, 0])
        return oracle.top_conv2d_f32(ins[0], w[op["name"] + "_filter"], w.get(op["name"] + "_bias"), stride=tuple(a.get("strides", [1, 1])),
                                     pads=(p[0], p[2], p[1], p[3]), do_relu=bool(a.get("do_relu", False)))
    if t == "top.Add":
        y = ins[0] + ins[1]
        return np.maximum(y, 0) if a.get("do_relu") else y
    if t == "top.MaxPool":
        p = a.get("pads", [0, 0, 0, 0])
        return oracle.top_pool2d_f32(ins[0], kernel=a["kernel_shape"], stride=a.get("strides", [1, 1]), pads=(p[0], p[2], p[1], p[3]), is_max=True)
    raise ValueError(t)


class HostTuner:
    """simple_tunner.py:334-507 with numpy arrays (default flags)."""

    def __init__(self, graph, weights, samples, thresholds, abs_max, tune_num, tune_steps=21):
        self.graph, self.w = graph, weights
        self.wq = {}
        for k, v in weights.items():               # fake_quant_weight (ModuleInterpreter.cpp:583-612)
            mx = np.abs(v).max()
            self.wq[k] = v if k.endswith("_bias") or mx == 0 else (np.round(v * 127 / mx) * mx / 127).astype(np.float32)
        self.tune_num, self.tune_steps = tune_num, tune_steps
        self.thresholds, self.initial = dict(thresholds), copy.deepcopy(thresholds)
        self.abs_max = abs_max
        self.ops = {o["name"]: o for o in graph["ops"]}
        self.ref = []
        for s in samples[:tune_num]:
            acts = {"input": s}
            for o in graph["ops"]:
                acts[o["name"]] = host_eval(o, [acts[i] for i in o["inputs"]], weights)
            self.ref.append(acts)
        self.tuned = []

    def distance(self, evaled, th):
        d = 0.0
        op = self.ops[evaled]
        for idx in range(self.tune_num):
            out = host_eval(op, [import_quant_bias(self.ref[idx][i], th) for i in op["inputs"]], self.wq)
            r = self.ref[idx][evaled]
            d += np.linalg.norm((r.astype(np.float64) - out).ravel()) / np.abs(r.astype(np.float64)).sum()
        return d / self.tune_num

    def find(self, evaled, tuned):
        th0, amax = self.initial[tuned], self.abs_max[tuned]
        step = (amax - th0) / self.tune_steps
        best, prev = th0, -1.0
        if step > 0 and abs(amax - th0) > 0.01:
            for i in range(self.tune_steps + 1):
                cur = th0 + step * i
                d = self.distance(evaled, cur)
                if prev == -1.0:
                    prev = d
                elif d < prev:
                    prev, best = d, cur
        if best > self.thresholds[tuned]:
            self.thresholds[tuned] = best

    def run(self):
        for o in self.graph["ops"]:
            pre = o["inputs"]
            if all(p in self.tuned for p in pre):
                self.find(o["name"], pre[0])
                self.tuned.append(pre[0])
                continue
            for t in pre:
                if t not in self.tuned:
                    self.find(o["name"], t)
                    self.tuned.append(t)
        return self.thresholds


def test_import_quant_bias_kernel_matches_numpy():
    import ctypes as C

    from tpu_mlir_b200 import _lib as L
    rng = np.random.default_rng(2)
    x = (rng.standard_normal(100003) * 3).astype(np.float32)
    x[:8] = [0.5, 1.5, 2.5, -0.5, -1.5, 1000.0, -1000.0, 0.0]      # ties round to even, both clips
    for th in (127.0, 3.3, 0.017, 211.7):
        xd = torch.from_numpy(x).cuda()
        yd = torch.empty_like(xd)
        L.check(L.lib().b200q_top_fake_quant_f32_dev(C.c_void_p(xd.data_ptr()), C.c_void_p(yd.data_ptr()), x.size, th, None))
        assert np.array_equal(yd.cpu().numpy(), import_quant_bias(x, th)), th


def test_tuner_matches_host_restatement():
    rng = np.random.default_rng(4)
    graph, w = small_graph(rng)
    samples = [rng.standard_normal((2, 4, 10, 10)).astype(np.float32) for _ in range(3)]
    # "calibration": thresholds at 60 % of each tensor's absolute maximum over the samples
    m = module()
    m.load(graph, w)
    abs_max = {n: 0.0 for n in graph["tensors"]}
    for s in samples:
        m.set_tensor("input", s)
        m.invoke()
        for n in abs_max:
            abs_max[n] = max(abs_max[n], float(np.abs(m.get_tensor(n)).max()))
    thresholds = {n: 0.6 * v for n, v in abs_max.items()}
    host = HostTuner(graph, w, samples, thresholds, abs_max, tune_num=3)
    want = host.run()
    tuner = SimpleTuner(graph, w, samples, thresholds, abs_max, tune_num=3)
    got = tuner.run()
    assert set(got) == set(want)
    assert tuner.evaluations > 0
    changed = 0
    for n in want:
        if got[n] != want[n]:
            # the same candidate grid: a different pick is only acceptable between candidates the host cannot tell apart
            user = next(o["name"] for o in graph["ops"] if n in o["inputs"])
            assert host.distance(user, got[n]) <= host.distance(user, want[n]) * (1 + 1e-4), (n, got[n], want[n])
        assert got[n] >= thresholds[n]
        changed += got[n] > thresholds[n]
    assert changed >= 2, "the tuner should have moved some thresholds on this graph"


def test_tuner_on_resnet50_head():
    """The first ops of the ResNet-50 Top graph (stem, pool, first bottleneck) with one sample: runs end to end, thresholds
    only grow and stay within the absolute maxima."""
    ops = resnet50.build_fp32()[:7]
    graph, w = resnet50.top_graph(ops, batch=1)
    x = np.random.default_rng(0).standard_normal((1, 3, 224, 224)).astype(np.float32)
    m = module()
    m.load(graph, w)
    m.set_tensor("input", x)
    m.invoke()
    abs_max = {n: float(np.abs(m.get_tensor(n)).max()) for n in graph["tensors"]}
    thresholds = {n: 0.5 * v for n, v in abs_max.items()}
    got = SimpleTuner(graph, w, [x], thresholds, abs_max, tune_num=1, tune_steps=5).run()
    for n, v in got.items():
        assert thresholds[n] <= v <= abs_max[n] * (1 + 1e-6)
