"""Random-init ResNet-50 for the whole-network configurations: the fp32 (Top-level) graph used for calibration
and its INT8 symmetric Tpu-dialect lowering for chip family bm1684x.

There are no trained weights or images here: weights are torchvision's default initialisation (Kaiming-normal
convolutions, BatchNorm gamma = 1, beta = 0, running statistics (0, 1)) under a fixed seed, BatchNorm is folded
into the preceding convolution and ReLU fused into its producer, as the reference's Top canonicalisation does
(lib/Dialect/Top/Canonicalize/BatchNorm.cpp:16, Scale.cpp:322-332, Relu.cpp:15-60).  Lowering rules: lowering.py.
"""
from __future__ import annotations

from typing import Dict, List

import numpy as np

from . import lowering as LW


def build_fp32(seed: int = 3) -> List[dict]:
    """Fused fp32 op list in execution order: conv (+relu), maxpool, add (+relu), avgpool, fc."""
    import torch
    import torchvision
    torch.manual_seed(seed)
    m = torchvision.models.resnet50(weights=None).eval()
    ops: List[dict] = []

    def conv(name, inp, c, bn, relu):
        w = (c.weight.detach() * (bn.weight.detach() / torch.sqrt(bn.running_var + bn.eps)).reshape(-1, 1, 1, 1))
        b = bn.bias.detach() - bn.running_mean * bn.weight.detach() / torch.sqrt(bn.running_var + bn.eps)
        ops.append(dict(type="conv", name=name, inputs=[inp], w=w.numpy().astype(np.float32), b=b.numpy().astype(np.float32),
                        stride=list(c.stride), pad=list(c.padding), relu=relu))
        return name

    x = conv("conv1", "input", m.conv1, m.bn1, True)
    ops.append(dict(type="maxpool", name="pool1", inputs=[x], kernel=[3, 3], stride=[2, 2], pad=[1, 1]))
    x = "pool1"
    for li, layer in enumerate([m.layer1, m.layer2, m.layer3, m.layer4], start=1):
        for bi, blk in enumerate(layer):
            p = f"layer{li}.{bi}"
            y = conv(p + ".conv1", x, blk.conv1, blk.bn1, True)
            y = conv(p + ".conv2", y, blk.conv2, blk.bn2, True)
            y = conv(p + ".conv3", y, blk.conv3, blk.bn3, False)
            idn = x
            if blk.downsample is not None:
                idn = conv(p + ".downsample", x, blk.downsample[0], blk.downsample[1], False)
            ops.append(dict(type="add", name=p + ".add", inputs=[y, idn], relu=True))
            x = p + ".add"
    ops.append(dict(type="avgpool", name="avgpool", inputs=[x], kernel=[7, 7]))
    ops.append(dict(type="fc", name="fc", inputs=["avgpool"], w=m.fc.weight.detach().numpy().T.copy().astype(np.float32),
                    b=m.fc.bias.detach().numpy().astype(np.float32)))
    return ops


class Fp32Forward:
    """fp32 forward of the fused graph with this library's Top-dialect kernels (full-fp32 implicit-GEMM convolution,
    pooling, add, matrix product: csrc/top_f32.cu); returns every activation (the calibration targets) as NCHW device
    tensors.  Needs the CUDA library: there is no other path."""

    def __init__(self, ops: List[dict], device):
        import ctypes as C

        import torch

        from . import _lib as L
        self.torch, self.C, self.L = torch, C, L
        self.ops = ops
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise L.B200QError(L.ERR_UNSUPPORTED, "Fp32Forward runs on a CUDA device only")
        self.par = {}
        self.handles = {}
        self.shape = {}
        with torch.cuda.device(self.device):
            shapes = {"input": (3, 224, 224)}
            for op in ops:
                cin = shapes[op["inputs"][0]]
                if op["type"] == "conv":
                    w = torch.from_numpy(op["w"]).to(self.device).contiguous()
                    b = torch.from_numpy(op["b"]).to(self.device).contiguous()
                    oc, _, kh, kw = op["w"].shape
                    d = L.TopConvDesc(n=1, ic=cin[0], ih=cin[1], iw=cin[2], oc=oc, kh=kh, kw=kw, sh=op["stride"][0],
                                      sw=op["stride"][1], dh=1, dw=1, pht=op["pad"][0], phb=op["pad"][0], pwl=op["pad"][1],
                                      pwr=op["pad"][1], groups=1, with_bias=1, do_relu=int(op["relu"]), relu_limit=-1.0)
                    h = C.c_void_p()
                    L.check(L.lib().b200q_top_conv2d_dev_create(C.byref(d), C.c_void_p(w.data_ptr()), C.c_void_p(b.data_ptr()),
                                                                C.byref(h)))
                    oh, ow = C.c_int64(), C.c_int64()
                    L.lib().b200q_top_conv2d_dev_output_shape(h, C.byref(oh), C.byref(ow))
                    self.handles[op["name"]] = h
                    self.par[op["name"]] = (w, b)          # the handle reads the bias in place: keep it alive
                    shapes[op["name"]] = (oc, oh.value, ow.value)
                elif op["type"] == "maxpool":
                    k, s_, p_ = op["kernel"], op["stride"], op["pad"]
                    shapes[op["name"]] = (cin[0], (cin[1] + 2 * p_[0] - k[0]) // s_[0] + 1, (cin[2] + 2 * p_[1] - k[1]) // s_[1] + 1)
                elif op["type"] == "add":
                    shapes[op["name"]] = cin
                elif op["type"] == "avgpool":
                    k = op["kernel"]
                    shapes[op["name"]] = (cin[0], (cin[1] - k[0]) // k[0] + 1, (cin[2] - k[1]) // k[1] + 1)
                elif op["type"] == "fc":
                    self.par[op["name"]] = (torch.from_numpy(op["w"]).to(self.device).contiguous(),
                                            torch.from_numpy(op["b"]).to(self.device).contiguous())
                    shapes[op["name"]] = (op["w"].shape[1],)
                else:
                    raise ValueError(op["type"])
            self.shape = shapes

    def __del__(self):
        try:
            for h in self.handles.values():
                self.L.lib().b200q_top_conv2d_dev_destroy(self.C.byref(h))
        except Exception:
            pass

    def __call__(self, x) -> Dict[str, "object"]:
        torch, C, L = self.torch, self.C, self.L
        lib = L.lib()
        P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
        x = x.to(self.device, dtype=torch.float32).contiguous()
        if tuple(x.shape[1:]) != self.shape["input"]:
            raise L.B200QError(L.ERR_INVALID, f"input must be [B, 3, 224, 224], got {tuple(x.shape)}")
        B = x.shape[0]
        acts = {"input": x}
        with torch.cuda.device(self.device):
            stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            for op in self.ops:
                a = acts[op["inputs"][0]]
                t = op["type"]
                y = torch.empty((B,) + tuple(self.shape[op["name"]]), dtype=torch.float32, device=self.device)
                if t == "conv":
                    L.check(lib.b200q_top_conv2d_dev_run(self.handles[op["name"]], P(a), P(y), B, stream))
                elif t == "maxpool":
                    k, s_, p_ = op["kernel"], op["stride"], op["pad"]
                    L.check(lib.b200q_top_pool2d_f32_dev(P(a), P(y), B * a.shape[1], a.shape[2], a.shape[3], k[0], k[1], s_[0],
                                                         s_[1], p_[0], p_[0], p_[1], p_[1], 1, 0, 0, -1.0, stream))
                elif t == "add":
                    L.check(lib.b200q_top_add_f32_dev(P(a), P(acts[op["inputs"][1]]), P(y), y.numel(), int(op["relu"]), -1.0, stream))
                elif t == "avgpool":
                    k = op["kernel"]
                    L.check(lib.b200q_top_pool2d_f32_dev(P(a), P(y), B * a.shape[1], a.shape[2], a.shape[3], k[0], k[1], k[0],
                                                         k[1], 0, 0, 0, 0, 0, 1, 0, -1.0, stream))
                elif t == "fc":
                    w, b = self.par[op["name"]]
                    L.check(lib.b200q_top_matmul_f32_dev(P(a), P(w), P(b), P(y), B, w.shape[0], w.shape[1], 0, -1.0, stream))
                else:
                    raise ValueError(t)
                acts[op["name"]] = y
        return acts


def fp32_forward_torch(ops: List[dict], x):
    """The same graph through torch's own operators (on CPU: oneDNN, the library the reference's Top dialect calls).
    Test infrastructure: a second opinion on Fp32Forward, never on the product path."""
    import torch
    F = torch.nn.functional
    acts = {"input": x}
    for op in ops:
        a = acts[op["inputs"][0]]
        t = op["type"]
        if t == "conv":
            y = F.conv2d(a, torch.from_numpy(op["w"]).to(a.device), torch.from_numpy(op["b"]).to(a.device), stride=op["stride"],
                         padding=op["pad"])
            y = F.relu(y) if op["relu"] else y
        elif t == "maxpool":
            y = F.max_pool2d(a, op["kernel"], op["stride"], op["pad"])
        elif t == "add":
            y = a + acts[op["inputs"][1]]
            y = F.relu(y) if op["relu"] else y
        elif t == "avgpool":
            y = F.avg_pool2d(a, op["kernel"])
        elif t == "fc":
            y = a.flatten(1) @ torch.from_numpy(op["w"]).to(a.device) + torch.from_numpy(op["b"]).to(a.device)
        else:
            raise ValueError(t)
        acts[op["name"]] = y
    return acts


def top_graph(ops: List[dict], batch: int):
    """The fused fp32 op list as a Top-dialect graph for the executor (module.py): (graph, weights)."""
    tensors = {"input": {"shape": [batch, 3, 224, 224], "dtype": "f32"}}
    gops, weights = [], {}
    for op in ops:
        cin = tensors[op["inputs"][0]]["shape"]
        t, name = op["type"], op["name"]
        if t == "conv":
            oc, _, kh, kw = op["w"].shape
            p, s_ = op["pad"], op["stride"]
            shape = [batch, oc, (cin[2] + 2 * p[0] - kh) // s_[0] + 1, (cin[3] + 2 * p[1] - kw) // s_[1] + 1]
            gops.append(dict(type="top.Conv", name=name, inputs=list(op["inputs"]),
                             attrs=dict(kernel_shape=[kh, kw], strides=list(s_), pads=[p[0], p[1], p[0], p[1]], do_relu=op["relu"])))
            weights[name + "_filter"], weights[name + "_bias"] = op["w"], op["b"]
        elif t == "maxpool":
            k, s_, p = op["kernel"], op["stride"], op["pad"]
            shape = [batch, cin[1], (cin[2] + 2 * p[0] - k[0]) // s_[0] + 1, (cin[3] + 2 * p[1] - k[1]) // s_[1] + 1]
            gops.append(dict(type="top.MaxPool", name=name, inputs=list(op["inputs"]),
                             attrs=dict(kernel_shape=list(k), strides=list(s_), pads=[p[0], p[1], p[0], p[1]])))
        elif t == "add":
            shape = list(cin)
            gops.append(dict(type="top.Add", name=name, inputs=list(op["inputs"]), attrs=dict(do_relu=op["relu"])))
        elif t == "avgpool":
            k = op["kernel"]
            shape = [batch, cin[1], cin[2] // k[0], cin[3] // k[1]]
            gops.append(dict(type="top.AvgPool", name=name, inputs=list(op["inputs"]),
                             attrs=dict(kernel_shape=list(k), strides=list(k), pads=[0, 0, 0, 0], count_include_pad=True)))
        elif t == "fc":
            shape = [batch, op["w"].shape[1]]
            gops.append(dict(type="top.MatMul", name=name, inputs=list(op["inputs"]), attrs={}))
            weights[name + "_filter"], weights[name + "_bias"] = op["w"], op["b"]
        else:
            raise ValueError(t)
        tensors[name] = {"shape": shape, "dtype": "f32"}
    return dict(inputs=["input"], outputs=[ops[-1]["name"]], tensors=tensors, ops=gops, state="TOP_F32"), weights


def lower_int8(ops: List[dict], table: Dict[str, tuple], batch: int):
    """INT8 symmetric lowering.  ``table[name] = (threshold, min, max)`` is the calibration table.  Returns
    (graph, weights) in the format module.load takes."""
    relu_of = {op["name"]: bool(op.get("relu", False)) for op in ops}
    shapes = {"input": [batch, 3, 224, 224]}
    q: Dict[str, tuple] = {}

    def qtype(name):
        th, vmin, _ = table[name]
        return LW.tensor_qtype(float(th), float(vmin), relu_of.get(name, False))

    q["input"] = qtype("input")
    tensors = {"input": dict(shape=shapes["input"], dtype="f32")}
    gops: List[dict] = []
    weights: Dict[str, np.ndarray] = {}

    def add_tensor(name, shape, dt, scale):
        tensors[name] = dict(shape=list(shape), dtype=dt, scale=float(scale), zp=0)
        shapes[name] = list(shape)

    add_tensor("input_q", shapes["input"], *q["input"])
    gops.append(dict(type="tpu.Cast", name="input_q", inputs=["input"]))
    alias = {"input": "input_q"}

    for op in ops:
        t, name = op["type"], op["name"]
        src = [alias.get(i, i) for i in op["inputs"]]
        ishape = shapes[src[0]]
        if t == "conv":
            q[name] = qtype(name)
            oc, _, kh, kw = op["w"].shape
            oh = (ishape[2] + 2 * op["pad"][0] - kh) // op["stride"][0] + 1
            ow = (ishape[3] + 2 * op["pad"][1] - kw) // op["stride"][1] + 1
            add_tensor(name, [batch, oc, oh, ow], *q[name])
            w_q, b_q, mult, rs = LW.lower_conv(op["w"], op["b"], tensors[src[0]]["scale"], q[name][1])
            weights[name + "_filter"], weights[name + "_bias"] = w_q, b_q
            gops.append(dict(type="tpu.Conv2D", name=name, inputs=src,
                             attrs=dict(kernel_shape=[kh, kw], strides=op["stride"], dilations=[1, 1],
                                        pads=[op["pad"][0], op["pad"][1], op["pad"][0], op["pad"][1]], group=1,
                                        do_relu=op["relu"], quant_mode="MultiplierShift", multiplier=mult.tolist(),
                                        rshift=rs.tolist())))
        elif t == "maxpool":
            # the output shares its input's calibrated type (ForwardCalibartion<MaxPoolOp>, TopToTpuPass.cpp:1835-1935)
            q[name] = (tensors[src[0]]["dtype"], tensors[src[0]]["scale"])
            oh = (ishape[2] + 2 * op["pad"][0] - op["kernel"][0]) // op["stride"][0] + 1
            ow = (ishape[3] + 2 * op["pad"][1] - op["kernel"][1]) // op["stride"][1] + 1
            add_tensor(name, [batch, ishape[1], oh, ow], *q[name])
            gops.append(dict(type="tpu.Pool2D", name=name, inputs=src,
                             attrs=dict(pool_mode="Max", kernel_shape=op["kernel"], strides=op["stride"],
                                        pads=[op["pad"][0], op["pad"][1], op["pad"][0], op["pad"][1]], do_relu=False)))
        elif t == "add":
            q[name] = qtype(name)
            add_tensor(name, ishape, *q[name])
            m, s = LW.lower_add([tensors[i]["scale"] for i in src], q[name][1])
            gops.append(dict(type="tpu.Add", name=name, inputs=src, attrs=dict(do_relu=op["relu"], multipliers=m, rshifts=s)))
        elif t == "avgpool":
            # sign follows the input (KeepSignPattern, TopToTpuPass.cpp:467-504): unsigned after a ReLU
            th = float(table[name][0])
            q[name] = ("u8", th / 255.0) if tensors[src[0]]["dtype"] == "u8" else ("i8", th / 127.0)
            add_tensor(name, [batch, ishape[1], 1, 1], *q[name])
            mlt, rs = LW.lower_avgpool(tensors[src[0]]["scale"], q[name][1], *op["kernel"])
            gops.append(dict(type="tpu.Pool2D", name=name, inputs=src,
                             attrs=dict(pool_mode="Avg", kernel_shape=op["kernel"], strides=[1, 1], pads=[0, 0, 0, 0],
                                        multiplier=mlt, rshift=rs, do_relu=False)))
        elif t == "fc":
            flat = name + "_flat"
            add_tensor(flat, [batch, ishape[1]], tensors[src[0]]["dtype"], tensors[src[0]]["scale"])
            gops.append(dict(type="tpu.Reshape", name=flat, inputs=src))
            q[name] = qtype(name)
            add_tensor(name, [batch, op["w"].shape[1]], *q[name])
            w_q, b_q, mlt, rs = LW.lower_fc(op["w"], op["b"], tensors[flat]["scale"], q[name][1])
            weights[name + "_filter"], weights[name + "_bias"] = w_q, b_q
            gops.append(dict(type="tpu.MatMul", name=name, inputs=[flat],
                             attrs=dict(do_relu=False, quant_mode="MultiplierShift", multipliers=[mlt], rshifts=[rs])))
    last = ops[-1]["name"]
    tensors["output"] = dict(shape=shapes[last], dtype="f32")
    gops.append(dict(type="tpu.Cast", name="output", inputs=[last]))
    graph = dict(inputs=["input"], outputs=["output"], tensors=tensors, ops=gops)
    return graph, weights


def self_calibration_table(ops: List[dict], images, batch: int = 16, math=None, dist=None) -> Dict[str, tuple]:
    """Calibration table (threshold, min, max) of every activation from the KLD calibrator on `images`
    (a torch tensor [S,3,224,224] on the device; with `dist`, the local shard of the sample order)."""
    from .calibration import ShardedCalibrator
    fwd = Fp32Forward(ops, images.device)
    cal = ShardedCalibrator(fwd, math=math, dist=dist)
    batches = [images[i:i + batch] for i in range(0, images.shape[0], batch)]
    res = cal.run(batches, samples_per_rank=images.shape[0])
    return {n: (r.threshold, r.min, r.max) for n, r in res.items()}
