"""Runs a Tpu-dialect graph dict (the executor's format) on the CPU with the oracle's op restatements."""
import numpy as np

import oracle

_DT = {"i8": oracle.DT_I8, "u8": oracle.DT_U8, "i32": oracle.DT_I32}
_QM = {"TFLite_LShift": 0, "TFLite": 1, "MultiplierShift": 2, "OnlyShift": 3, "QDM": 4, "OnlyScale": 5}


def run(graph, weights, inputs):
    T = dict(inputs)
    info = graph["tensors"]
    for op in graph["ops"]:
        t, a, name = op["type"], op.get("attrs", {}), op["name"]
        x = T[op["inputs"][0]]
        o = info[name]
        if t == "tpu.Cast":
            i = info[op["inputs"][0]]
            if i["dtype"] == "f32":
                T[name] = oracle.cast_f32_to_q8(x, o["scale"], o["zp"], out_dt=_DT[o["dtype"]])
            else:
                T[name] = oracle.cast_q8_to_f32(x, i["scale"], i["zp"])
        elif t == "tpu.Conv2D":
            p = a["pads"]
            out, viol = oracle.conv2d_int8(x, weights[name + "_filter"], weights.get(name + "_bias"), stride=a["strides"],
                                           pads=(p[0], p[2], p[1], p[3]), dilation=a["dilations"], groups=a["group"],
                                           do_relu=a["do_relu"], qmode=_QM[a["quant_mode"]], mult=a["multiplier"],
                                           rshift=a["rshift"], out_zp=o["zp"], out_dt=_DT[o["dtype"]], return_violations=True)
            assert viol == 0, name
            T[name] = out
        elif t == "tpu.MatMul":
            fuse_rq = bool(a.get("fuse_rq", False))
            mult = oracle.through_f32(weights[name + "_multi"]) if fuse_rq else a["multipliers"]
            if a.get("left_transpose", False):      # stored [K, M]: lib/Support/Dnnl/MatMul.cpp:182-186 transposes it first
                x = np.ascontiguousarray(x.T)
            T[name] = oracle.matmul_int8(x, weights[name + "_filter"], weights.get(name + "_bias"), do_relu=a["do_relu"],
                                         right_transpose=bool(a.get("right_transpose", False)),
                                         input_zp=int(a.get("input_zp", 0)), right_zp=int(a.get("right_zp", 0)),
                                         qmode=_QM[a["quant_mode"]], fuse_rq=fuse_rq, mult=mult, rshift=a["rshifts"][:1] if fuse_rq else a["rshifts"],
                                         out_zp=o["zp"], out_dt=_DT[o["dtype"]])
            if a.get("output_transpose", False):    # stored [N, M]: lib/Support/Dnnl/MatMul.cpp:229-238
                T[name] = np.ascontiguousarray(T[name].T)
        elif t == "tpu.Add":
            m, s = a["multipliers"], a["rshifts"]
            T[name] = oracle.add_int8(x, T[op["inputs"][1]], m[0], s[0], m[1], s[1], do_relu=a["do_relu"], out_dt=_DT[o["dtype"]])
        elif t == "tpu.Pool2D":
            p = a["pads"]
            T[name] = oracle.pool2d_int8(x, a["kernel_shape"], a["strides"], (p[0], p[2], p[1], p[3]),
                                         mode="max" if a["pool_mode"] == "Max" else "avg", multi=a.get("multiplier", 1),
                                         rshift=a.get("rshift", 0), do_relu=a["do_relu"], out_dt=_DT[o["dtype"]])
        elif t == "tpu.Reshape":
            T[name] = x.reshape(o["shape"])
        else:
            raise ValueError(t)
    return T
