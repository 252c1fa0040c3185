"""GPU-resident executor for an INT8 Tpu-dialect graph: the role of the reference's ModuleInterpreter /
``pymlir.module`` and ``pymlir.cuda`` (bindings/pymlir/pymlir.cpp:101-131,
bindings/pymlir/host/ModuleInterpreter.cpp:396-492,:631-1012, bindings/pymlir/pycuda.cpp:438-669).

Method names and meaning follow ``pymlir.module``: ``load, set_tensor, set_tensor_from_int, invoke(fixed_to_float),
invoke_at, invoke_from, fake_quant_weight, get_tensor, get_fp32_tensor, get_all_tensor, before_invoke / after_invoke /
clear_hooks, get_tensor_qinfo, input_names, output_names, all_tensor_names, all_weight_names``; ``parser`` answers the
graph queries of the reference's MlirParser (graph_queries.py).  Tensors live on the device in their native storage type (like ``py_cuda``), ops run in graph
order through the device face of libb200q.so.  A graph is a plain dict whose op types and attribute names are the Tpu
dialect's (``load`` also takes the path of a lowered model's ``.mlir`` text and reads it into this form, mlir_text.py):

    {"inputs": [...], "outputs": [...],
     "tensors": {name: {"shape": [...], "dtype": "f32|i8|u8|i32", "scale": s, "zp": z}},
     "ops": [{"type": "tpu.Conv2D", "name": out_tensor, "inputs": [...], "attrs": {...}}, ...]}

with weights in a dict ``name -> numpy array`` (``<op>_filter``, ``<op>_bias``).

``module(channels_last=True)`` keeps the 4-D activations that convolutions, adds and pools produce as [N][H][W][C]
on the device (the order the tensor-core kernels read and write), so no transposing kernel runs between ops;
``get_tensor`` / ``set_tensor`` still speak NCHW, and the values are identical.  ``module(cuda_graph=True)`` makes
``invoke()`` replay one captured CUDA graph of all ops while no hook is registered (small per-GPU batches are
otherwise bound by the host's launch rate).
"""
from __future__ import annotations

import ctypes as C
import itertools
from typing import Callable, Dict, List, Optional

import numpy as np

from . import _lib as L

_DT = {"i8": L.DT_I8, "u8": L.DT_U8, "i32": L.DT_I32, "f32": L.DT_F32}
_RM = {"HalfAwayFromZero": 0, "HalfUp": 1, "HalfDown": 2, "HalfToEven": 3, "HalfToOdd": 4, "HalfTowardsZero": 5, "TowardsZero": 6,
       "AwayFromZero": 7, "Up": 8, "Down": 9}
_QM = {"TFLite_LShift": 0, "TFLite": 1, "MultiplierShift": 2, "OnlyShift": 3, "QDM": 4, "OnlyScale": 5}


# Tpu-dialect ops that, on f32 tensors, compute what the Top op of the same name computes
_TPU_F32_AS_TOP = ("tpu.Sub", "tpu.Div", "tpu.MaxConst", "tpu.MinConst", "tpu.SubConst", "tpu.Softmax", "tpu.LayerNorm", "tpu.Reduce")
# Tpu_ActiveMode (include/tpu_mlir/Dialect/Tpu/IR/TpuOps.td:284-321)
_ACTIVE_MODES = {n: i for i, n in enumerate(
    "TANH SIGMOID RELU EXP ELU SQRT SQUARE RSQRT ABSVAL LN ROUND CEIL FLOOR SIN COS IS_FINITE MISH SWISH HSWISH SILU ARCSIN ARCCOS "
    "ARCSINH ARCCOSH ARCTANH SINH COSH TAN SIGN GELU ERF HSIGMOID LOG_SIGMOID SOFT_PLUS SOFT_SIGN LOG2 TGELU QGELU".split())}
# Tpu-dialect ops whose plans take NCHW-stored tensors only (a channels-last executor keeps their inputs NCHW)
_NCHW_ONLY = ("tpu.Deconv", "tpu.PRelu", "tpu.Sub", "tpu.MaxConst", "tpu.MinConst", "tpu.SubConst", "tpu.Reduce", "tpu.RequantFp",
              "tpu.RequantIntAxis", "tpu.Gather", "tpu.GatherElements", "tpu.Arg", "tpu.Interp", "tpu.GridSampler", "tpu.Depth2Space",
              "tpu.Active", "tpu.Div", "tpu.Softmax", "tpu.LayerNorm", "tpu.AddConst", "tpu.MulConst", "tpu.Relu")
_MOVE_OPS = ("Slice", "Permute", "Tile", "Upsample", "Pad", "Concat", "Squeeze", "Unsqueeze", "Depth2Space", "SwapDimInner")


def _P(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


class module:  # noqa: N801  (name of the reference class)
    def __init__(self, device: Optional[int] = None, channels_last: bool = False, cuda_graph: bool = False,
                 fuse_residual_add: bool = False):
        import torch
        self.channels_last = bool(channels_last)
        # A tpu.Add whose later operand is a convolution output nobody else reads runs inside that convolution's
        # kernel: the Add's tensor receives the same values, the convolution's own tensor is never written (reading
        # it raises).  Off by default: the reference materialises every tensor.
        self.fuse_residual_add = bool(fuse_residual_add)
        self._fuse_into: Dict[str, dict] = {}     # convolution name -> the Add op fused into it
        self._fused_adds: Dict[str, str] = {}     # Add name -> convolution name
        self.cuda_graph = bool(cuda_graph)  # invoke() without hooks replays one captured CUDA graph of all ops
        self._graph = None
        self._nhwc = set()  # names of the tensors stored as [N][H][W][C]
        self.torch = torch
        if not torch.cuda.is_available():
            raise L.B200QError(L.ERR_NO_DEVICE, "the executor needs a CUDA device (there is no CPU fallback)")
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None else device)
        self.lib = L.lib()
        self.graph = None
        self.tensors: Dict[str, "torch.Tensor"] = {}
        self._plans: List[Callable] = []
        self._handles: List[C.c_void_p] = []
        self._top_handles: List[C.c_void_p] = []   # fp32 Top-dialect convolutions
        self._keep = []
        self._before: List[Callable] = []
        self._after: List[Callable] = []
        self._expressed = False   # the last invoke() asked for float ("expressed") tensors
        self._status: List = []   # (op name, device status word or conv handle): checked after invoke

    # ------------------------------------------------------------------ loading
    def load(self, graph, weights: Optional[Dict[str, np.ndarray]] = None):
        """``graph`` is the dict described above, or the path of a lowered model's ``.mlir`` text (module state
        TPU_LOWERED); in that case ``weights`` may name the weight file, else the module's ``module.weight_file``
        attribute is followed (mlir_text.load_mlir)."""
        torch = self.torch
        if isinstance(graph, str):
            from .mlir_text import load_mlir
            graph, weights = load_mlir(graph, weights if isinstance(weights, str) else None)
        self.graph = graph
        self._extra_info = {}        # expanded copies of broadcast operands (not tensors of the graph)
        self.input_names = list(graph["inputs"])
        self.output_names = list(graph["outputs"])
        self.all_tensor_names = list(graph["tensors"].keys())
        self.all_weight_names = list(weights.keys())
        tdt = {"i8": torch.int8, "u8": torch.uint8, "i32": torch.int32, "f32": torch.float32}
        self._nhwc = self._assign_layouts(graph, weights) if self.channels_last else set()
        for name, info in graph["tensors"].items():
            shape = tuple(info["shape"])
            if name in self._nhwc:
                shape = (shape[0], shape[2], shape[3], shape[1])
            self.tensors[name] = torch.zeros(shape, dtype=tdt[info["dtype"]], device=self.device)
        self.weights = {k: torch.from_numpy(np.ascontiguousarray(v)).to(self.device) for k, v in weights.items()}
        from .graph_queries import MlirParser
        self.parser = MlirParser(graph)
        self._build_plans()

    def _build_plans(self):
        self._release_handles()
        self._plans, self._keep, self._status, self._graph = [], [], [], None
        self._fuse_into, self._fused_adds = self._find_residual_adds() if self.fuse_residual_add else ({}, {})
        for op in self.graph["ops"]:
            self._plans.append(self._plan(op))
        self.torch.cuda.synchronize(self.device)

    def _find_residual_adds(self):
        """Adds that can run in the epilogue of the convolution producing their later operand."""
        ops = self.graph["ops"]
        order = {op["name"]: i for i, op in enumerate(ops)}
        by_name = {op["name"]: op for op in ops}
        uses: Dict[str, int] = {}
        for op in ops:
            for n in op["inputs"]:
                uses[n] = uses.get(n, 0) + 1
        fuse_into, fused = {}, {}
        for op in ops:
            if op["type"] != "tpu.Add" or len(op["inputs"]) != 2:
                continue
            a = op.get("attrs", {})
            m, s = a.get("multipliers", []), a.get("rshifts", [])
            if len(m) != 2 or len(s) != 2 or not all(abs(int(v)) < (1 << 23) for v in m) or not all(1 <= int(v) <= 31 for v in s):
                continue
            i0, i1 = op["inputs"]
            later = i0 if order.get(i0, -1) > order.get(i1, -1) else i1
            other = i1 if later == i0 else i0
            prod = by_name.get(later)
            if prod is None or prod["type"] != "tpu.Conv2D" or uses.get(later, 0) != 1 or later in self.graph["outputs"]:
                continue
            if prod.get("attrs", {}).get("group", 1) != 1 or later in fuse_into or \
                    prod.get("attrs", {}).get("quant_mode", "MultiplierShift") != "MultiplierShift":   # the kernel's fused form
                continue
            infos = [self._info(later), self._info(other), self._info(op["name"])]
            if any(i["dtype"] not in ("i8", "u8") for i in infos) or list(infos[0]["shape"]) != list(infos[1]["shape"]):
                continue
            if (later in self._nhwc) != (other in self._nhwc) or (later in self._nhwc) != (op["name"] in self._nhwc):
                continue
            fuse_into[later] = dict(add=op, other=other, self_index=0 if later == i0 else 1)
            fused[op["name"]] = later
        return fuse_into, fused

    def _release_handles(self):
        for h in self._handles:
            self.lib.b200q_conv2d_dev_destroy(C.byref(h))
        self._handles = []
        for h in self._top_handles:
            self.lib.b200q_top_conv2d_dev_destroy(C.byref(h))
        self._top_handles = []

    def __del__(self):
        try:
            self._release_handles()
        except Exception:
            pass

    def _info(self, name):
        info = self.graph["tensors"].get(name)
        return info if info is not None else self._extra_info[name]

    @staticmethod
    def _assign_layouts(graph, weights):
        """Which tensors are stored channels-last: the output of a convolution that a tensor-core route takes (one
        group, output channels a multiple of 16), and whatever an Add, Pool2D or Cast derives from such tensors."""
        nhwc = set()
        tens = graph["tensors"]
        pinned = set()      # tensors some consumer can only read as NCHW: their producers write NCHW
        while True:
            nhwc, again = set(), False
            for op in graph["ops"]:
                t, a, name = op["type"], op.get("attrs", {}), op["name"]
                ins = op["inputs"]
                stored = [i for i in ins if i in nhwc]
                if t == "tpu.Conv2D":
                    if a.get("group", 1) != 1 and stored:          # the CUDA-core kernels of grouped convolutions read NCHW
                        pinned.update(stored)
                        again = True
                        break
                    oc = tens[name]["shape"][1] if len(tens[name]["shape"]) == 4 else 0
                    if a.get("group", 1) == 1 and oc and oc % 16 == 0 and tens[name]["dtype"] in ("i8", "u8") and name not in pinned:
                        nhwc.add(name)
                elif t in ("tpu.Add", "tpu.Mul"):
                    if len(stored) == len(ins) and len(tens[name]["shape"]) == 4 and name not in pinned and \
                            all(list(tens[i]["shape"]) == list(tens[name]["shape"]) for i in ins):
                        nhwc.add(name)
                    elif stored:                                    # mixed layouts, a pinned result or broadcasting: all NCHW
                        pinned.update(stored)
                        again = True
                        break
                elif t in ("tpu.Pool2D", "tpu.Cast", "tpu.Lut", "tpu.MulShift"):
                    if stored and name not in pinned:
                        nhwc.add(name)
                    elif stored:
                        pinned.update(stored)
                        again = True
                        break
                elif t.split(".", 1)[-1] in _MOVE_OPS and t.split(".", 1)[-1] != "Depth2Space":
                    pass                                            # the index-mapping kernel reads either storage order, writes NCHW
                elif stored and (t in _NCHW_ONLY or t.startswith("top.")):      # these plans read NCHW only
                    pinned.update(stored)
                    again = True
                    break
            if not again:
                break
        return nhwc

    def _plan(self, op) -> Callable:
        t, a, lib = op["type"], op.get("attrs", {}), self.lib
        ins = [self.tensors[n] for n in op["inputs"]]
        out = self.tensors[op["name"]]
        iinfo = [self._info(n) for n in op["inputs"]]
        oinfo = self._info(op["name"])
        stream = lambda: C.c_void_p(self.torch.cuda.current_stream(self.device).cuda_stream)  # noqa: E731
        if t.split(".", 1)[-1] in ("Add", "Mul", "Sub", "Div") and len(ins) == 2 and \
                (list(iinfo[0]["shape"]) != list(oinfo["shape"]) or list(iinfo[1]["shape"]) != list(oinfo["shape"])):
            return self._plan_broadcast(op, stream)
        if t.split(".", 1)[-1] in _MOVE_OPS:
            return self._plan_move(op, stream)
        if t in ("top.Interp", "tpu.Interp"):
            modes = {"nearest": 0, "linear": 1}
            coords = {"half_pixel": 0, "pytorch_half_pixel": 1, "align_corners": 2, "asymmetric": 3}
            plats = {"ONNX": 0, "TORCH": 1, "TFLITE": 2, "CAFFE": 3}
            ishape, oshape = list(iinfo[0]["shape"]), list(oinfo["shape"])
            if iinfo[0]["dtype"] != "f32" or oinfo["dtype"] != "f32" or a.get("mode") not in modes or a.get("coord_mode") not in coords \
                    or len(ishape) != 4 or op["inputs"][0] in self._nhwc or op["name"] in self._nhwc or len(ins) > 1:
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: {t} takes a 4-D f32 NCHW tensor, mode nearest / linear, a fixed output shape")
            nc, ih, iw, oh, ow = ishape[0] * ishape[1], ishape[2], ishape[3], oshape[2], oshape[3]
            mode, coord = modes[a["mode"]], coords[a["coord_mode"]]
            plat = plats.get(str(a.get("platform", self.graph.get("platform", "ONNX"))).upper(), 0)
            return lambda: L.check(lib.b200q_interp_f32_dev(_P(ins[0]), _P(out), nc, ih, iw, oh, ow, mode, coord, plat, stream()))
        if t in ("top.GridSampler", "tpu.GridSampler"):
            gshape = list(iinfo[1]["shape"])
            if any(i["dtype"] != "f32" for i in iinfo) or oinfo["dtype"] != "f32" or len(gshape) != 4 or gshape[3] != 2 \
                    or any(nm in self._nhwc for nm in list(op["inputs"]) + [op["name"]]):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: {t} takes f32 NCHW tensors and a [N, OH, OW, 2] grid")
            nb, ch, ih, iw = iinfo[0]["shape"]
            oh, ow = gshape[1], gshape[2]
            mode, pad, al = int(a.get("mode", 0)), int(a.get("padding_mode", 0)), int(bool(a.get("align_corners", False)))
            return lambda: L.check(lib.b200q_grid_sampler_f32_dev(_P(ins[0]), _P(ins[1]), _P(out), nb, ch, ih, iw, oh, ow, mode, pad, al, stream()))
        if t in ("top.Arg", "tpu.Arg"):
            # Arg.cpp:39-83; the op's own tensor holds the indices (f32 as the reference stores them, or i32), the optional
            # `values` entry of the op names the tensor of the extreme values
            if iinfo[0]["dtype"] != "f32" or oinfo["dtype"] not in ("f32", "i32") or op["inputs"][0] in self._nhwc:
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: {t} takes an f32 NCHW tensor and writes f32 or i32 indices")
            if a["mode"] not in ("ArgMax", "ArgMin"):
                raise L.B200QError(L.ERR_INVALID, f"{op['name']}: mode {a['mode']}")
            shape = list(iinfo[0]["shape"])
            ax = int(a["axis"])
            ax += len(shape) if ax < 0 else 0
            outer, inner = int(np.prod(shape[:ax])), int(np.prod(shape[ax + 1:]))
            vals = self.tensors[op["values"]] if op.get("values") else None
            if out.numel() != outer * inner or (vals is not None and (vals.numel() != outer * inner or self._info(op["values"])["dtype"] != "f32")):
                raise L.B200QError(L.ERR_INVALID, f"{op['name']}: output shapes do not match the reduction")
            is_max, last, isf = int(a["mode"] == "ArgMax"), int(bool(a.get("select_last_index", True))), int(oinfo["dtype"] == "f32")
            return lambda: L.check(lib.b200q_arg_f32_dev(_P(ins[0]), outer, shape[ax], inner, is_max, last, _P(out), isf, _P(vals), stream()))
        if t == "top.Cast":
            # Cast.cpp:18-68
            to = {"INT8": "i8", "UINT8": "u8", "INT16": "i16", "UINT16": "u16", "INT32": "i32", "UINT32": "i32", "F32": "f32"}.get(a.get("to", ""))
            codes = dict(_DT, i16=L.DT_I16, u16=L.DT_U16)
            if to is None or iinfo[0]["dtype"] != "f32" or oinfo["dtype"] not in ("f32", to):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: top.Cast to '{a.get('to')}' from {iinfo[0]['dtype']} into {oinfo['dtype']}")
            if (op["inputs"][0] in self._nhwc) != (op["name"] in self._nhwc):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: top.Cast between differently stored tensors")
            n, rm = out.numel(), _RM[a.get("round_mode", "HalfAwayFromZero")]
            return lambda: L.check(lib.b200q_top_cast_f32_dev(_P(ins[0]), n, codes[to], rm, codes[oinfo["dtype"]], _P(out), stream()))
        if t.split(".", 1)[-1] in ("Gather", "GatherElements"):
            return self._plan_gather(op, ins, out, iinfo, stream)
        if t.startswith("top."):
            return self._plan_top(op, ins, out, iinfo, stream)
        if t in _TPU_F32_AS_TOP and oinfo["dtype"] == "f32" and all(i["dtype"] == "f32" for i in iinfo):
            # F32-mode Tpu ops whose inference is the Top op's arithmetic (lib/Dialect/Tpu/Interfaces/Common/<Op>.cpp)
            top_op = dict(op, type="top." + t[4:])
            if t == "tpu.Reduce" and op.get("attrs", {}).get("mode") == "ReduceMean":
                top_op["attrs"] = dict(op["attrs"], mode="ReduceMeanRcp")
            return self._plan_top(top_op, ins, out, iinfo, stream)
        if t in ("tpu.RequantFp", "tpu.RequantIntAxis"):
            if op["inputs"][0] in self._nhwc or op["name"] in self._nhwc:
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: {t} on channels-last stored tensors")
            n = out.numel()
            qm, rm = _QM[a["quant_mode"]], _RM[a.get("round_mode", "HalfAwayFromZero")]
            idt, odt = _DT[iinfo[0]["dtype"]], _DT[oinfo["dtype"]]
            if t == "tpu.RequantFp":
                sc, of, zp = float(a["scale"]), float(a.get("offset", 0.0)), int(oinfo.get("zp", 0))
                return lambda: L.check(lib.b200q_requant_fp_dev(_P(ins[0]), idt, n, sc, of, zp, qm, rm, odt, _P(out), stream()))
            # RequantIntAxis.cpp:16-125, quant operand [C][3] = (multiplier, shift, zero point) (the BM1684X layout, :45-48)
            if iinfo[0]["dtype"] != "i32":
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: tpu.RequantIntAxis takes an int32 tensor here")
            shape = list(oinfo["shape"])
            fuse = bool(a.get("fuse_rq_axis", False))
            ch = shape[-1] if fuse else shape[1]
            inner = 1 if fuse else (int(np.prod(shape[2:])) if len(shape) > 2 else 1)
            outer = n // (ch * inner)
            table = self.weights[op["name"] + "_quant"].to(self.torch.int32).reshape(-1)
            if table.numel() != 3 * ch:
                raise L.B200QError(L.ERR_INVALID, f"{op['name']}: the quant table must hold (multiplier, shift, zero point) per channel")
            table = table.reshape(ch, 3)
            tf = qm in (L.QM_TFLITE, L.QM_TFLITE_LSHIFT)
            if not tf and qm != L.QM_MULTIPLIER_SHIFT:
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: tpu.RequantIntAxis quant_mode {a['quant_mode']}")
            mu = table[:, 0].contiguous()
            sh = (table[:, 1] if (tf or fuse) else -table[:, 1]).contiguous()          # :96-98 negates the shift word; :73-87 does not
            zp = table[:, 2].contiguous()
            self._keep.append((mu, sh, zp))
            dialect = L.RQ_QDM if tf else L.RQ_MULTIPLIER_SHIFT
            izp = int(iinfo[0].get("zp", 0))
            return lambda: L.check(lib.b200q_requant_int_axis_dev(_P(ins[0]), outer, ch, inner, _P(mu), _P(sh), _P(zp), dialect, rm, izp, odt,
                                                                  _P(out), stream()))
        if t == "tpu.PRelu":
            fl = oinfo["dtype"] == "f32"
            w = self.weights[op["name"] + "_slope"]
            w = (w.to(self.torch.float32) if fl else w.to(self.torch.int8)).contiguous().reshape(-1)
            self._keep.append(w)
            if op["inputs"][0] in self._nhwc or op["name"] in self._nhwc:
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: tpu.PRelu on channels-last stored tensors")
            shape = list(iinfo[0]["shape"])
            inner = int(np.prod(shape[2:])) if len(shape) > 2 else 1
            n, ns, sft = out.numel(), w.numel(), int(a.get("rshift", 0))
            return lambda: L.check(lib.b200q_prelu_dev(_P(ins[0]), _DT[iinfo[0]["dtype"]], _P(w), n, inner, ns, sft, _DT[oinfo["dtype"]],
                                                       _P(out), stream()))
        if t == "tpu.Active":
            if oinfo["dtype"] != "f32" or iinfo[0]["dtype"] != "f32":
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: tpu.Active runs on f32 tensors here")
            mode = a["mode"]
            mode = _ACTIVE_MODES[mode] if isinstance(mode, str) else int(mode)
            co = [float(v) for v in (a.get("coeffs") or [])] + [0.0, 0.0]
            n = out.numel()
            return lambda: L.check(lib.b200q_active_f32_dev(mode, _P(ins[0]), co[0], co[1], _P(out), n, stream()))
        if t == "tpu.Cast":
            n = out.numel()
            if iinfo[0]["dtype"] == "f32":
                return lambda: L.check(lib.b200q_cast_f32_to_q8_dev(_P(ins[0]), n, float(oinfo["scale"]), int(oinfo["zp"]),
                                                                    L.ROUND_HALF_AWAY_FROM_ZERO, _DT[oinfo["dtype"]],
                                                                    _P(out), stream()))
            return lambda: L.check(lib.b200q_cast_q8_to_f32_dev(_P(ins[0]), _DT[iinfo[0]["dtype"]], n,
                                                                float(iinfo[0]["scale"]), int(iinfo[0]["zp"]), _P(out),
                                                                stream()))
        if t == "tpu.Conv2D":
            from .ops import Conv2DOp
            w = self.weights[op["name"] + "_filter"]
            b = self.weights.get(op["name"] + "_bias")
            pads = a.get("pads", [0, 0, 0, 0])
            cop = Conv2DOp(input_shape=tuple(iinfo[0]["shape"]), oc=w.shape[0], kernel_shape=tuple(a["kernel_shape"]),
                           strides=tuple(a.get("strides", [1, 1])), dilations=tuple(a.get("dilations", [1, 1])),
                           pads=tuple(pads), group=a.get("group", 1), with_bias=b is not None,
                           do_relu=bool(a.get("do_relu", False)), input_dtype=_DT[iinfo[0]["dtype"]],
                           out_dtype=_DT[oinfo["dtype"]], quant_mode=_QM[a.get("quant_mode", "MultiplierShift")],
                           out_zp=int(oinfo.get("zp", 0)), multiplier=a["multiplier"], rshift=a["rshift"])
            h = C.c_void_p()
            L.check(lib.b200q_conv2d_dev_create(C.byref(cop.desc), _P(w), _P(b), C.byref(h)))
            self._handles.append(h)
            self._keep.append(cop)
            self._status.append((op["name"], h))
            xl = L.LAYOUT_NHWC if op["inputs"][0] in self._nhwc else L.LAYOUT_NCHW
            yl = L.LAYOUT_NHWC if op["name"] in self._nhwc else L.LAYOUT_NCHW
            fz = self._fuse_into.get(op["name"])
            if fz is not None and lib.b200q_conv2d_dev_route(h) == 0:      # the CUDA-core route does not fuse
                del self._fused_adds[fz["add"]["name"]]
                del self._fuse_into[op["name"]]
                fz = None
            if fz is not None:
                add, si = fz["add"], fz["self_index"]
                aa = add["attrs"]
                res = self.tensors[fz["other"]]
                fa = L.FusedAdd(residual=res.data_ptr(), residual_dtype=_DT[self._info(fz["other"])["dtype"]],
                                conv_multiplier=int(aa["multipliers"][si]), conv_rshift=int(aa["rshifts"][si]),
                                residual_multiplier=int(aa["multipliers"][1 - si]), residual_rshift=int(aa["rshifts"][1 - si]),
                                do_relu=int(bool(aa.get("do_relu", False))), out_dtype=_DT[self._info(add["name"])["dtype"]])
                self._keep.append(fa)
                add_out = self.tensors[add["name"]]
                return lambda: L.check(lib.b200q_conv2d_dev_run_add(h, _P(ins[0]), xl, _P(add_out), yl, C.byref(fa), stream()))
            if self.channels_last:
                return lambda: L.check(lib.b200q_conv2d_dev_run_layout(h, _P(ins[0]), xl, _P(out), yl, stream()))
            return lambda: L.check(lib.b200q_conv2d_dev_run(h, _P(ins[0]), _P(out), stream()))
        if t == "tpu.Deconv":
            # tpu.Deconv with 8-bit tensors (lib/Dialect/Tpu/Interfaces/Common/Deconv.cpp:95-150) the way the reference's own
            # zero-point route computes it (lib/Support/Dnnl/Deconv.cpp:17-46,:95-110 with pad_tensor_for_deconv, MathUtils.cpp:673-705):
            # the input is spread by the strides into a buffer filled with the input zero point, then convolved at stride 1
            # with the filter turned by 180 degrees, on the INT8 convolution kernel.  ReLU acts on the accumulator there
            # (a library post-op), here after the requantisation, which is the same while no multiplier is negative.
            from .ops import Conv2DOp
            name = op["name"]
            w = self.weights[name + "_filter"]
            b = self.weights.get(name + "_bias")
            n, ic, ih, iw = iinfo[0]["shape"]
            kh, kw = a["kernel_shape"]
            sh, sw = a.get("strides", [1, 1])
            dh, dw = a.get("dilations", [1, 1])
            pt, pl, pb, pr = a.get("pads", [0, 0, 0, 0])
            oph, opw = a.get("output_padding", [0, 0])
            izp = int(iinfo[0].get("zp", 0))
            if iinfo[0]["dtype"] not in ("i8", "u8") or oinfo["dtype"] != "i8" or op["inputs"][0] in self._nhwc or name in self._nhwc:
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{name}: tpu.Deconv takes an 8-bit NCHW tensor and writes int8 (the reference saturates to int8)")
            if izp != 0 and (dh != 1 or dw != 1):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{name}: a dilated tpu.Deconv with an input zero point is not implemented")
            top_, left, bot, right = dh * (kh - 1) - pt, dw * (kw - 1) - pl, dh * (kh - 1) - pb + oph, dw * (kw - 1) - pr + opw
            if min(top_, left, bot, right) < 0:
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{name}: tpu.Deconv pads larger than the dilated kernel are not implemented")
            if a.get("do_relu", False) and any(int(m) < 0 for m in a["multiplier"]):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{name}: tpu.Deconv with do_relu and a negative multiplier is not implemented")
            hs, ws = (ih - 1) * sh + 1 + top_ + bot, (iw - 1) * sw + 1 + left + right
            stage = self.torch.full((n, ic, hs, ws), izp, dtype=ins[0].dtype, device=self.device)
            spread = L.RemapDesc(dims=(C.c_int64 * 6)(1, 1, n, ic, ih, iw), src_stride=(C.c_int64 * 6)(0, 0, ic * ih * iw, ih * iw, iw, 1),
                                 mul=(C.c_int64 * 6)(*[1] * 6), div=(C.c_int64 * 6)(*[1] * 6), mod=(C.c_int64 * 6)(*[0] * 6),
                                 off=(C.c_int64 * 6)(*[0] * 6), extent=(C.c_int64 * 6)(1, 1, n, ic, ih, iw),
                                 dst_stride=(C.c_int64 * 6)(0, 0, ic * hs * ws, hs * ws, sh * ws, sw), dst_offset=top_ * ws + left)
            w_rot = w.flip(2, 3).contiguous()
            cop = Conv2DOp(input_shape=(n, ic, hs, ws), oc=w.shape[0], kernel_shape=(kh, kw), strides=(1, 1), dilations=(dh, dw),
                           pads=(0, 0, 0, 0), group=a.get("group", 1), with_bias=b is not None, do_relu=bool(a.get("do_relu", False)),
                           input_dtype=_DT[iinfo[0]["dtype"]], out_dtype=_DT[oinfo["dtype"]],
                           quant_mode=_QM[a.get("quant_mode", "MultiplierShift")], out_zp=int(oinfo.get("zp", 0)),
                           multiplier=a["multiplier"], rshift=a["rshift"])
            if tuple(cop.out_shape) != tuple(oinfo["shape"]):
                raise L.B200QError(L.ERR_INVALID, f"{name}: output shape {oinfo['shape']} does not match the deconvolution ({cop.out_shape})")
            h = C.c_void_p()
            L.check(lib.b200q_conv2d_dev_create(C.byref(cop.desc), _P(w_rot), _P(b), C.byref(h)))
            self._handles.append(h)
            self._keep.append((cop, stage, spread, w_rot))
            self._status.append((name, h))
            eb = ins[0].element_size()

            def run_deconv():
                L.check(lib.b200q_remap_dev(_P(ins[0]), _P(stage), eb, C.byref(spread), None, stream()))
                L.check(lib.b200q_conv2d_dev_run(h, _P(stage), _P(out), stream()))
            return run_deconv
        if t == "tpu.MatMul":
            # What the reference reads from the op (MatMul.cpp:24-135,:636-728): anything this plan does not honour is
            # refused, never computed differently.
            qmode = a.get("quant_mode", "MultiplierShift")
            if a.get("hdim_is_batch", False):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: tpu.MatMul with hdim_is_batch is not implemented")
            lt, ot = bool(a.get("left_transpose", False)), bool(a.get("output_transpose", False))
            if (lt or ot) and (int(np.prod(iinfo[0]["shape"][:-2])) != 1 or len(iinfo[0]["shape"]) < 2):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: the executor takes left/output transposes of 2-D operands only")
            izp, rzp = int(a.get("input_zp", 0)), int(a.get("right_zp", 0))   # the op's attributes (MatMul.cpp:30-33), subtracted first
            w = self.weights[op["name"] + "_filter"]
            w_nk = w.contiguous() if a.get("right_transpose", False) else w.t().contiguous()   # right operand K-major
            b = self.weights.get(op["name"] + "_bias")
            N, K = w_nk.shape
            # left_transpose: the input is stored [K, M]; output_transpose: the output is stored [N, M]
            # (MatMul.cpp:24-135, lib/Support/Dnnl/MatMul.cpp:182-186,:229-238)
            M = int(iinfo[0]["shape"][-1]) if lt else int(np.prod(iinfo[0]["shape"][:-1]))
            mults, shifts = [int(v) for v in a["multipliers"]], [int(v) for v in a["rshifts"]]
            fuse_rq = bool(a.get("fuse_rq", False))
            if qmode == "MultiplierShift" and fuse_rq:
                # per-channel multipliers arrive as the float `multi` operand, one common shift (MatMul.cpp:709-716)
                multi = self.weights[op["name"] + "_multi"].to(self.torch.float32).to(self.torch.int64)
                mult = multi.to(self.torch.int32).contiguous()
                shift = self.torch.full((N,), shifts[0], dtype=self.torch.int32, device=self.device)
                dialect, rmode, per_channel = L.RQ_MULTIPLIER_SHIFT, L.ROUND_HALF_UP, 1
            elif qmode == "MultiplierShift":
                mult = self.torch.tensor([mults[0]], dtype=self.torch.int32, device=self.device)
                shift = self.torch.tensor([shifts[0]], dtype=self.torch.int32, device=self.device)
                dialect, rmode, per_channel = L.RQ_MULTIPLIER_SHIFT, L.ROUND_HALF_UP, 0
            elif qmode in ("TFLite", "TFLite_LShift"):
                # MultiplyByQuantizedMultiplier(acc, multiplier, -rshift), half away from zero (MatMul.cpp:696-707)
                mult = self.torch.tensor([mults[0]], dtype=self.torch.int32, device=self.device)
                shift = self.torch.tensor([-shifts[0]], dtype=self.torch.int32, device=self.device)
                dialect, rmode, per_channel = L.RQ_QDM, L.ROUND_HALF_AWAY_FROM_ZERO, 0
            else:
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: tpu.MatMul quant_mode {qmode} is not implemented by the executor")
            e = L.Epilogue(dialect=dialect, round_mode=rmode, per_channel=per_channel,
                           out_zp=int(oinfo.get("zp", 0)), relu=L.RELU_BEFORE_REQUANT if a.get("do_relu") else L.RELU_NONE,
                           out_dtype=_DT[oinfo["dtype"]], scale=0.0, bias=b.data_ptr() if b is not None else None,
                           multiplier=mult.data_ptr(), shift=shift.data_ptr())
            status = self.torch.zeros(1, dtype=self.torch.int32, device=self.device)
            self._keep += [w_nk, mult, shift, e, status]
            self._status.append((op["name"], status))
            if lt or ot:
                def run_transposed():
                    x_mk = ins[0].reshape(K, M).t().contiguous() if lt else ins[0]
                    y_mn = self.torch.empty((M, N), dtype=out.dtype, device=self.device) if ot else out
                    L.check(lib.b200q_gemm_i8_zp_dev(_P(x_mk), _DT[iinfo[0]["dtype"]], _P(w_nk), L.DT_I8, M, N, K, izp, rzp, C.byref(e),
                                                     _P(y_mn), _P(status), L.ALGO_AUTO, stream()))
                    if ot:
                        out.copy_(y_mn.t().reshape(out.shape))
                return run_transposed
            return lambda: L.check(lib.b200q_gemm_i8_zp_dev(_P(ins[0]), _DT[iinfo[0]["dtype"]], _P(w_nk), L.DT_I8, M, N, K, izp, rzp,
                                                            C.byref(e), _P(out), _P(status), L.ALGO_AUTO, stream()))
        if t == "tpu.Add":
            if op["name"] in self._fused_adds:      # computed by the producing convolution's kernel
                return lambda: None
            m, s = a["multipliers"], a["rshifts"]
            n = out.numel()
            return lambda: L.check(lib.b200q_add_i8_dev(_P(ins[0]), _DT[iinfo[0]["dtype"]], _P(ins[1]), _DT[iinfo[1]["dtype"]],
                                                        n, int(m[0]), int(s[0]), int(m[1]), int(s[1]),
                                                        int(bool(a.get("do_relu", False))), _DT[oinfo["dtype"]], _P(out),
                                                        stream()))
        if t == "tpu.Reduce":
            # int8 form (Reduce.cpp:101-214): the reduction runs on the float-stored integers exactly as the f32 form does (mean =
            # sum * float(1 / n)), the result is cut to an integer toward zero, multiplied and shifted half-up, and saturated to
            # int8 (to_int8, whatever the output's signedness) - unless multiplier 1 and shift 0, which leave it as it is
            if iinfo[0]["dtype"] not in ("i8", "u8") or oinfo["dtype"] != "i8" or op["inputs"][0] in self._nhwc or op["name"] in self._nhwc:
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: tpu.Reduce takes f32 tensors, or 8-bit NCHW ones with an int8 result")
            modes = {"ReduceMean": 7, "ReduceSum": 1, "ReduceMax": 2, "ReduceMin": 3, "ReduceProd": 4, "ReduceL2": 5, "ReduceL1": 6}
            shape = list(iinfo[0]["shape"])
            axes = sorted(int(v) + (len(shape) if int(v) < 0 else 0) for v in a["axes"])
            if a["mode"] not in modes or any(axes[i] + 1 != axes[i + 1] for i in range(len(axes) - 1)):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: tpu.Reduce over one run of adjacent axes only")
            outer, ax = int(np.prod(shape[:axes[0]])), int(np.prod(shape[axes[0]:axes[-1] + 1]))
            inner = int(np.prod(shape[axes[-1] + 1:]))
            mu = int((a.get("multiplier") or [1])[0])
            sh = int((a.get("rshift") or [0])[0])
            plain = mu == 1 and sh == 0
            if plain and a["mode"] not in ("ReduceMax", "ReduceMin"):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: an unscaled integer {a['mode']} leaves the 8-bit range in the reference")
            torch = self.torch
            xf = torch.empty(ins[0].numel(), dtype=torch.float32, device=self.device)
            rf = torch.empty(out.numel(), dtype=torch.float32, device=self.device)
            ri = torch.empty(out.numel(), dtype=torch.int32, device=self.device)
            tab = torch.tensor([mu, sh, 0], dtype=torch.int32, device=self.device)
            self._keep.append((xf, rf, ri, tab))
            mode, nin, nout, idt = modes[a["mode"]], ins[0].numel(), out.numel(), _DT[iinfo[0]["dtype"]]

            def run_reduce():
                L.check(lib.b200q_cast_q8_to_f32_dev(_P(ins[0]), idt, nin, 1.0, 0, _P(xf), stream()))
                L.check(lib.b200q_top_reduce_f32_dev(mode, _P(xf), _P(rf), outer, ax, inner, stream()))
                L.check(lib.b200q_top_cast_f32_dev(_P(rf), nout, L.DT_I32, L.ROUND_TOWARDS_ZERO, L.DT_I32, _P(ri), stream()))
                L.check(lib.b200q_requant_int_axis_dev(_P(ri), nout, 1, 1, _P(tab[0:1]), _P(tab[1:2]), _P(tab[2:3]), L.RQ_MULTIPLIER_SHIFT,
                                                       L.ROUND_HALF_UP, 0, L.DT_I8, _P(out), stream()))
            return run_reduce
        if t in ("tpu.MaxConst", "tpu.MinConst", "tpu.SubConst"):
            # 8-bit forms (MaxConst.cpp:27-42, SubConst.cpp:26-112); the f32 forms went to the Top arithmetic above
            if iinfo[0]["dtype"] not in ("i8", "u8") or oinfo["dtype"] not in ("i8", "u8"):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: {t} takes f32 or 8-bit tensors")
            if (op["inputs"][0] in self._nhwc) != (op["name"] in self._nhwc):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: {t} between differently stored tensors")
            sub = t == "tpu.SubConst"
            if sub and (int(iinfo[0].get("zp", 0)) != 0 or int(oinfo.get("zp", 0)) != 0):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: asymmetric tpu.SubConst is not implemented")
            form = (3 if a.get("is_reverse", False) else 2) if sub else (0 if t == "tpu.MaxConst" else 1)
            n, mu, sft, cv = out.numel(), int(a.get("multiplier", 1)), int(a.get("rshift", 0)), float(a["const_val"])
            izp = 0 if sub else int(iinfo[0].get("zp", 0))
            relu, limit = int(bool(a.get("do_relu", False))), float(a.get("relu_limit", -1.0))
            return lambda: L.check(lib.b200q_constop_i8_dev(form, _P(ins[0]), _DT[iinfo[0]["dtype"]], n, mu, cv, sft, izp, relu, limit,
                                                            _DT[oinfo["dtype"]], _P(out), stream()))
        if t == "tpu.Sub":
            # 8-bit symmetric form (Sub.cpp:88-113; the f32 form went to the Top arithmetic above).  The reference re-binds its
            # operands in order on this route whatever is_reverse says; a reversed op is refused rather than guessed at.
            if a.get("is_reverse", False) or any(i["dtype"] not in ("i8", "u8") for i in iinfo) or oinfo["dtype"] not in ("i8", "u8"):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: tpu.Sub takes f32 tensors, or 8-bit ones without is_reverse")
            if any(nm in self._nhwc for nm in list(op["inputs"]) + [op["name"]]):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: tpu.Sub on channels-last stored tensors")
            m, s = a["multipliers"], a["rshifts"]
            n = out.numel()
            return lambda: L.check(lib.b200q_sub_i8_dev(_P(ins[0]), _DT[iinfo[0]["dtype"]], _P(ins[1]), _DT[iinfo[1]["dtype"]],
                                                        n, int(m[0]), int(s[0]), int(m[1]), int(s[1]),
                                                        int(bool(a.get("do_relu", False))), _DT[oinfo["dtype"]], _P(out), stream()))
        if t == "tpu.Pool2D":
            nb, c, ih, iw = iinfo[0]["shape"]
            kh, kw = a["kernel_shape"]
            sh, sw = a.get("strides", [1, 1])
            pht, pwl, phb, pwr = a.get("pads", [0, 0, 0, 0])
            is_avg = a["pool_mode"] == "Avg"
            if op["inputs"][0] in self._nhwc:
                return lambda: L.check(lib.b200q_pool2d_i8_nhwc_dev(
                    _P(ins[0]), _DT[iinfo[0]["dtype"]], nb, c, ih, iw, kh, kw, sh, sw, pht, phb, pwl, pwr, int(is_avg),
                    int(a.get("multiplier", 1)), int(a.get("rshift", 0)), int(bool(a.get("do_relu", False))),
                    _DT[oinfo["dtype"]], _P(out), stream()))
            return lambda: L.check(lib.b200q_pool2d_i8_dev(_P(ins[0]), _DT[iinfo[0]["dtype"]], nb * c, ih, iw, kh, kw, sh, sw,
                                                           pht, phb, pwl, pwr, int(is_avg), int(a.get("multiplier", 1)),
                                                           int(a.get("rshift", 0)), int(bool(a.get("do_relu", False))),
                                                           _DT[oinfo["dtype"]], _P(out), stream()))
        if t == "tpu.Lut":
            table = self.weights[op["name"] + "_table"]      # 256 entries in the output's storage type
            n = out.numel()
            return lambda: L.check(lib.b200q_lut_dev(_P(ins[0]), n, _P(table), _DT[oinfo["dtype"]], _P(out), stream()))
        if t == "tpu.MulShift":
            n = out.numel()
            return lambda: L.check(lib.b200q_mulshift_i8_dev(_P(ins[0]), _DT[iinfo[0]["dtype"]], n, int(a["multiplier"]),
                                                             int(a["rshift"]), int(iinfo[0].get("zp", 0)),
                                                             int(oinfo.get("zp", 0)), _DT[oinfo["dtype"]], _P(out), stream()))
        if t == "tpu.Relu":
            if float(a.get("relu_limit", -1.0)) > 0:
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: tpu.Relu with a limit is not implemented")
            n = out.numel()
            if iinfo[0]["dtype"] == "f32":
                return lambda: L.check(lib.b200q_top_relu_f32_dev(_P(ins[0]), _P(out), n, -1.0, stream()))
            # function_relu on integer storage (MathUtils.cpp:891-903): max(x, 0), saturated to the output type
            return lambda: L.check(lib.b200q_addconst_i8_dev(_P(ins[0]), _DT[iinfo[0]["dtype"]], n, 1, 0.0, 0, 0, 1,
                                                             _DT[oinfo["dtype"]], _P(out), stream()))
        if t in ("tpu.AddConst", "tpu.MulConst"):
            n = out.numel()
            cv = float(a.get("const_val", 0.0)) if t == "tpu.AddConst" else 0.0
            izp = int(iinfo[0].get("zp", 0)) if t == "tpu.AddConst" else 0
            if t == "tpu.MulConst" and (int(iinfo[0].get("zp", 0)) != 0 or int(oinfo.get("zp", 0)) != 0):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: asymmetric tpu.MulConst is not implemented")
            return lambda: L.check(lib.b200q_addconst_i8_dev(_P(ins[0]), _DT[iinfo[0]["dtype"]], n, int(a["multiplier"]), cv,
                                                             int(a["rshift"]), izp, int(bool(a.get("do_relu", False))),
                                                             _DT[oinfo["dtype"]], _P(out), stream()))
        if t == "tpu.Mul":
            if tuple(iinfo[0]["shape"]) != tuple(iinfo[1]["shape"]):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: tpu.Mul with broadcasting is not implemented")
            n = out.numel()
            return lambda: L.check(lib.b200q_mul_i8_dev(_P(ins[0]), _DT[iinfo[0]["dtype"]], _P(ins[1]), _DT[iinfo[1]["dtype"]],
                                                        n, int(a["multiplier"]), int(a["rshift"]),
                                                        int(bool(a.get("do_relu", False))), _DT[oinfo["dtype"]], _P(out),
                                                        stream()))
        if t == "tpu.Reshape":
            if op["inputs"][0] in self._nhwc:
                return lambda: out.copy_(ins[0].permute(0, 3, 1, 2).reshape(out.shape))
            return lambda: out.copy_(ins[0].reshape(out.shape))
        raise L.B200QError(L.ERR_UNSUPPORTED, f"op type {t} is not implemented by the executor")

    def _strides(self, name):
        """Element strides of tensor `name` in its graph (NCHW) index order, whatever its storage order."""
        shape = list(self._info(name)["shape"])
        if name in self._nhwc:
            n, c, h, w = shape
            return [h * w * c, 1, w * c, c]
        st, acc = [], 1
        for d in reversed(shape):
            st.insert(0, acc)
            acc *= d
        return st

    def _plan_broadcast(self, op, stream) -> Callable:
        """A binary op whose operands broadcast (numpy rules, as the reference's binary ops do through their library call):
        the smaller operand is expanded to the output's shape by the index-mapping kernel (stride 0 along the broadcast
        dimensions), then the op's equal-shape kernel runs."""
        name, lib = op["name"], self.lib
        oshape = list(self._info(name)["shape"])
        r = len(oshape)
        if r > 6 or name in self._nhwc:
            raise L.B200QError(L.ERR_UNSUPPORTED, f"{name}: broadcasting {op['type']} takes NCHW tensors of at most six dimensions")
        runs, new_inputs = [], []
        for k, nm in enumerate(op["inputs"]):
            ish = list(self._info(nm)["shape"])
            if ish == oshape:
                new_inputs.append(nm)
                continue
            ish = [1] * (r - len(ish)) + ish
            if nm in self._nhwc or len(ish) != r or any(d not in (1, o) for d, o in zip(ish, oshape)):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{name}: operand {nm} {ish} does not broadcast to {oshape}")
            syn = f"{name}__operand{k}"
            self._extra_info[syn] = dict(self._info(nm), shape=oshape)
            src = self.tensors[nm]
            self.tensors[syn] = self.torch.empty(oshape, dtype=src.dtype, device=self.device)
            sstr, acc = [], 1
            for d in reversed(ish):
                sstr.insert(0, 0 if d == 1 else acc)
                acc *= d
            ostr, acc = [], 1
            for d in reversed(oshape):
                ostr.insert(0, acc)
                acc *= d
            pad6 = lambda v, fill: (C.c_int64 * 6)(*([fill] * (6 - r) + [int(x) for x in v]))  # noqa: E731
            d_ = L.RemapDesc(dims=pad6(oshape, 1), src_stride=pad6(sstr, 0), mul=pad6([1] * r, 1), div=pad6([1] * r, 1), mod=pad6([0] * r, 0),
                             off=pad6([0] * r, 0), extent=pad6(oshape, 1), dst_stride=pad6(ostr, 0), dst_offset=0)
            runs.append((nm, syn, d_, src.element_size()))
            new_inputs.append(syn)
        inner = self._plan(dict(op, inputs=new_inputs))
        self._keep.append(runs)

        def run():
            for nm, syn, d_, eb in runs:
                L.check(lib.b200q_remap_dev(_P(self.tensors[nm]), _P(self.tensors[syn]), eb, C.byref(d_), None, stream()))
            inner()
        return run

    def _plan_move(self, op, stream) -> Callable:
        """Slice, Permute, Tile, Upsample, Pad, Concat, Squeeze, Unsqueeze of either dialect: pure data movement, one index
        mapping kernel per input (lib/Dialect/Top/Interfaces/{Slice,Permute,Tile,Upsample,Pad,Concat}.cpp; the Tpu-dialect
        ops move the stored values the same way)."""
        t, a, lib = op["type"].split(".", 1)[-1], op.get("attrs", {}), self.lib
        name, srcs = op["name"], op["inputs"]
        out = self.tensors[name]
        oshape = list(self._info(name)["shape"])
        odt = self._info(name)["dtype"]
        if name in self._nhwc:
            raise L.B200QError(L.ERR_UNSUPPORTED, f"{name}: data-movement ops write NCHW tensors")
        if any(self._info(sn)["dtype"] != odt for sn in srcs):
            raise L.B200QError(L.ERR_UNSUPPORTED, f"{name}: {op['type']} moves values of one storage type")
        if bool(a.get("do_relu", False)) and not (odt == "f32" and t in ("Upsample", "Concat")):
            raise L.B200QError(L.ERR_UNSUPPORTED, f"{name}: do_relu on {op['type']} is implemented for f32 Upsample / Concat only")
        ebytes = out.element_size()
        ostr, acc = [], 1
        for d in reversed(oshape):
            ostr.insert(0, acc)
            acc *= d

        def desc(dims, sstr, mul, div, mod, off, ext, dstr, doff=0):
            r = len(dims)
            if r > 6:
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{name}: more than six dimensions")
            padn = 6 - r
            f = lambda v, fill: (C.c_int64 * 6)(*([fill] * padn + [int(x) for x in v]))  # noqa: E731
            return L.RemapDesc(dims=f(dims, 1), src_stride=f(sstr, 0), mul=f(mul, 1), div=f(div, 1), mod=f(mod, 0), off=f(off, 0),
                               extent=f(ext, 1), dst_stride=f(dstr, 0), dst_offset=int(doff))

        runs, pre = [], []
        pad_buf = None
        ishape = list(self._info(srcs[0])["shape"])
        istr = self._strides(srcs[0])
        r = len(oshape)
        ones, zeros = [1] * r, [0] * r
        if t in ("Squeeze", "Unsqueeze"):
            src = self.tensors[srcs[0]]
            if srcs[0] in self._nhwc:
                return lambda: out.copy_(src.permute(0, 3, 1, 2).reshape(out.shape))
            return lambda: out.copy_(src.reshape(out.shape))
        if t == "Slice":
            off = list(a.get("offset", zeros)) + [0] * (r - len(a.get("offset", zeros)))
            steps = list(a.get("steps", ones)) + [1] * (r - len(a.get("steps", ones)))
            off = [o + ishape[i] if o < 0 else o for i, o in enumerate(off)]
            runs.append((srcs[0], desc(oshape, istr, steps, ones, zeros, off, ishape, ostr)))
        elif t == "Permute":
            order = list(a["order"])
            runs.append((srcs[0], desc(oshape, [istr[o] for o in order], ones, ones, zeros, zeros, [ishape[o] for o in order], ostr)))
        elif t == "Tile":
            runs.append((srcs[0], desc(oshape, istr, ones, ones, ishape, zeros, ishape, ostr)))
        elif t == "Upsample":
            div = [1] * (r - 2) + [int(a.get("scale_h", 1)), int(a.get("scale_w", 1))]
            runs.append((srcs[0], desc(oshape, istr, ones, div, zeros, zeros, ishape, ostr)))
        elif t == "Pad":
            mode = str(a.get("mode", "constant"))
            pads = list(a["paddings"])
            if len(pads) != 2 * r:
                raise L.B200QError(L.ERR_INVALID, f"{name}: paddings must hold 2 x rank values")
            if mode in ("reflect", "edge"):
                # Pad.cpp:72-160: the last two dimensions only; reflect mirrors about the edge element without repeating it,
                # edge repeats it.  Each padded dimension is three pieces (before, body, after), each piece one linear map.
                if r < 2 or any(pads[i] != 0 or pads[r + i] != 0 for i in range(r - 2)) or any(v < 0 for v in pads):
                    raise L.B200QError(L.ERR_UNSUPPORTED, f"{name}: Pad mode {mode} pads the last two dimensions, by non-negative amounts")
                if mode == "reflect" and any(pads[i] >= ishape[i] or pads[r + i] >= ishape[i] for i in (r - 2, r - 1)):
                    raise L.B200QError(L.ERR_INVALID, f"{name}: a reflecting pad must be smaller than the dimension")

                def pieces(n_, pb, pe):      # (count, mul, off, first output index)
                    if mode == "reflect":
                        return [(pb, -1, pb, 0), (n_, 1, 0, pb), (pe, -1, n_ - 2, pb + n_)]
                    return [(pb, 0, 0, 0), (n_, 1, 0, pb), (pe, 0, n_ - 1, pb + n_)]
                for ph_ in pieces(ishape[r - 2], pads[r - 2], pads[2 * r - 2]):
                    for pw_ in pieces(ishape[r - 1], pads[r - 1], pads[2 * r - 1]):
                        if ph_[0] == 0 or pw_[0] == 0:
                            continue
                        dims_ = ishape[:r - 2] + [ph_[0], pw_[0]]
                        mul_ = [1] * (r - 2) + [ph_[1], pw_[1]]
                        off_ = [0] * (r - 2) + [ph_[2], pw_[2]]
                        runs.append((srcs[0], desc(dims_, istr, mul_, ones, zeros, off_, ishape, ostr, ph_[3] * ostr[r - 2] + pw_[3] * ostr[r - 1])))
            elif mode != "constant":
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{name}: Pad mode {mode} is not implemented (the reference has none for it either)")
            else:
                pad_buf = self.torch.tensor([a.get("val", 0.0)]).to(out.dtype).to(self.device)      # the pad value in the storage type
                runs.append((srcs[0], desc(oshape, istr, ones, ones, zeros, [-p for p in pads[:r]], ishape, ostr)))
        elif t == "SwapDimInner":
            # SwapDimInner.cpp:17-46 with swap_dim_data (lib/Support/MathUtils.cpp:1539-1564): every axis with an offset is rotated,
            # out[b] = in[(b + offset) % dim]; the two halves of each such axis are one run each
            offs = list(a["offset"]) + [0] * (r - len(a["offset"]))
            axes = [i for i, o in enumerate(offs) if o != 0]
            if any(not 0 < offs[i] <= ishape[i] for i in axes):
                raise L.B200QError(L.ERR_INVALID, f"{name}: SwapDimInner offsets must lie inside their axes")
            for combo in itertools.product((0, 1), repeat=len(axes)):
                dims, off, dstart = list(ishape), [0] * r, [0] * r
                for ax, part in zip(axes, combo):
                    if part == 0:
                        dims[ax], off[ax] = ishape[ax] - offs[ax], offs[ax]
                    else:
                        dims[ax], dstart[ax] = offs[ax], ishape[ax] - offs[ax]
                if all(d > 0 for d in dims):
                    runs.append((srcs[0], desc(dims, istr, ones, ones, zeros, off, ishape, ostr, sum(x * y for x, y in zip(dstart, ostr)))))
        elif t == "Depth2Space":
            # Depth2Space.cpp:19-103: the deep tensor's channel is (new_c, l1, l2) in CRD or (l1, l2, new_c) in DCR order (l1, l2
            # swapped in the channel index when swap_cr), the shallow tensor's pixel is (h * bh + l1, w * bw + l2); either tensor
            # may be NHWC; is_inversed copies the other way.  Every index is linear in (n, new_c, l1, l2, h, w): one remap.
            if srcs[0] in self._nhwc:
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{name}: Depth2Space on a channels-last stored input")
            bh, bw = int(a["block_h"]), int(a["block_w"])
            crd, inv, swap = bool(a.get("is_CRD", False)), bool(a.get("is_inversed", False)), bool(a.get("swap_cr", False))
            in_nchw, out_nchw = bool(a.get("in_is_NCHW", True)), bool(a.get("out_is_NCHW", True))

            def nchw(shape, is_nchw):
                return (shape[0], shape[1], shape[2], shape[3]) if is_nchw else (shape[0], shape[3], shape[1], shape[2])

            def strides(c, h, w, is_nchw):     # (n, c, h, w) element strides
                return (c * h * w, h * w, w, 1) if is_nchw else (c * h * w, 1, w * c, c)
            n_, ic, ih, iw = nchw(ishape, in_nchw)
            _, oc, oh, ow = nchw(oshape, out_nchw)
            sn, sc_, sh_, sw_ = strides(ic, ih, iw, in_nchw)
            dn, dc, dh, dw = strides(oc, oh, ow, out_nchw)
            if inv:   # the "input" of the formulas is the op's output and the copy runs backwards
                ic, oc, ih, oh, iw, ow = oc, ic, oh, ih, ow, iw
                (sn, sc_, sh_, sw_), (dn, dc, dh, dw) = (dn, dc, dh, dw), (sn, sc_, sh_, sw_)
            if ic != oc * bh * bw:
                raise L.B200QError(L.ERR_INVALID, f"{name}: Depth2Space shapes do not match the block")
            cm = 1 if crd else oc                                         # channel step of one unit of `left`
            deep = [sn, (bh * bw if crd else 1) * sc_, (1 if swap else bw) * cm * sc_, (bh if swap else 1) * cm * sc_, sh_, sw_]
            shallow = [dn, dc, dh, dw, bh * dh, bw * dw]
            shallow = [shallow[0], shallow[1], shallow[2], shallow[3], shallow[4], shallow[5]]
            dims6 = [n_, oc, bh, bw, ih, iw]
            big = [1 << 40] * 6
            src_s, dst_s = (shallow, deep) if inv else (deep, shallow)
            runs.append((srcs[0], L.RemapDesc(dims=(C.c_int64 * 6)(*dims6), src_stride=(C.c_int64 * 6)(*src_s), mul=(C.c_int64 * 6)(*[1] * 6),
                                              div=(C.c_int64 * 6)(*[1] * 6), mod=(C.c_int64 * 6)(*[0] * 6), off=(C.c_int64 * 6)(*[0] * 6),
                                              extent=(C.c_int64 * 6)(*big), dst_stride=(C.c_int64 * 6)(*dst_s), dst_offset=0)))
        elif t == "Concat":
            axis = int(a.get("axis", 1))
            axis += r if axis < 0 else 0
            # tpu.Concat's per-input multipliers / rshifts act in the CV18xx interpreter only (Concat.cpp:43-60); for every other
            # chip the reference copies the stored values as they are, and so does this
            mults = [int(m) for m in a.get("multipliers", [])] + [1] * len(srcs)
            rsh = [int(v) for v in a.get("rshifts", [])] + [0] * len(srcs)
            cv18 = str(self.graph.get("chip", "")).lower().startswith("cv18") and odt in ("i8", "u8")
            at = 0
            for k_, sn in enumerate(srcs):
                if cv18 and (mults[k_] != 1 or rsh[k_] != 0):
                    if sn in self._nhwc:
                        raise L.B200QError(L.ERR_UNSUPPORTED, f"{name}: a requantised Concat input stored channels-last")
                    syn = f"{name}__input{k_}"
                    self._extra_info[syn] = dict(self._info(sn))
                    self.tensors[syn] = self.torch.empty_like(self.tensors[sn])
                    pre.append((sn, syn, mults[k_], rsh[k_], self.tensors[sn].numel()))
                    sn = syn
                sshape = list(self._info(sn)["shape"])
                runs.append((sn, desc(sshape, self._strides(sn), ones, ones, zeros, zeros, sshape, ostr, at * ostr[axis])))
                at += sshape[axis]
        else:
            raise L.B200QError(L.ERR_UNSUPPORTED, f"op type {op['type']} is not implemented by the executor")
        self._keep.append((runs, pad_buf))
        relu = bool(a.get("do_relu", False))
        limit = float(a.get("relu_limit", -1.0))
        pad_host = None
        if pad_buf is not None:
            pad_host = pad_buf.cpu().numpy().tobytes()
            self._keep.append(pad_host)

        qdt = _DT.get(odt, 0)

        def run():
            for sn, syn, mu, sh, cnt in pre:      # CV18xx Concat: saturate(RSR(x * m, rshift, half up)) of an input before the copy
                L.check(lib.b200q_mulshift_i8_dev(_P(self.tensors[sn]), qdt, cnt, mu, sh, 0, 0, qdt, _P(self.tensors[syn]), stream()))
            for sn, d in runs:
                L.check(lib.b200q_remap_dev(_P(self.tensors[sn]), _P(out), ebytes, C.byref(d), pad_host, stream()))
            if relu:
                L.check(lib.b200q_top_relu_f32_dev(_P(out), _P(out), out.numel(), limit, stream()))
        return run

    def _plan_gather(self, op, ins, out, iinfo, stream) -> Callable:
        """Gather / GatherElements of either dialect (lib/Dialect/Top/Interfaces/Gather.cpp:17-49, GatherElements.cpp:20-107).  The
        indices are the second input (f32 as the reference's interpreter stores them, or i32) or the weight `<name>_indices`."""
        t, a, lib = op["type"].split(".", 1)[-1], op.get("attrs", {}), self.lib
        name = op["name"]
        if op["inputs"][0] in self._nhwc or name in self._nhwc:
            raise L.B200QError(L.ERR_UNSUPPORTED, f"{name}: {op['type']} on channels-last stored tensors")
        if iinfo[0]["dtype"] != self._info(name)["dtype"]:
            raise L.B200QError(L.ERR_UNSUPPORTED, f"{name}: {op['type']} moves values of one storage type")
        if len(ins) > 1:
            idx, idx_shape, idt = ins[1], list(iinfo[1]["shape"]), iinfo[1]["dtype"]
        else:
            w = self.weights[name + "_indices"]
            idt = "i32" if not w.dtype.is_floating_point else "f32"
            idx = w.to(self.torch.int32 if idt == "i32" else self.torch.float32).contiguous()
            idx_shape = list(w.shape)
            self._keep.append(idx)
        if idt not in ("f32", "i32"):
            raise L.B200QError(L.ERR_UNSUPPORTED, f"{name}: indices must be f32 or i32")
        is_float = int(idt == "f32")
        shape = list(iinfo[0]["shape"])
        ax = int(a.get("axis", 0))
        ax += len(shape) if ax < 0 else 0
        eb = out.element_size()
        if t == "Gather":
            outer, inner = int(np.prod(shape[:ax])), int(np.prod(shape[ax + 1:]))
            nidx = int(np.prod(idx_shape)) if idx_shape else 1
            if out.numel() != outer * nidx * inner:
                raise L.B200QError(L.ERR_INVALID, f"{name}: output shape does not match the gather")
            return lambda: L.check(lib.b200q_gather_dev(_P(ins[0]), eb, _P(idx), is_float, _P(out), outer, shape[ax], nidx, inner, stream()))
        if len(idx_shape) != len(shape) or out.numel() != int(np.prod(idx_shape)):
            raise L.B200QError(L.ERR_INVALID, f"{name}: GatherElements takes indices of the input's rank and an output of their shape")
        ss, ish = (C.c_int64 * len(shape))(*shape), (C.c_int64 * len(shape))(*idx_shape)
        return lambda: L.check(lib.b200q_gather_elements_dev(_P(ins[0]), eb, _P(idx), is_float, _P(out), len(shape), ss, ish, ax, stream()))

    def _plan_top(self, op, ins, out, iinfo, stream) -> Callable:
        """fp32 Top-dialect ops (the float graph a calibration pass and the threshold tuner run): top.Conv, top.MatMul,
        top.Add, top.MaxPool, top.AvgPool, top.Relu, top.Reshape, with the attribute names of TopOps.td."""
        t, a, lib = op["type"], op.get("attrs", {}), self.lib
        limit = float(a.get("relu_limit", -1.0))
        relu = int(bool(a.get("do_relu", False)))
        if any(i["dtype"] != "f32" for i in iinfo) or self._info(op["name"])["dtype"] != "f32":
            raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: Top-dialect ops run on f32 tensors")
        if t == "top.Conv":
            w = self.weights[op["name"] + "_filter"].to(self.torch.float32).contiguous()
            b = self.weights.get(op["name"] + "_bias")
            b = b.to(self.torch.float32).contiguous() if b is not None else None
            n, ic, ih, iw = iinfo[0]["shape"]
            kh, kw = a["kernel_shape"]
            sh, sw = a.get("strides", [1, 1])
            dh, dw = a.get("dilations", [1, 1])
            pht, pwl, phb, pwr = a.get("pads", [0, 0, 0, 0])
            d = L.TopConvDesc(n=n, ic=ic, ih=ih, iw=iw, oc=w.shape[0], kh=kh, kw=kw, sh=sh, sw=sw, dh=dh, dw=dw, pht=pht, phb=phb,
                              pwl=pwl, pwr=pwr, groups=a.get("group", 1), with_bias=int(b is not None), do_relu=relu, relu_limit=limit)
            h = C.c_void_p()
            L.check(lib.b200q_top_conv2d_dev_create(C.byref(d), _P(w), _P(b), C.byref(h)))
            self._top_handles.append(h)
            self._keep.append((w, b))
            return lambda: L.check(lib.b200q_top_conv2d_dev_run(h, _P(ins[0]), _P(out), n, stream()))
        if t == "top.MatMul":
            # top::MatMulOp (lib/Dialect/Top/Interfaces/MatMul.cpp): a weight or a second activation as the right operand, batched
            # over the leading dimensions; right_transpose reads it [.., N, K].  One launch of the fp32 kernel per batch entry.
            if a.get("left_transpose") or a.get("output_transpose") or a.get("hdim_is_batch"):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: top.MatMul with left / output transposes is not implemented")
            rt = bool(a.get("right_transpose", False))
            b = self.weights.get(op["name"] + "_bias")
            b = b.to(self.torch.float32).contiguous() if b is not None else None
            if len(ins) == 1:
                w = self.weights[op["name"] + "_filter"].to(self.torch.float32)
                w = (w.transpose(-1, -2) if rt else w).contiguous()      # [K, N]
                K, N = w.shape[-2], w.shape[-1]
                M = ins[0].numel() // K
                self._keep.append((w, b))
                return lambda: L.check(lib.b200q_top_matmul_f32_dev(_P(ins[0]), _P(w), _P(b), _P(out), M, K, N, relu, limit, stream()))
            ls, rs = list(iinfo[0]["shape"]), list(iinfo[1]["shape"])
            if len(rs) < 2 or len(ls) < 2 or op["inputs"][0] in self._nhwc or op["inputs"][1] in self._nhwc:
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: top.MatMul operands must be NCHW tensors of rank two or more")
            K, N = (rs[-1], rs[-2]) if rt else (rs[-2], rs[-1])
            M = ls[-2]
            rb, lb = int(np.prod(rs[:-2])), int(np.prod(ls[:-2]))
            if ls[-1] != K or rb not in (1, lb):
                raise L.B200QError(L.ERR_INVALID, f"{op['name']}: top.MatMul shapes {ls} x {rs} do not match")
            if rb == 1 and not rt:          # a shared right operand folds the batch into M
                M, lb = M * lb, 1
            right = ins[1]
            # the kernel wants 16-byte aligned operands: a batch entry whose size is not a multiple of four floats is staged
            # through a buffer with a padded pitch
            pad4 = lambda v: (v + 3) // 4 * 4  # noqa: E731
            px, pr, po = pad4(M * K), pad4(K * N), pad4(M * N)
            torch = self.torch
            xs = torch.empty(lb * px, dtype=torch.float32, device=self.device) if px != M * K and lb > 1 else None
            rsb = torch.empty(rb * pr, dtype=torch.float32, device=self.device) if (rt or (pr != K * N and rb > 1)) else None
            os_ = torch.empty(lb * po, dtype=torch.float32, device=self.device) if po != M * N and lb > 1 else None
            self._keep.append((b, xs, rsb, os_))
            xin, yout = ins[0], out

            def run_matmul():
                x0, sx = xin.data_ptr(), M * K
                if xs is not None:
                    xs.view(lb, px)[:, :M * K].copy_(xin.reshape(lb, M * K))
                    x0, sx = xs.data_ptr(), px
                r0, sr = right.data_ptr(), K * N
                if rsb is not None:      # [.., N, K] -> [.., K, N] when transposed, at the padded pitch
                    src = right.reshape(rb, N, K).transpose(1, 2) if rt else right.reshape(rb, K, N)
                    rsb.view(rb, pr)[:, :K * N].view(rb, K, N).copy_(src) if pr == K * N else \
                        rsb.view(rb, pr)[:, :K * N].copy_(src.reshape(rb, K * N))
                    r0, sr = rsb.data_ptr(), pr
                y0, so = yout.data_ptr(), M * N
                if os_ is not None:
                    y0, so = os_.data_ptr(), po
                for i in range(lb):
                    L.check(lib.b200q_top_matmul_f32_dev(C.c_void_p(x0 + 4 * i * sx), C.c_void_p(r0 + 4 * (i if rb > 1 else 0) * sr), _P(b),
                                                         C.c_void_p(y0 + 4 * i * so), M, K, N, relu, limit, stream()))
                if os_ is not None:
                    yout.view(lb, M * N).copy_(os_.view(lb, po)[:, :M * N])
            return run_matmul
        if t == "top.Add":
            if len(ins) != 2 or tuple(iinfo[0]["shape"]) != tuple(iinfo[1]["shape"]):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: top.Add takes two tensors of one shape here")
            n = out.numel()
            return lambda: L.check(lib.b200q_top_add_f32_dev(_P(ins[0]), _P(ins[1]), _P(out), n, relu, limit, stream()))
        if t in ("top.MaxPool", "top.AvgPool"):
            nb, c, ih, iw = iinfo[0]["shape"]
            kh, kw = a["kernel_shape"]
            sh, sw = a.get("strides", [1, 1])
            pht, pwl, phb, pwr = a.get("pads", [0, 0, 0, 0])
            is_max = int(t == "top.MaxPool")
            cip = int(bool(a.get("count_include_pad", False)))
            return lambda: L.check(lib.b200q_top_pool2d_f32_dev(_P(ins[0]), _P(out), nb * c, ih, iw, kh, kw, sh, sw, pht, phb, pwl,
                                                                pwr, is_max, cip, relu, limit, stream()))
        if t == "top.Relu":
            n = out.numel()
            return lambda: L.check(lib.b200q_top_relu_f32_dev(_P(ins[0]), _P(out), n, limit, stream()))
        if t == "top.Reshape":
            return lambda: out.copy_(ins[0].reshape(out.shape))
        n_el = out.numel()
        const_ops = {"top.AddConst": L.TOP_ADD_CONST, "top.MulConst": L.TOP_MUL_CONST, "top.MaxConst": L.TOP_MAX_CONST,
                     "top.MinConst": L.TOP_MIN_CONST}
        if t in const_ops or t == "top.SubConst":
            code = const_ops.get(t, L.TOP_RSUB_CONST if a.get("is_reverse", False) else L.TOP_SUB_CONST)
            cv = float(a["const_val"])
            return lambda: L.check(lib.b200q_top_eltwise_f32_dev(code, _P(ins[0]), None, cv, _P(out), n_el, relu, limit, stream()))
        binary = {"top.Mul": (L.TOP_MUL, L.TOP_MUL), "top.Sub": (L.TOP_SUB, L.TOP_RSUB), "top.Div": (L.TOP_DIV, L.TOP_RDIV)}
        if t in binary:
            if len(ins) != 2 or tuple(iinfo[0]["shape"]) != tuple(iinfo[1]["shape"]):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: {t} takes two tensors of one shape here")
            code = binary[t][1 if a.get("is_reverse", False) else 0]
            return lambda: L.check(lib.b200q_top_eltwise_f32_dev(code, _P(ins[0]), _P(ins[1]), 0.0, _P(out), n_el, relu, limit, stream()))
        unary = {"top.SiLU": L.TOP_SILU, "top.GELU": L.TOP_GELU, "top.Floor": L.TOP_FLOOR}
        if t in unary or t == "top.Sigmoid":
            code = unary.get(t, L.TOP_LOG_SIGMOID if a.get("log", False) else L.TOP_SIGMOID)
            return lambda: L.check(lib.b200q_top_eltwise_f32_dev(code, _P(ins[0]), None, 0.0, _P(out), n_el, 0, -1.0, stream()))
        if t == "top.Reduce":
            modes = {"ReduceMean": 0, "ReduceSum": 1, "ReduceMax": 2, "ReduceMin": 3, "ReduceProd": 4, "ReduceL2": 5, "ReduceL1": 6, "ReduceMeanRcp": 7}
            shape = list(iinfo[0]["shape"])
            axes = sorted(int(x) + (len(shape) if int(x) < 0 else 0) for x in a["axes"])
            if a["mode"] not in modes or any(axes[i] + 1 != axes[i + 1] for i in range(len(axes) - 1)):
                raise L.B200QError(L.ERR_UNSUPPORTED, f"{op['name']}: top.Reduce over one run of adjacent axes only")
            outer, ax = int(np.prod(shape[:axes[0]])), int(np.prod(shape[axes[0]:axes[-1] + 1]))
            inner = int(np.prod(shape[axes[-1] + 1:]))
            mode = modes[a["mode"]]
            return lambda: L.check(lib.b200q_top_reduce_f32_dev(mode, _P(ins[0]), _P(out), outer, ax, inner, stream()))
        if t == "top.Softmax":
            shape = list(iinfo[0]["shape"])
            axis = int(a.get("axis", 1))
            axis += len(shape) if axis < 0 else 0
            outer, ch, inner = int(np.prod(shape[:axis])), shape[axis], int(np.prod(shape[axis + 1:]))
            lg = int(bool(a.get("log", False)))
            return lambda: L.check(lib.b200q_top_softmax_f32_dev(_P(ins[0]), _P(out), outer, ch, inner, lg, stream()))
        if t == "top.LayerNorm":
            shape = list(iinfo[0]["shape"])
            axis = int(a.get("axis", -1))
            axis += len(shape) if axis < 0 else 0
            outer, inner = int(np.prod(shape[:axis])), int(np.prod(shape[axis:]))
            w = self.weights.get(op["name"] + "_weight")
            b = self.weights.get(op["name"] + "_bias")
            w = w.to(self.torch.float32).contiguous() if w is not None else None
            b = b.to(self.torch.float32).contiguous() if b is not None else None
            eps = float(a.get("eps", 1e-5))
            self._keep.append((w, b))
            return lambda: L.check(lib.b200q_top_layernorm_f32_dev(_P(ins[0]), _P(w), _P(b), _P(out), outer, inner, eps, stream()))
        if t == "top.Scale":
            sc = self.weights[op["name"] + "_scale"].to(self.torch.float32).contiguous()
            bi = self.weights[op["name"] + "_bias"].to(self.torch.float32).contiguous()
            shape = list(iinfo[0]["shape"])
            ch = shape[1]
            inner = int(np.prod(shape[2:])) if len(shape) > 2 else 1
            self._keep.append((sc, bi))
            return lambda: L.check(lib.b200q_top_scale_f32_dev(_P(ins[0]), _P(sc), _P(bi), _P(out), shape[0], ch, inner, relu, limit, stream()))
        raise L.B200QError(L.ERR_UNSUPPORTED, f"op type {t} is not implemented by the executor")

    # ------------------------------------------------------------------ pymlir.module surface
    def set_tensor(self, name: str, data, shape=None):
        """Float input of the graph (quantisation happens in the graph's own tpu.Cast, as in a lowered model)."""
        t = self.tensors[name]
        src = self.torch.as_tensor(np.ascontiguousarray(data)) if not isinstance(data, self.torch.Tensor) else data
        if name in self._nhwc:
            n, h, w, c = t.shape
            src = src.reshape(n, c, h, w).permute(0, 2, 3, 1)
        t.copy_(src.reshape(t.shape).to(t.dtype), non_blocking=True)

    def set_tensor_from_int(self, name: str, data, shape=None):
        """``setTensor(..., is_integer=true)`` (ModuleInterpreter.cpp:1313-1362): `data` already holds storage values.
        This executor keeps tensors in their storage type, so integer and float-stored-integer data take one route."""
        self.set_tensor(name, data, shape)

    def before_invoke(self, fn: Callable):
        self._before.append(fn)

    def after_invoke(self, fn: Callable):
        self._after.append(fn)

    def clear_hooks(self):
        self._before, self._after = [], []

    def _capture(self):
        """All ops of the graph as one CUDA graph (every launch of the device face is asynchronous on the current
        stream and allocates nothing).  One eager pass first, so that one-time set-up is not captured."""
        torch = self.torch
        for run in self._plans:
            run()
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for run in self._plans:
                run()
        self._graph = g

    def _run_ops(self, ops_and_plans):
        for op, run in ops_and_plans:
            for fn in self._before:
                fn(op["name"])
            run()
            for fn in self._after:
                fn(op["name"])

    def invoke(self, fixed_to_float: bool = True):
        """Runs every op in graph order.  As in the reference (ModuleInterpreter.cpp:992-1011), ``fixed_to_float``
        decides what ``get_tensor`` returns afterwards for quantized tensors: their expressed float values
        ``(q - zp) * scale`` (True, the default) or the raw storage values (False).  The device tensors themselves
        always keep the storage values."""
        self._expressed = bool(fixed_to_float)
        if self.cuda_graph and not self._before and not self._after:
            if self._graph is None:
                self._capture()
            self._graph.replay()
            return
        self._run_ops(zip(self.graph["ops"], self._plans))

    def invoke_at(self, name: str):
        """One op, with its hooks; returns its output as stored (ModuleInterpreter.cpp:1210-1231)."""
        target = self._fused_adds.get(name, name)      # a fused Add is computed by its convolution's kernel
        for op, run in zip(self.graph["ops"], self._plans):
            if op["name"] == target:
                self._expressed = False
                self._run_ops([(op, run)])
                return self.get_tensor(name)
        raise KeyError(name)

    def invoke_op(self, name: str):
        """invoke_at without the copy to the host: the op's output stays in ``tensors[name]`` on the device."""
        target = self._fused_adds.get(name, name)
        for op, run in zip(self.graph["ops"], self._plans):
            if op["name"] == target:
                self._expressed = False
                self._run_ops([(op, run)])
                return
        raise KeyError(name)

    def invoke_from(self, name: str):
        """Every op from `name` to the end of the graph, with hooks (ModuleInterpreter.cpp:1233-1253)."""
        names = [op["name"] for op in self.graph["ops"]]
        if name not in names:
            raise KeyError(name)
        i = names.index(name)
        self._expressed = False
        self._run_ops(list(zip(self.graph["ops"], self._plans))[i:])

    def fake_quant_weight(self):
        """ModuleInterpreter::fake_quant_weight (ModuleInterpreter.cpp:583-612): every weight except the bias operand
        of a convolution / matmul is rounded to 127 levels of its own absolute maximum,
        ``round(w * 127 / max) * max / 127``; the operators then work from the rewritten weights."""
        torch = self.torch
        for name, w in self.weights.items():
            if name.endswith("_bias"):
                continue
            f = w.to(torch.float32)
            mx = f.abs().max()
            if float(mx) == 0.0:
                continue
            q = torch.round(f * 127 / mx) * mx / 127
            self.weights[name] = q.to(w.dtype) if not w.dtype.is_floating_point else q
        self._build_plans()   # device handles hold repacked copies of the weights

    def check_status(self):
        """Raises B200QError(ERR_TIMEOUT) if a bounded wait inside one of the graph's tensor-core kernels ran out
        during an earlier invoke (the kernel returns early then and its output is not valid)."""
        self.torch.cuda.synchronize(self.device)
        for name, st in self._status:
            if isinstance(st, C.c_void_p):
                rc = self.lib.b200q_conv2d_dev_status(st, None)
                if rc != L.OK:
                    raise L.B200QError(rc, f"{name}: " + self.lib.b200q_last_error().decode("utf-8", "replace"))
            else:
                code = int(st.item())
                if code != 0:
                    st.zero_()
                    raise L.B200QError(L.ERR_TIMEOUT, f"{name}: a bounded wait inside the kernel ran out (wait site {code})")

    def get_tensor(self, name: str) -> np.ndarray:
        """The tensor in the graph's own (NCHW) shape: expressed float values after ``invoke(fixed_to_float=True)``,
        raw storage values (integers for quantized tensors) otherwise.  Reading a tensor is where a kernel-side timeout
        of the preceding run surfaces."""
        self.check_status()
        if self._expressed:
            return self.get_fp32_tensor(name)
        return self._nchw(name).cpu().numpy()

    def get_raw_tensor(self, name: str) -> np.ndarray:
        """Storage values regardless of the last invoke's ``fixed_to_float``."""
        self.check_status()
        return self._nchw(name).cpu().numpy()

    def _nchw(self, name: str):
        if name in self._fuse_into:
            raise L.B200QError(L.ERR_UNSUPPORTED, f"{name} is not materialised: its Add ({self._fuse_into[name]['add']['name']}) runs inside "
                               "the convolution kernel (module(fuse_residual_add=True))")
        t = self.tensors[name]
        return t.permute(0, 3, 1, 2).contiguous() if name in self._nhwc else t

    def get_fp32_tensor(self, name: str) -> np.ndarray:
        """The tensor as the interpreter "expresses" it: (q - zp) * scale (ModuleInterpreter.cpp:992-1011)."""
        info = self._info(name)
        v = self._nchw(name).cpu().numpy()
        if info["dtype"] == "f32":
            return v
        return ((v.astype(np.float32) - np.float32(info.get("zp", 0))) * np.float32(info["scale"])).astype(np.float32)

    def get_all_tensor(self) -> Dict[str, np.ndarray]:
        self.check_status()
        return {n: self.get_fp32_tensor(n) for n in self.all_tensor_names if n not in self._fuse_into}

    def get_tensor_qinfo(self, name: str):
        info = self._info(name)
        return info["dtype"], float(info.get("scale", 1.0)), int(info.get("zp", 0))
