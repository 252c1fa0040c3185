"""Reader (and writer) for the textual subset of MLIR that a lowered tpu-mlir model uses, so that the executor can load
``*_tpu.mlir`` + ``*_weight.npz`` files directly.

The text is MLIR's generic operation form, one op per line (what ``tpuc-opt`` prints; sample:
test/Transforms/Parallel/Conv.mlir:16-25 in the reference tree):

    %2 = "tpu.Conv2D"(%arg0, %0, %1) {dilations = [1, 1], do_relu = false, ..., quant_mode = #tpu<rq_mode MultiplierShift>}
         : (tensor<4x16x100x100xf32>, tensor<..>, tensor<..>) -> tensor<1x65x100x100x!quant.uniform<i8:f32, 0.0646>> loc(#loc4)
    #loc4 = loc("output_Conv")

Tensor names are the ``loc`` strings (that is how the interpreter names tensors, and ``top.Weight`` results name the
arrays of the weight file); element types follow python/mlir_ast/nodes.py:198-231 of the reference
(``f32``, ``i8``/``si8``/``ui8``, ``!quant.uniform<i8:f32, scale[:zp]>``, ``!quant.calibrated<...>``, an optional
``, address : i64`` suffix).  Only a flat ``func.func @main`` is read (module state ``TPU_LOWERED``); subnet-divided
modules with ``func.call`` are rejected.
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np


class MlirTextError(ValueError):
    pass


@dataclass
class TensorType:
    shape: List[int]
    dtype: str                  # "f32", "i8", "u8", "i16", "u16", "i32", "bf16", "f16", "none"
    scale: Optional[float] = None
    zp: int = 0
    address: Optional[int] = None


@dataclass
class Op:
    results: List[str]          # SSA ids
    type: str                   # e.g. "tpu.Conv2D"
    operands: List[str]         # SSA ids
    attrs: Dict[str, object]
    in_types: List[TensorType]
    out_types: List[TensorType]
    loc: str                    # tensor name (first name of a fused loc)


@dataclass
class Module:
    name: str = ""
    attrs: Dict[str, object] = field(default_factory=dict)
    args: List[Tuple[str, TensorType, str]] = field(default_factory=list)   # (ssa id, type, loc name)
    ops: List[Op] = field(default_factory=list)
    returns: List[str] = field(default_factory=list)


# ------------------------------------------------------------------------------------------------ scanning helpers
def _match_close(s: str, i: int) -> int:
    """Index just past the bracket that closes s[i] ('(', '[', '{' or '<'), skipping strings."""
    pairs = {"(": ")", "[": "]", "{": "}", "<": ">"}
    stack = [pairs[s[i]]]
    j = i + 1
    while j < len(s):
        c = s[j]
        if c == '"':
            j = _skip_string(s, j)
            continue
        if c in pairs:
            stack.append(pairs[c])
        elif c == ">" and j > 0 and s[j - 1] == "-":
            pass  # the arrow of a function type
        elif c == stack[-1]:
            stack.pop()
            if not stack:
                return j + 1
        j += 1
    raise MlirTextError("unbalanced brackets: " + s[i:i + 60])


def _skip_string(s: str, i: int) -> int:
    j = i + 1
    while j < len(s):
        if s[j] == "\\":
            j += 2
            continue
        if s[j] == '"':
            return j + 1
        j += 1
    raise MlirTextError("unterminated string")


def _split_top(s: str, sep: str = ",") -> List[str]:
    """Split at separators that are not inside brackets or strings."""
    out, depth, start, j = [], 0, 0, 0
    while j < len(s):
        c = s[j]
        if c == '"':
            j = _skip_string(s, j)
            continue
        if c in "([{<":
            depth += 1
        elif c in ")]}":
            depth -= 1
        elif c == ">" and not (j > 0 and s[j - 1] == "-"):
            depth -= 1
        elif c == sep and depth == 0:
            out.append(s[start:j].strip())
            start = j + 1
        j += 1
    tail = s[start:].strip()
    if tail:
        out.append(tail)
    return out


# ------------------------------------------------------------------------------------------------ types
_STORAGE = {"i8": "i8", "si8": "i8", "ui8": "u8", "u8": "u8", "i16": "i16", "si16": "i16", "ui16": "u16", "u16": "u16",
            "i32": "i32", "si32": "i32", "ui32": "u32", "i4": "i4", "si4": "i4", "ui4": "u4"}


def parse_type(t: str) -> TensorType:
    t = t.strip()
    if t == "none":
        return TensorType([], "none")
    if not t.startswith("tensor<") or not t.endswith(">"):
        raise MlirTextError("not a tensor type: " + t)
    body = t[len("tensor<"):-1]
    address = None
    m = re.search(r",\s*(-?\d+)\s*:\s*i64\s*$", body)
    if m:
        address = int(m.group(1))
        body = body[:m.start()]
    q = body.find("!")
    if q >= 0:
        shape_s, elem = body[:q].rstrip("x"), body[q:].strip()
    else:
        shape_s, elem = body.rsplit("x", 1) if "x" in body else ("", body)
    shape = [int(d) if d not in ("?", "") else -1 for d in shape_s.split("x")] if shape_s else []
    if elem.startswith("!quant.uniform<"):
        inner = elem[len("!quant.uniform<"):-1]
        storage, rest = inner.split(":", 1)
        storage = storage.split("<")[0].strip()                       # drop a storage range like i8<-127:127>
        params = rest.split(",", 1)[1].strip()
        if params.startswith("{"):
            raise MlirTextError("per-axis quantized types are not supported: " + elem)
        sz = params.split(":")
        return TensorType(shape, _STORAGE.get(storage, storage), float(sz[0]), int(sz[1]) if len(sz) > 1 else 0, address)
    if elem.startswith("!quant.calibrated<"):
        return TensorType(shape, elem[len("!quant.calibrated<"):].split("<")[0].strip(), None, 0, address)
    return TensorType(shape, _STORAGE.get(elem, elem), None, 0, address)


def format_type(t: TensorType) -> str:
    if t.dtype == "none":
        return "none"
    dims = "x".join(str(d) for d in t.shape)
    st = {"i8": "i8", "u8": "u8", "i16": "i16", "u16": "u16", "i32": "i32"}.get(t.dtype, t.dtype)
    if t.scale is not None:
        zp = ":%d" % t.zp if t.zp else ""
        elem = "!quant.uniform<%s:f32, %s%s>" % (st, repr(float(t.scale)), zp)
    else:
        elem = {"i8": "si8", "u8": "ui8", "i32": "si32", "i16": "si16", "u16": "ui16"}.get(t.dtype, t.dtype)
    return "tensor<%s%s%s>" % (dims, "x" if dims else "", elem)


# ------------------------------------------------------------------------------------------------ attributes
def parse_attr_value(v: str):
    v = v.strip()
    if v in ("true", "false"):
        return v == "true"
    if v == "unit":
        return True
    if v.startswith('"'):
        return bytes(v[1:_skip_string(v, 0) - 1], "utf-8").decode("unicode_escape")
    if v.startswith("["):
        return [parse_attr_value(e) for e in _split_top(v[1:_match_close(v, 0) - 1])]
    if v.startswith("array<"):
        inner = v[len("array<"):-1]
        return [parse_attr_value(e) for e in _split_top(inner.split(":", 1)[1])] if ":" in inner else []
    if v.startswith("#"):
        m = re.match(r"#[\w.]+<\s*\w+\s+([^>]+)>", v)      # #tpu<rq_mode MultiplierShift> -> "MultiplierShift"
        return m.group(1).strip() if m else v
    m = re.match(r"^(-?[0-9][0-9a-fA-FxX.eE+\-]*|-?inf|nan)\s*(?::\s*([\w<>]+))?$", v)
    if m:
        num = m.group(1)
        if m.group(2) is None or m.group(2)[0] in "iu" or m.group(2) == "index":
            try:
                return int(num, 0)
            except ValueError:
                pass
        return float(num)
    return v  # affine maps, dense<...>, symbol refs: kept as text


def parse_attr_dict(s: str) -> Dict[str, object]:
    s = s.strip()
    if not s:
        return {}
    out = {}
    for item in _split_top(s[1:-1]):
        if "=" in item:
            k, v = item.split("=", 1)
            out[k.strip().strip('"')] = parse_attr_value(v)
        else:
            out[item.strip().strip('"')] = True
    return out


# ------------------------------------------------------------------------------------------------ module
_LOC_DEF = re.compile(r'^\s*(#loc\w*)\s*=\s*loc\((.*)\)\s*$')


def _loc_name(spec: str, table: Dict[str, str]) -> str:
    spec = spec.strip()
    if spec.startswith("#"):
        return table.get(spec, spec)
    if spec.startswith("fused"):
        inner = spec[spec.index("[") + 1:spec.rindex("]")]
        return _loc_name(_split_top(inner)[0], table)
    if spec.startswith('"'):
        return spec[1:_skip_string(spec, 0) - 1]
    return spec  # unknown


def parse_module(text: str) -> Module:
    lines = text.splitlines()
    raw_locs: Dict[str, str] = {}
    for ln in lines:
        m = _LOC_DEF.match(ln)
        if m:
            raw_locs[m.group(1)] = m.group(2)
    locs: Dict[str, str] = {}
    for k, v in raw_locs.items():
        locs[k] = _loc_name(v, {kk: _loc_name(vv, {}) for kk, vv in raw_locs.items()})
    mod = Module()
    funcs = 0
    for ln in lines:
        s = ln.strip()
        if not s or s.startswith("//") or _LOC_DEF.match(ln):
            continue
        if s.startswith("module"):
            m = re.match(r"module\s+@?([\w.\-]*)\s*attributes\s*", s)
            if m and not mod.name:
                mod.name = m.group(1)
                i = s.index("{", m.end() - 1)
                mod.attrs = parse_attr_dict(s[i:_match_close(s, i)])
            continue
        if s.startswith("func.func"):
            funcs += 1
            if funcs > 1:
                raise MlirTextError("subnet-divided modules (several functions / func.call) are not supported; "
                                    "load the model in state TPU_LOWERED")
            i = s.index("(")
            for a in _split_top(s[i + 1:_match_close(s, i) - 1]):
                m = re.match(r"(%\w+)\s*:\s*(.*?)\s*(?:loc\((.*)\))?$", a)
                if not m:
                    raise MlirTextError("cannot read function argument: " + a)
                mod.args.append((m.group(1), parse_type(m.group(2)), _loc_name(m.group(3) or m.group(1), locs)))
            continue
        if s.startswith("return") or s.startswith('"func.return"'):
            mod.returns = re.findall(r"%[\w#]+", s.split(":")[0])
            continue
        if s.startswith("}"):
            continue
        if "func.call" in s:
            raise MlirTextError("func.call is not supported; load the model in state TPU_LOWERED")
        if "=" in s and '"' in s:
            mod.ops.append(_parse_op(s, locs))
    return mod


def _parse_op(s: str, locs: Dict[str, str]) -> Op:
    lhs, rest = s.split("=", 1)
    results = []
    for r in re.findall(r"%[\w]+(?::\d+)?", lhs):
        if ":" in r:
            base, n = r.split(":")
            results += ["%s#%d" % (base, i) for i in range(int(n))]
        else:
            results.append(r)
    rest = rest.strip()
    q1 = rest.index('"')
    q2 = _skip_string(rest, q1)
    name = rest[q1 + 1:q2 - 1]
    i = rest.index("(", q2)
    j = _match_close(rest, i)
    operands = re.findall(r"%[\w]+(?:#\d+)?", rest[i:j])
    k = j
    while rest[k] == " ":
        k += 1
    attrs = {}
    if rest[k] == "{":
        e = _match_close(rest, k)
        attrs = parse_attr_dict(rest[k:e])
        k = e
    if rest[k:].lstrip().startswith("("):      # a region: not used by the supported ops
        raise MlirTextError("operations with regions are not supported: " + name)
    c = rest.index(":", k)
    sig = rest[c + 1:]
    loc = ""
    lm = re.search(r"\sloc\((.*)\)\s*$", sig)
    if lm:
        loc = _loc_name(lm.group(1), locs)
        sig = sig[:lm.start()]
    sig = sig.strip()
    i = sig.index("(")
    j = _match_close(sig, i)
    in_types = [parse_type(t) for t in _split_top(sig[i + 1:j - 1])]
    out_s = sig[j:].strip()
    if not out_s.startswith("->"):
        raise MlirTextError("missing result type: " + s[:80])
    out_s = out_s[2:].strip()
    if out_s.startswith("("):
        out_types = [parse_type(t) for t in _split_top(out_s[1:_match_close(out_s, 0) - 1])]
    else:
        out_types = [parse_type(out_s)]
    return Op(results, name, operands, attrs, in_types, out_types, loc)


# ------------------------------------------------------------------------------------------------ executor graph
_SUPPORTED = {"tpu.Conv2D", "tpu.MatMul", "tpu.Add", "tpu.Pool2D", "tpu.Cast", "tpu.Reshape", "tpu.Lut", "tpu.MulShift",
              "tpu.Mul"}


def _tensor_entry(t: TensorType) -> dict:
    d = dict(shape=list(t.shape), dtype=t.dtype)
    if t.scale is not None:
        d.update(scale=float(t.scale), zp=int(t.zp))
    return d


def to_graph(mod: Module, weight_arrays: Dict[str, np.ndarray]):
    """(graph, weights) in the form ``module.load`` takes.  ``weight_arrays`` is the model's weight file
    (``numpy.load(<module.weight_file>)``), keyed by the loc names of the ``top.Weight`` results."""
    name_of: Dict[str, str] = {}
    kind: Dict[str, str] = {}
    tensors: Dict[str, dict] = {}
    inputs, gops, weights = [], [], {}
    for ssa, t, loc in mod.args:
        name_of[ssa] = loc
    for op in mod.ops:
        for i, r in enumerate(op.results):
            name_of[r] = op.loc if i == 0 else "%s_%d" % (op.loc, i)
        r0 = op.results[0] if op.results else None
        if op.type == "top.None":
            kind[r0] = "none"
        elif op.type == "top.Weight":
            kind[r0] = "weight"
        elif op.type == "top.Input":
            src = name_of[op.operands[0]]
            # the executor's input tensor carries the op's name (set_tensor(name) as with the interpreter)
            name_of[op.operands[0]] = op.loc
            inputs.append(op.loc)
            tensors[op.loc] = _tensor_entry(op.out_types[0])
            name_of[r0] = op.loc
            del src
        elif op.type in _SUPPORTED:
            acts = [o for o in op.operands if kind.get(o) not in ("none", "weight")]
            wts = [o for o in op.operands if kind.get(o) == "weight"]
            attrs = dict(op.attrs)
            if op.type == "tpu.Conv2D":
                names = ["_filter", "_bias"]
            elif op.type == "tpu.MatMul":
                names = ["_filter", "_bias", "_multi"]   # operands: input, right, bias, multi, buffer (TpuOps.td:4592-4616)
            elif op.type == "tpu.Lut":
                names = ["_table"]      # operands: input, table (TpuOps.td LutOp)
            else:
                names = []
            # operand order: input, filter/right, bias (None operands keep their slot)
            for slot, o in enumerate(op.operands[1:]):   # positional: filter / right operand, then bias
                if slot < len(names) and kind.get(o) == "weight":
                    key = name_of[o]
                    if key not in weight_arrays:
                        raise MlirTextError("weight %r is not in the weight file" % key)
                    weights[op.loc + names[slot]] = np.asarray(weight_arrays[key])
            del wts
            if op.type == "tpu.Conv2D" and (op.loc + "_filter") in weights:
                w = weights[op.loc + "_filter"]
                ks = attrs.get("kernel_shape", [1, 1])
                oc = op.out_types[0].shape[1]
                weights[op.loc + "_filter"] = w.reshape(oc, -1, ks[0], ks[1]).astype(np.int8)
                if (op.loc + "_bias") in weights:
                    weights[op.loc + "_bias"] = weights[op.loc + "_bias"].reshape(-1).astype(np.int32)
            if op.type == "tpu.MatMul" and (op.loc + "_filter") in weights:
                w = weights[op.loc + "_filter"]
                weights[op.loc + "_filter"] = w.reshape(w.shape[-2], w.shape[-1]).astype(np.int8)
                if (op.loc + "_bias") in weights:
                    weights[op.loc + "_bias"] = weights[op.loc + "_bias"].reshape(-1).astype(np.int32)
                if (op.loc + "_multi") in weights:   # per-channel multipliers of fuse_rq, float-stored
                    weights[op.loc + "_multi"] = weights[op.loc + "_multi"].reshape(-1).astype(np.float32)
            tensors[op.loc] = _tensor_entry(op.out_types[0])
            gops.append(dict(type=op.type, name=op.loc, inputs=[name_of[o] for o in acts], attrs=attrs))
        else:
            raise MlirTextError("op type %s is not implemented by the executor" % op.type)
    outputs = [name_of[r] for r in mod.returns]
    return dict(inputs=inputs, outputs=outputs, tensors=tensors, ops=gops), weights


def load_mlir(path: str, weight_file: Optional[str] = None):
    """Read ``path`` (and the weight file its module attribute names, relative to it) into (graph, weights)."""
    import os
    with open(path) as f:
        mod = parse_module(f.read())
    wf = weight_file or mod.attrs.get("module.weight_file")
    if not wf:
        raise MlirTextError("the module names no weight file")
    if not os.path.isabs(wf):
        wf = os.path.join(os.path.dirname(os.path.abspath(path)), wf)
    with np.load(wf) as z:
        arrays = {k: z[k] for k in z.files}
    return to_graph(mod, arrays)


# ------------------------------------------------------------------------------------------------ writer
def _fmt_attr(v) -> str:
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, int):
        return "%d : i64" % v
    if isinstance(v, float):
        return "%s : f64" % repr(v)
    if isinstance(v, str):
        if v in ("Max", "Avg"):
            return "#tpu<pool_mode %s>" % v
        if v in ("TFLite_LShift", "TFLite", "MultiplierShift", "OnlyShift", "QDM", "OnlyScale"):
            return "#tpu<rq_mode %s>" % v
        return '"%s"' % v
    if isinstance(v, (list, tuple)):
        return "[" + ", ".join(str(int(e)) if isinstance(e, (int, np.integer)) else repr(float(e)) for e in v) + "]"
    raise MlirTextError("cannot write attribute value %r" % (v,))


def emit_module(graph: dict, weights: Dict[str, np.ndarray], name: str = "model", weight_file: str = "model_weight.npz") -> str:
    """The executor's graph as generic-form MLIR text (state TPU_LOWERED); weights are referenced by name."""
    tens = graph["tensors"]

    def ttype(n):
        t = tens[n]
        return format_type(TensorType(t["shape"], t["dtype"], t.get("scale"), int(t.get("zp", 0))))

    locs: List[str] = []

    def loc(nm):
        locs.append(nm)
        return "loc(#loc%d)" % len(locs)

    lines = []
    args = ", ".join("%%arg%d: %s %s" % (i, ttype(n), loc(n)) for i, n in enumerate(graph["inputs"]))
    rets = ", ".join(ttype(n) for n in graph["outputs"])
    ssa: Dict[str, str] = {}
    body = []
    cnt = 0

    def new():
        nonlocal cnt
        cnt += 1
        return "%%%d" % (cnt - 1)

    for i, n in enumerate(graph["inputs"]):
        r = new()
        body.append('%s = "top.Input"(%%arg%d) : (%s) -> %s %s' % (r, i, ttype(n), ttype(n), loc(n)))
        ssa[n] = r
    none = None
    for op in graph["ops"]:
        operands, types = [ssa[i] for i in op["inputs"]], [ttype(i) for i in op["inputs"]]
        if op["type"] in ("tpu.Conv2D", "tpu.MatMul", "tpu.Lut"):
            suffixes = ("_table",) if op["type"] == "tpu.Lut" else ("_filter", "_bias", "_multi") if op["type"] == "tpu.MatMul" else ("_filter", "_bias")
            for suffix in suffixes:
                key = op["name"] + suffix
                if key in weights:
                    w = weights[key]
                    r = new()
                    wt = format_type(TensorType(list(w.shape), {"int8": "i8", "int32": "i32", "uint8": "u8", "float32": "f32"}[str(w.dtype)]))
                    body.append('%s = "top.Weight"() : () -> %s %s' % (r, wt, loc(key)))
                    operands.append(r)
                    types.append(wt)
                else:
                    if none is None:
                        none = new()
                        body.append('%s = "top.None"() : () -> none %s' % (none, loc("none")))
                    operands.append(none)
                    types.append("none")
        r = new()
        attrs = op.get("attrs", {})
        a = (" {" + ", ".join("%s = %s" % (k, _fmt_attr(attrs[k])) for k in sorted(attrs)) + "}") if attrs else ""
        body.append('%s = "%s"(%s)%s : (%s) -> %s %s' % (r, op["type"], ", ".join(operands), a, ", ".join(types),
                                                        ttype(op["name"]), loc(op["name"])))
        ssa[op["name"]] = r
    lines.append('module @%s attributes {module.chip = "bm1684x", module.state = "TPU_LOWERED", module.weight_file = "%s"} {'
                 % (name, weight_file))
    lines.append("  func.func @main(%s) -> (%s) {" % (args, rets))
    lines += ["    " + b for b in body]
    lines.append("    return %s : %s loc(#loc)" % (", ".join(ssa[n] for n in graph["outputs"]), rets))
    lines.append("  } loc(#loc)")
    lines.append("} loc(#loc)")
    lines.append("#loc = loc(unknown)")
    lines += ['#loc%d = loc("%s")' % (i + 1, nm) for i, nm in enumerate(locs)]
    return "\n".join(lines) + "\n"
