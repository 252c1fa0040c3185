"""Graph queries over a loaded model, with the method names and answers of the reference's ``MlirParser``
(python/utils/mlir_parser.py:168-383).  The reference parses the ``.mlir`` text through MLIR's Python bindings; here
the same questions are answered from the graph dict the executor runs (module.py), read from a dict or from a lowered
model's ``.mlir`` text by mlir_text.py.  The calibrator walks a model with exactly these calls
(python/calibration/kld_calibrator.py, python/calibration/simple_tunner.py).

Like the reference's list, ``ops`` holds every operation that has a tensor result except weights and the None op:
the graph's inputs appear as operations of type ``top.Input`` without operands, an operation is named after its
(first) output tensor, and its operands are the names of the tensors it reads (weights excluded).
"""
from __future__ import annotations

from itertools import chain
from typing import Dict, List, Optional


class Operation:
    """One entry of ``MlirParser.ops``: ``name, type, opds, outputs, attrs, shape`` (mlir_parser.py:20-165)."""

    def __init__(self, name: str, type_: str, opds: List[str], outputs: List[str], attrs: Dict, shape: List[int]):
        self.name = name
        self.type = type_
        self.opds = list(opds)
        self.outputs = list(outputs)
        self.attrs = dict(attrs)
        self.shape = list(shape)

    def __repr__(self):
        return f"{self.name},{self.type},{self.attrs},{self.shape},{self.opds}"


class MlirParser:
    def __init__(self, graph_or_mlir_file, weights: Optional[str] = None):
        if isinstance(graph_or_mlir_file, str):
            from .mlir_text import load_mlir
            graph, _ = load_mlir(graph_or_mlir_file, weights)
        else:
            graph = graph_or_mlir_file
        self.graph = graph
        self.module_name = graph.get("name", "")
        self.module_state = graph.get("state", "TPU_LOWERED")
        self.module_chip = graph.get("chip", "")
        self.module_weight_file = graph.get("weight_file", "")
        tensors = graph["tensors"]
        self.ops: List[Operation] = []
        self.inputs: List[Operation] = []
        for name in graph["inputs"]:
            op = Operation(name, "top.Input", [], [name], {}, tensors[name]["shape"])
            self.ops.append(op)
            self.inputs.append(op)
        produced = set(graph["inputs"]) | {o["name"] for o in graph["ops"]}
        for o in graph["ops"]:
            opds = [t for t in o["inputs"] if t in produced]
            self.ops.append(Operation(o["name"], o["type"], opds, [o["name"]], o.get("attrs", {}), tensors[o["name"]]["shape"]))
        self._outputs = list(graph["outputs"])

    # ---- the calls of mlir_parser.py:217-383, same names and meaning
    def get_op_name_list(self):
        return [op.name for op in self.ops]

    def get_op_output_name_list(self):
        return list(chain(*[op.outputs for op in self.ops]))

    def get_input_num(self):
        return len(self.inputs)

    def get_input_shapes(self):
        return [list(op.shape) for op in self.inputs]

    def get_input_types(self):
        return [self.graph["tensors"][op.name]["dtype"] for op in self.inputs]

    def get_batch_size(self):
        return self.inputs[0].shape[0]

    def get_pre_op_by_op_name(self, op_name):
        outs = set(self.get_op_output_name_list())
        res = []
        for op in self.ops:
            if op.name == op_name:
                res += [opd for opd in op.opds if opd in outs]
        return res

    def get_next_op_by_op_name(self, op_name):
        outs = set(self.get_op_output_name_list())
        return [op.name for op in self.ops if op_name in op.opds and op.name in outs]

    def get_all_pre_ops_by_op_name(self, op_name):
        all_pre_ops = [op_name] + self.get_pre_op_by_op_name(op_name)
        cur = self.get_pre_op_by_op_name(op_name)
        while cur:
            tmp = cur.pop(0)
            for p in self.get_pre_op_by_op_name(tmp):
                if p not in all_pre_ops:
                    cur.append(p)
                    if self.get_pre_op_by_op_name(p):
                        all_pre_ops.append(p)
        return all_pre_ops

    def get_all_next_ops_by_op_name(self, op_name):
        all_next_ops = [op_name] + self.get_next_op_by_op_name(op_name)
        cur = self.get_next_op_by_op_name(op_name)
        while cur:
            tmp = cur.pop(0)
            for n in self.get_next_op_by_op_name(tmp):
                if n not in all_next_ops:
                    cur.append(n)
                    all_next_ops.append(n)
        return all_next_ops

    def get_user_count_by_op_name(self, op_name):
        return sum(1 for op in self.ops if op_name in op.opds)

    def get_use_count_by_op_name(self, op_name):
        return sum(op.opds.count(op_name) for op in self.ops)

    def get_outputs_by_op_name(self, op_name):
        for op in self.ops:
            if op.name == op_name:
                return op.outputs
        return None

    def get_op_by_op_name(self, op_name):
        for op in self.ops:
            if op.name == op_name:
                return op
        return None

    def get_opds_by_op_name(self, op_name):
        for op in self.ops:
            if op.name == op_name:
                return op.opds
        return None

    def get_op_type_by_op_name(self, op_name):
        for op in self.ops:
            if op.name == op_name:
                return op.type
        return None

    def get_output_op_names_n_shapes(self):
        return {name: list(self.graph["tensors"][name]["shape"]) for name in self._outputs}

    def collect_op_name_dict(self):
        return {op.name: op for op in self.ops}
