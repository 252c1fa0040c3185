"""The MlirParser-shaped graph queries (tpu-mlir_b200/graph_queries.py) on the lowered ResNet-50 graph and on a small
graph that goes through the .mlir text."""
import numpy as np

from tpu_mlir_b200 import mlir_text as MT
from tpu_mlir_b200 import resnet50
from tpu_mlir_b200.graph_queries import MlirParser


def _resnet_graph(batch=4):
    ops = resnet50.build_fp32(seed=3)
    names = ["input"] + [op["name"] for op in ops]
    table = {n: (1.0 + 0.01 * i, -1.0 if i % 3 else 0.0, 1.0) for i, n in enumerate(names)}   # any thresholds do here
    return resnet50.lower_int8(ops, table, batch=batch)


def test_resnet50_graph_queries():
    graph, _ = _resnet_graph()
    p = MlirParser(graph)
    names = p.get_op_name_list()
    assert names[0] == "input" and names[1] == "input_q" and len(names) == len(graph["ops"]) + 1
    assert p.get_batch_size() == 4 and p.get_input_num() == 1 and p.get_input_shapes() == [[4, 3, 224, 224]]
    assert p.get_op_type_by_op_name("input") == "top.Input"
    assert p.get_op_type_by_op_name("conv1") == "tpu.Conv2D"
    assert p.get_pre_op_by_op_name("conv1") == ["input_q"] and p.get_pre_op_by_op_name("input") == []
    # a residual add reads the block's last convolution and the shortcut
    add = "layer1.0.add"
    pre = p.get_pre_op_by_op_name(add)
    assert len(pre) == 2 and all(p.get_op_type_by_op_name(n) == "tpu.Conv2D" for n in pre)
    # its output feeds the next block's first convolution and that block's add (identity shortcut)
    nxt = p.get_next_op_by_op_name(add)
    assert len(nxt) == 2 and p.get_use_count_by_op_name(add) == 2 and p.get_user_count_by_op_name(add) == 2
    assert p.get_outputs_by_op_name(add) == [add] and p.get_outputs_by_op_name("nope") is None
    assert p.get_opds_by_op_name(add) == pre
    # transitive closures reach the ends of the graph
    assert "input" in p.get_all_pre_ops_by_op_name("fc") or "input_q" in p.get_all_pre_ops_by_op_name("fc")
    assert graph["outputs"][0] in p.get_all_next_ops_by_op_name("conv1")
    assert list(p.get_output_op_names_n_shapes().values()) == [[4, 1000]]
    assert set(p.collect_op_name_dict()) == set(names)


def test_queries_from_mlir_text(tmp_path):
    from test_mlir_text import small_graph
    graph, weights = small_graph()
    (tmp_path / "m.mlir").write_text(MT.emit_module(graph, weights, weight_file="w.npz"))
    np.savez(tmp_path / "w.npz", **weights)
    p = MlirParser(str(tmp_path / "m.mlir"))
    assert p.get_op_name_list() == ["input", "input_q", "conv", "pool", "sum", "flat", "fc", "output"]
    assert p.get_use_count_by_op_name("pool") == 2 and p.get_user_count_by_op_name("pool") == 1   # tpu.Add reads it twice
    assert p.get_next_op_by_op_name("pool") == ["sum"] and p.get_pre_op_by_op_name("sum") == ["pool", "pool"]
