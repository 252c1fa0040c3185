"""Calibration-table text I/O: the writer's line format and the reader's block logic."""
import datetime
import glob
import os

import pytest

from tpu_mlir_b200 import cali_table as CT

# a checkout of the reference, when there is one (TPU_MLIR_REFERENCE overrides the default location)
REF_TABLES = os.path.join(os.environ.get("TPU_MLIR_REFERENCE", "/root/reference"), "regression/cali_tables")


def test_write_then_read_round_trip(tmp_path):
    rows = [("input", 2.5680201, -2.10256, 2.5680201), ("conv1", 1.0 / 3.0, 0.0, 4.4452448), ("dead", 0.0, 0.0, 0.0),
            ("nan_th", float("nan"), -1.0, 1.0)]
    p = tmp_path / "t_cali_table"
    CT.write_cali_table(str(p), rows, mlir_file="m.mlir", method="use_kl", num_samples=100, tune_num=5,
                        int4_rows=[("conv1", 0.7)], asym_ops=["conv1"], now=datetime.datetime(2024, 1, 2, 3, 4, 5))
    text = p.read_text().splitlines()
    assert text[0] == "# mlir version: b200q cali version 1.0"
    assert text[2] == "# genetated time: 2024-01-02 03:04:05"
    assert "# op_name    threshold    min    max" in text
    assert "input 2.5680201 -2.1025600 2.5680201" in text
    assert "conv1 0.3333333 0.0000000 4.4452448" in text
    assert "dead 0.0000100 0.0000000 0.0000000" in text      # threshold floor 1e-5
    assert "nan_th 0.0000100 -1.0000000 1.0000000" in text
    t = CT.read_cali_table(str(p))
    assert list(t.int8) == ["input", "conv1", "dead", "nan_th"]
    assert t.int8["conv1"] == (0.3333333, 0.0, 4.4452448)
    assert t.int4["conv1"] == (0.7, pytest.approx(-0.8), 0.7)
    assert t.asym_op == ["conv1"]


def test_reader_blocks_inf_and_crlf(tmp_path):
    p = tmp_path / "x_cali_table"
    p.write_text("# op_name    threshold    min    max\r\n"
                 "a 1.5 -inf inf\r\n"
                 "info_layer 2.0 -1.0 1.0\n"          # a NAME holding "inf" is not a field
                 "bad line without numbers\n"
                 "#weight_scale\n"
                 "w1 3 0.1 0.2 0.3\n"
                 "#int4_th\n"
                 "# a plain comment keeps the int4 block open\n"
                 "b 0.5 -0.6 0.5\n"
                 "#int4_op\n"
                 "b\n")
    t = CT.read_cali_table(str(p))
    assert t.int8 == {"a": (1.5, -65000.0, 65000.0), "info_layer": (2.0, -1.0, 1.0)}
    assert t.weight_scale == {"w1": [0.1, 0.2, 0.3]}
    assert t.int4 == {"b": (0.5, -0.6, 0.5)}
    assert t.int4_op == ["b"]


@pytest.mark.skipif(not os.path.isdir(REF_TABLES), reason="the reference tree is not present on this machine")
def test_reference_tables_parse_and_reserialise():
    """Every table of the reference's regression set parses, and its int8 rows re-serialise to the same text."""
    files = sorted(glob.glob(os.path.join(REF_TABLES, "*_cali_table")))  # the folder also holds qtables
    assert len(files) > 50
    rows_total = 0
    for f in files:
        t = CT.read_cali_table(f)
        assert t.int8, f
        lines = set(l.rstrip("\r\n") for l in open(f))
        same = sum(1 for name, (th, lo, hi) in t.int8.items() if CT.format_row(name, th, lo, hi) in lines)
        # tables written by other tools may use other float formats; the calibrator's own must match exactly
        if any("quantization threshold calculation method" in h or "histogram number" in h for h in t.header):
            assert same >= 0.99 * len(t.int8), (f, same, len(t.int8))
        rows_total += len(t.int8)
    assert rows_total > 5000


def test_dump_calibrator_results(tmp_path):
    from tpu_mlir_b200.calibration import TensorResult, dump_cali_table
    res = {"conv1": TensorResult("conv1", -0.25, 3.5, 3.5, 2048, 0.001, 3.1234567, 3.1234567),
           "input": TensorResult("input", -2.0, 2.5, 2.5, 2048, 0.001, 2.4, 2.4)}
    p = tmp_path / "r_cali_table"
    dump_cali_table(str(p), res, order=["input", "conv1", "missing"], num_samples=64)
    t = CT.read_cali_table(str(p))
    assert list(t.int8) == ["input", "conv1"]
    assert t.int8["conv1"] == (3.1234567, -0.25, 3.5)
    assert "# sample number: 64" in t.header
