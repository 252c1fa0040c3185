"""Calibration-table text I/O in the reference's format.

Writer: the file ``ActivationCalibrator.dump_cali_table`` produces (python/calibration/kld_calibrator.py:804-884):
a ``#`` header, then one ``name threshold min max`` line per activation with seven decimals, optional ``#int4_th``
and ``#asym_op`` blocks.  Reader: the block logic of the ImportCalibration pass
(lib/Dialect/Top/Transforms/ImportCalibration.cpp:42-160): the int8 block is open from the start, comments holding
``#weight_scale``, ``#int4_th``, ``#tpu-mlir-fp8``, ``mqbench-fp8``, ``asym_op`` or ``int4_op`` switch blocks (other
comments do not), data lines must match ``\\S+\\s+[-0-9.e]+\\s+[-0-9.e]+\\s+[-0-9.e]+``, ``inf`` fields become ``6.5e4``.
"""
from __future__ import annotations

import datetime
import math
import re
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Tuple

_CALI_LINE = re.compile(r"\S+\s+[-0-9.e]+\s+[-0-9.e]+\s+[-0-9.e]+")
MIN_THRESHOLD = 1e-5  # thresholds at or below this (or NaN) are written as 1e-5 (kld_calibrator.py:851-855)


@dataclass
class CaliTable:
    """Parsed table: name -> (threshold, min, max) per block, plus the name lists of the op blocks."""
    int8: Dict[str, Tuple[float, float, float]] = field(default_factory=dict)
    int4: Dict[str, Tuple[float, float, float]] = field(default_factory=dict)
    fp8: Dict[str, Tuple[float, float, float]] = field(default_factory=dict)
    weight_scale: Dict[str, List[float]] = field(default_factory=dict)
    asym_op: List[str] = field(default_factory=list)
    int4_op: List[str] = field(default_factory=list)
    header: List[str] = field(default_factory=list)


def format_row(name: str, threshold: float, vmin: float, vmax: float) -> str:
    return "{} {:.7f} {:.7f} {:.7f}".format(name, threshold, vmin, vmax)


def write_cali_table(path: str, rows: Iterable[Tuple[str, float, float, float]], *, mlir_file: str = "",
                     method: str = "use_kl", histogram_bin_num: int = 2048, num_samples: int = 0, tune_num: int = 0,
                     version: str = "b200q", int4_rows: Optional[Iterable[Tuple[str, float]]] = None,
                     asym_ops: Optional[Iterable[str]] = None, now: Optional[datetime.datetime] = None) -> None:
    """Write `rows` = (tensor name, threshold, min, max) in graph order."""
    with open(path, "w") as f:
        f.write("# mlir version: {} cali version 1.0\n".format(version))
        f.write("# mlir: {}\n".format(mlir_file))
        f.write("# genetated time: {}\n".format(now or datetime.datetime.now()))  # spelling of the reference
        f.write("# quantization threshold calculation method: {}\n".format(method))
        f.write("# histogram number: {}\n".format(histogram_bin_num))
        f.write("# sample number: {}\n###\n".format(num_samples))
        f.write("# tune number: {}\n###\n".format(tune_num))
        f.write("# op_name    threshold    min    max\n")
        for name, th, vmin, vmax in rows:
            if th <= MIN_THRESHOLD or math.isnan(th):
                th = MIN_THRESHOLD
            f.write(format_row(name, th, vmin, vmax) + "\n")
        if int4_rows is not None:
            f.write("\n#int4_th\n")
            for name, th in int4_rows:
                f.write(format_row(name, th, -th * 8.0 / 7.0, th) + "\n")
        if asym_ops is not None:
            f.write("\n#asym_op\n")
            for name in asym_ops:
                f.write("{}\n".format(name))


def _flag(line: str) -> int:
    if not line.startswith("#"):
        return 0
    if "#weight_scale" in line:
        return 1
    if "#int4_th" in line:
        return 2
    if "#tpu-mlir-fp8" in line:
        return 3
    if "mqbench-fp8" in line:
        return 4
    if "asym_op" in line:
        return 5
    if "int4_op" in line:
        return 6
    return 0


def _replace_inf(line: str) -> str:
    # an "inf" that follows a blank is a data field (ImportCalibration.cpp:85-101)
    pos = line.rfind("inf")
    if pos == -1 or (line.rfind(" ", 0, pos + 1) == -1 and line.rfind("\t", 0, pos + 1) == -1):
        return line
    out, i = [], 0
    first_sep = min([p for p in (line.find(" "), line.find("\t")) if p != -1])
    while True:
        j = line.find("inf", i)
        if j == -1:
            out.append(line[i:])
            break
        if j > first_sep:
            out.append(line[i:j] + "6.5e4")
        else:
            out.append(line[i:j + 3])
        i = j + 3
    return "".join(out)


def read_cali_table(path: str) -> CaliTable:
    t = CaliTable()
    block = 0  # the int8 block is open from the start
    with open(path) as f:
        for raw in f:
            line = raw.rstrip("\n")
            if line.endswith("\r"):
                line = line[:-1]
            if not line:
                continue
            line = _replace_inf(line)
            if line.startswith("#"):
                t.header.append(line)
                flag = _flag(line)
                if flag:
                    block = flag  # only the flag comments switch blocks; any other comment leaves the block open
                continue      # (a comment never matches the data pattern; in the name-list blocks it is skipped here)
            parts = line.split()
            if block == 0 or block == 2 or block == 3 or block == 4:
                if not _CALI_LINE.fullmatch(line.strip()):
                    continue
                rec = (float(parts[1]), float(parts[2]), float(parts[3]))
                (t.int8 if block == 0 else t.int4 if block == 2 else t.fp8)[parts[0]] = rec
            elif block == 1:
                n = int(parts[1])
                t.weight_scale[parts[0]] = [float(v) for v in parts[2:2 + n]]
            elif block == 5:
                t.asym_op.append(parts[0])
            elif block == 6:
                t.int4_op.append(parts[0])
    return t


def table_for_lowering(t: CaliTable) -> Dict[str, Tuple[float, float, float]]:
    """The int8 block in the form resnet50.lower_int8 takes."""
    return dict(t.int8)
