"""Threshold tuning after the KLD calibration: the reference's ``SimpleTuner``
(python/calibration/simple_tunner.py:52-539, run by run_calibration.py with ``--tune_num`` samples, default 5).

What it does, op by op in graph order: the op is evaluated on a copy of the float graph whose weights were rounded to
their int8 grid (``module.fake_quant_weight``), with its inputs taken from the fp32 reference run and pushed through
``import_quant_bias`` (simple_tunner.py:43-50) at a candidate threshold; the candidate's distance is the mean over the
tune samples of ``||ref - out||_2 / ||ref||_1`` (calc_distance, :334-358).  Candidates run from the calibrated
threshold to the tensor's absolute maximum in ``tune_steps`` (21) equal steps; the first one sets the distance to beat,
every later one that is strictly closer becomes the best (find_better_threshold, :360-449).  An op with several inputs
tunes those not tuned yet, an op whose inputs are all tuned tunes its first input again (run, :458-507); a tensor's
threshold only ever grows (:444-448).  The reference's default flags are followed (fp32 tensors as the inputs of the
evaluated op; no ``find_lower_th``).

Here both graphs live on the GPU: the float graph runs through the executor's Top-dialect ops (module.py), the rounding
and the distance sums are device kernels, and only five doubles per evaluation reach the host.
"""
from __future__ import annotations

import copy
import ctypes as C
from typing import Dict, List, Sequence

import numpy as np

from . import _lib as L
from .module import module


def import_quant_bias(value: np.ndarray, threshold: float) -> np.ndarray:
    """simple_tunner.py:43-50 on the host (numpy), for tests and small uses."""
    scale = 127 / threshold
    v = np.round(np.asarray(value, dtype=np.float32) * scale)
    v[v > 127] = 127
    v[v < -128] = -128
    v /= scale
    return v.astype(np.float32)


class SimpleTuner:
    """``SimpleTuner(graph, weights, samples, thresholds, abs_max, tune_num=5).run()`` returns ``{tensor: threshold}``.

    ``graph`` / ``weights``: a Top-dialect graph in the executor's dict form.  ``samples``: arrays (or device tensors) for
    the graph's single input, each of the graph's batch size.  ``thresholds``: the calibration table's thresholds
    (``{name: threshold}``), ``abs_max``: each tensor's absolute maximum over the calibration set (the reference's
    ``abs_max_dict``).
    """

    def __init__(self, graph: dict, weights: Dict[str, np.ndarray], samples: Sequence, thresholds: Dict[str, float],
                 abs_max: Dict[str, float], tune_num: int = 5, tune_steps: int = 21, min_tuned_diff: float = 0.01,
                 device=None):
        import torch
        self.torch = torch
        self.tune_num = min(len(samples), int(tune_num))
        if self.tune_num < 1:
            raise ValueError("the tuner needs at least one sample")
        if len(graph["inputs"]) != 1:
            raise L.B200QError(L.ERR_UNSUPPORTED, "the tuner takes graphs with one input")
        self.tune_steps = int(tune_steps)
        self.min_tuned_diff = float(min_tuned_diff)
        self.thresholds = {k: float(v) for k, v in thresholds.items()}       # threshold_table.thresholds_map[...][0]
        self.initial_threshold = copy.deepcopy(self.thresholds)
        self.abs_max = abs_max
        self.module = module(device=device)
        self.module.load(graph, weights)
        self.module_dq = module(device=device)
        self.module_dq.load(graph, weights)
        self.module_dq.fake_quant_weight()
        self.parser = self.module.parser
        self.lib = L.lib()
        self.tuned_op_list: List[str] = []
        self.evaluations = 0
        # fp32 reference activations of every tune sample, kept on the device (the reference drops them by use count
        # to save host memory; the values are the same)
        self.ref: List[Dict[str, "torch.Tensor"]] = []
        inp = graph["inputs"][0]
        for i in range(self.tune_num):
            self.module.set_tensor(inp, samples[i])
            self.module.invoke()
            self.ref.append({n: t.clone() for n, t in self.module.tensors.items()})
        self._sums = torch.zeros(5, dtype=torch.float64, device=self.module.device)

    def _stream(self):
        return C.c_void_p(self.torch.cuda.current_stream(self.module.device).cuda_stream)

    def calc_distance(self, evaled_op: str, threshold: float):
        """(mean distance, mean cosine similarity) of `evaled_op` with every input quantised at `threshold`."""
        P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
        distance = 0.0
        total_cos = 0.0
        pre_ops = self.parser.get_pre_op_by_op_name(evaled_op)
        for idx in range(self.tune_num):
            for name in pre_ops:
                src, dst = self.ref[idx][name], self.module_dq.tensors[name]
                L.check(self.lib.b200q_top_fake_quant_f32_dev(P(src), P(dst), src.numel(), float(threshold), self._stream()))
            self.module_dq.invoke_op(evaled_op)
            out, ref = self.module_dq.tensors[evaled_op], self.ref[idx][evaled_op]
            self._sums.zero_()
            L.check(self.lib.b200q_top_distance_f32_dev(P(out), P(ref), ref.numel(), P(self._sums), self._stream()))
            d2, r1, dot, xx, rr = self._sums.cpu().tolist()
            distance += float(np.sqrt(d2)) / r1 if r1 > 0 else 0.0
            total_cos += dot / float(np.sqrt(xx) * np.sqrt(rr)) if xx > 0 and rr > 0 else 0.0
            self.evaluations += 1
        return distance / self.tune_num, total_cos / self.tune_num

    def find_better_threshold(self, evaled_op: str, tuned_op: str) -> None:
        prev_distance = -1.0
        threshold = self.initial_threshold[tuned_op]
        abs_max = float(self.abs_max[tuned_op])
        th_min = threshold
        best_threshold = threshold
        diff = abs(abs_max - th_min)
        step = (abs_max - th_min) / self.tune_steps
        if step > 0 and diff > self.min_tuned_diff:
            for i in range(self.tune_steps + 1):
                cur_threshold = th_min + step * i
                cur_distance, _ = self.calc_distance(evaled_op, cur_threshold)
                if prev_distance == -1.0:
                    prev_distance = cur_distance
                    continue
                if cur_distance < prev_distance:
                    prev_distance = cur_distance
                    best_threshold = cur_threshold
        if best_threshold > self.thresholds[tuned_op]:
            self.thresholds[tuned_op] = best_threshold

    def run(self) -> Dict[str, float]:
        for evaled_op in self.parser.get_op_name_list():
            if self.parser.get_op_type_by_op_name(evaled_op) in (None, "top.Input"):
                continue
            pre_ops = self.parser.get_pre_op_by_op_name(evaled_op)
            if not pre_ops:
                continue
            if all(p in self.tuned_op_list for p in pre_ops):
                self.find_better_threshold(evaled_op, pre_ops[0])
                self.tuned_op_list.append(pre_ops[0])
                continue
            for tuned_op in pre_ops:
                if tuned_op not in self.tuned_op_list:
                    self.find_better_threshold(evaled_op, tuned_op)
                    self.tuned_op_list.append(tuned_op)
        return dict(self.thresholds)
