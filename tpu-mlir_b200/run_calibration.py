"""Calibration of a float graph end to end, the flow of the reference's ``run_calibration.py``
(python/tools/run_calibration.py:24-115 driving python/calibration/kld_calibrator.py:629-945 and simple_tunner.py):

  float forward over the calibration samples -> per-tensor min / max and histogram -> KLD threshold
  -> optional threshold tuning on ``tune_num`` samples -> calibration table.

Everything runs on the GPU through this package's own kernels: the executor's Top-dialect ops (module.py) make the
activations, ``ShardedCalibrator`` the statistics and thresholds (samples sharded over the ranks of a process group when one
is given), ``SimpleTuner`` the tuning.  The graph is the executor's dict form (or the path of a ``.mlir`` file it can load)
with ONE input; its batch size is the first dimension of that input, and the samples come as an array whose first
dimension is a multiple of it.  Tensors whose first dimension is not the batch (none in the usual vision / transformer
graphs) are left out of the table.
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np

from .calibration import ShardedCalibrator, dump_cali_table
from .module import module


def run_calibration(graph, weights, samples, *, tune_num: int = 0, out_table: Optional[str] = None, dist=None, device=None,
                    histogram_bin_num: int = 2048) -> Dict[str, float]:
    """Returns ``{tensor: threshold}`` (after tuning when ``tune_num`` > 0) and writes ``out_table`` when given."""
    import torch
    m = module(device=device)
    m.load(graph, weights)
    g = m.graph
    if len(g["inputs"]) != 1:
        raise ValueError("run_calibration takes graphs with one input")
    inp = g["inputs"][0]
    batch = int(g["tensors"][inp]["shape"][0])
    samples = np.asarray(samples, dtype=np.float32) if not isinstance(samples, torch.Tensor) else samples
    total = int(samples.shape[0])
    if total == 0 or total % batch != 0:
        raise ValueError(f"{total} samples do not fill batches of {batch}")
    names = [inp] + [op["name"] for op in g["ops"] if g["tensors"][op["name"]]["dtype"] == "f32" and g["tensors"][op["name"]]["shape"]
                     and int(g["tensors"][op["name"]]["shape"][0]) == batch]
    rank, world = (dist.get_rank(), dist.get_world_size()) if (dist is not None and dist.is_initialized()) else (0, 1)
    if (total // batch) % world != 0:
        raise ValueError(f"{total // batch} batches do not divide over {world} ranks")
    per_rank = total // world
    local = samples[rank * per_rank:(rank + 1) * per_rank]

    def forward(b):
        m.set_tensor(inp, b)
        m.invoke()
        return {n: m._nchw(n) if n in m._nhwc else m.tensors[n] for n in names}

    class Batches:      # re-iterable: the calibrator walks the samples twice
        def __iter__(self):
            return (local[i:i + batch] for i in range(0, per_rank, batch))
    cal = ShardedCalibrator(forward, dist=dist, bin_num=histogram_bin_num)
    results = cal.run(Batches(), per_rank)
    thresholds = {n: float(r.threshold) for n, r in results.items()}
    if tune_num > 0:
        from .simple_tuner import SimpleTuner
        tune_batches = [samples[i:i + batch] for i in range(0, min(total, tune_num * batch), batch)]
        abs_max = {n: float(r.abs_max) for n, r in results.items()}
        tuned = SimpleTuner(g, m_weights(m), tune_batches, thresholds, abs_max, tune_num=tune_num, device=device).run()
        for n, th in tuned.items():
            thresholds[n] = th
            results[n].threshold = th
    if out_table and rank == 0:
        dump_cali_table(out_table, results, order=names, num_samples=total, tune_num=tune_num, histogram_bin_num=histogram_bin_num)
    return thresholds


def m_weights(m: module) -> Dict[str, np.ndarray]:
    """The weights a loaded executor holds, back as host arrays (for a second executor over the same graph)."""
    return {k: v.cpu().numpy() for k, v in m.weights.items()}
