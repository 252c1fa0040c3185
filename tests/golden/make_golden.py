#!/usr/bin/env python3
"""Generate the golden vectors under tests/golden/ from the reference itself.

Run in a container that has the reference checkout (default location below, or $TPU_MLIR_REFERENCE):

    python tests/golden/make_golden.py

It imports the reference's python/calibration/cali_math.py *by path* (nothing is copied) and calls the
reference's bindings/kld/calibration_math.cpp compiled into oracle/_ref/ by oracle/Makefile.  Outputs:

    calib_hist.npz      inputs + CaliMathCpu.histogram / combine_histogram results
    calib_kld.npz       histograms + kl_diversity_hist thresholds of the compiled reference
    rounding_kat.json   the rounding known answers written in include/tpu_mlir/Support/MathUtils.h:29-40
"""
import ctypes as C
import importlib.util
import json
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("TPU_MLIR_REFERENCE", "/root/reference")


def load_cali_math():
    spec = importlib.util.spec_from_file_location("ref_cali_math", os.path.join(REF, "python/calibration/cali_math.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.CaliMathCpu()


def load_ref_kld():
    subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "ref"], check=True)
    L = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "calibration_math.so"))
    L.kl_diversity_hist.restype = C.c_float

    def kld(hist, width, dst_bins=128):
        h = np.ascontiguousarray(hist, dtype=np.int32)
        return np.float32(L.kl_diversity_hist(h.ctypes.data_as(C.POINTER(C.c_int)), C.c_float(float(width)),
                                              C.c_longlong(h.size), C.c_longlong(dst_bins)))

    return kld


def stream(math_impl, samples, bin_num=2048):
    """The per-tensor control flow of kld_calibrator.py:391-398,:462-476, driving the REFERENCE math_impl."""
    mn, mx = float("inf"), float("-inf")
    state = None
    for a in samples:
        a = a.flatten()
        mn = min(np.min(a), mn)
        mx = max(np.max(a), mx)
        abs_value = max(abs(mn), abs(mx))
        if np.abs(a).max() < 1e-8:
            continue
        if state is None:
            hist, width = math_impl.histogram(a, abs_value, bin_num)
            state = (hist, width, mn, mx, abs_value)
        else:
            state = math_impl.combine_histogram(state, a, mn, mx, abs_value, bin_num)
    return state, mn, mx


def fold(hist, width, dst_bins=128):
    """kld_calibrator.py:329-342 (padding + folding before the KLD call)."""

    def pad(h):
        r = len(h) % dst_bins
        return h if r == 0 else np.concatenate((h, np.zeros(dst_bins - r, dtype=h.dtype)))

    h = pad(hist)
    while len(h) > 64 * 2048:
        h = pad(h[::2] + h[1::2])
        width = width * 2.0
    return h, width


def main():
    m = load_cali_math()
    kld = load_ref_kld()
    rng = np.random.default_rng(20240)
    out = {}
    # ---- single histograms
    singles = {
        "normal": rng.standard_normal(6000).astype(np.float32),
        "relu": np.maximum(rng.standard_normal(6000), 0).astype(np.float32),
        "small": (rng.standard_normal(3000) * 1e-3).astype(np.float32),
        "heavy": (rng.standard_t(2, 4000) * 3).astype(np.float32),
        "ties": (rng.integers(-40, 41, 5000) * 0.5).astype(np.float32),
    }
    for name, a in singles.items():
        abs_max = max(abs(np.min(a)), abs(np.max(a)))
        for bins in (2048, 777):
            h, w = m.histogram(a, abs_max, bins)
            out[f"single/{name}/{bins}/hist"] = h
            out[f"single/{name}/{bins}/width"] = np.float32(w)
        out[f"single/{name}/x"] = a
    # ---- streaming (bins grow)
    streams = {
        "grow": [(rng.standard_normal(3000) * s).astype(np.float32) for s in (1.0, 0.5, 1.7, 1.1, 3.3, 2.0, 3.4)],
        "zero_then": [np.zeros(500, np.float32)] + [(rng.standard_normal(2000) * s).astype(np.float32)
                                                     for s in (0.2, 0.21, 1.0)],
        "reset": [(rng.standard_normal(1000) * 1e-4).astype(np.float32),
                  (rng.standard_normal(1000) * 10).astype(np.float32),
                  (rng.standard_normal(1000) * 11).astype(np.float32)],
    }
    kld_cases = {}
    for name, samples in streams.items():
        state, mn, mx = stream(m, samples)
        hist, width, _, _, th = state
        for i, a in enumerate(samples):
            out[f"stream/{name}/x{i}"] = a
        out[f"stream/{name}/n"] = np.int64(len(samples))
        out[f"stream/{name}/hist"] = hist
        out[f"stream/{name}/width"] = np.float32(width)
        out[f"stream/{name}/th"] = np.float32(th)
        out[f"stream/{name}/min"] = np.float32(mn)
        out[f"stream/{name}/max"] = np.float32(mx)
        kld_cases[f"stream_{name}"] = (hist, width)
    np.savez_compressed(os.path.join(HERE, "calib_hist.npz"), **out)

    # ---- KLD thresholds from the compiled reference
    kout = {}
    h, w = m.histogram(singles["normal"], 4.5, 2048)
    kld_cases["normal2048"] = (h, w)
    big = np.abs(rng.standard_normal(400000)).astype(np.float32)
    h, w = m.histogram(big, big.max(), 2048)
    kld_cases["halfnormal_400k"] = (h, w)
    h, w = m.histogram(big * (1 + 40 * (rng.random(400000) < 1e-4)), float((big * 41).max()), 9000)
    kld_cases["outliers_9000"] = (h, w)
    lap = rng.laplace(0, 1, 300000).astype(np.float32)
    h, w = m.histogram(lap, np.abs(lap).max(), 150000)      # > 131072 bins: exercises the fold
    kld_cases["laplace_fold"] = (h, w)
    sparse = np.zeros(4096, np.int32)
    sparse[[3, 40, 41, 500, 1999, 4000]] = [100000, 5000, 7000, 300, 20, 1]
    kld_cases["sparse"] = (sparse, np.float32(0.01))
    huge = (rng.integers(0, 3, 2048) * 20000000).astype(np.int32)   # float sums leave the exact range
    kld_cases["huge_counts"] = (huge, np.float32(0.125))
    for name, (hist, width) in kld_cases.items():
        hf, wf = fold(np.asarray(hist, dtype=np.int32), width)
        kout[f"{name}/hist"] = np.asarray(hist, dtype=np.int32)
        kout[f"{name}/width"] = np.float32(width)
        kout[f"{name}/folded_len"] = np.int64(len(hf))
        kout[f"{name}/folded_width"] = np.float32(wf)
        kout[f"{name}/threshold"] = kld(hf, wf)
    np.savez_compressed(os.path.join(HERE, "calib_kld.npz"), **kout)

    # ---- rounding known answers (MathUtils.h:29-40): value = num / 2**shift
    kat = {
        "source": "include/tpu_mlir/Support/MathUtils.h:29-40 (comments beside the RoundingMode enum)",
        "cases": [
            {"mode": 0, "name": "HALF_AWAY_FROM_ZERO", "pairs": [[1.5, 2], [-1.5, -2]]},
            {"mode": 1, "name": "HALF_UP", "pairs": [[1.5, 2], [-1.5, -1]]},
            {"mode": 2, "name": "HALF_DOWN", "pairs": [[1.5, 1], [-1.5, -2]]},
            {"mode": 3, "name": "HALF_TO_EVEN", "pairs": [[1.5, 2], [2.5, 2]]},
            {"mode": 6, "name": "TOWARDS_ZERO", "pairs": [[1.6, 1], [-1.6, -1]]},
            {"mode": 8, "name": "UP", "pairs": [[1.4, 2], [-1.6, -1]]},
            {"mode": 9, "name": "DOWN", "pairs": [[1.6, 1], [-1.4, -2]]},
        ],
    }
    with open(os.path.join(HERE, "rounding_kat.json"), "w") as f:
        json.dump(kat, f, indent=1)
    print("golden vectors written:", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    sys.exit(main())
