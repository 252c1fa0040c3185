"""The oracle against the reference's own outputs (tests/golden/, made by make_golden.py) and against
the rounding known answers in the reference header."""
import json
import os

import numpy as np
import pytest

import oracle

G = os.path.join(os.path.dirname(__file__), "golden")


def test_rounding_known_answers():
    kat = json.load(open(os.path.join(G, "rounding_kat.json")))
    for case in kat["cases"]:
        for value, want in case["pairs"]:
            # float face (to_int) and fixed-point face (RightShiftRound with value = num / 2^10)
            assert oracle.to_int(value, case["mode"]) == want, (case["name"], value)
            num = int(round(value * 1024))
            # 1.6 / 1.4 are not dyadic: the nearest 10-bit fraction keeps the same side of .5
            assert oracle.rshift_round(num, 10, case["mode"]) == want, (case["name"], value)


def test_rshift_round_edges():
    assert oracle.rshift_round(5, 0, oracle.RM_HALF_UP) == 5
    assert oracle.rshift_round(5, -3, oracle.RM_HALF_UP) == 40          # negative shift = left shift
    assert oracle.rshift_round(-1, 80, oracle.RM_HALF_UP) == 0           # shift clamps to 63; mantissa >= half
    assert oracle.rshift_round(-1, 80, oracle.RM_DOWN) == -1
    assert oracle.rshift_round(-3, 1, oracle.RM_HALF_UP) == -1
    assert oracle.rshift_round(-3, 1, oracle.RM_HALF_AWAY) == -2
    assert oracle.rshift_round(-5, 1, oracle.RM_HALF_EVEN) == -2
    assert oracle.rshift_round(-5, 1, oracle.RM_TOWARDS_ZERO) == -2
    assert oracle.rshift_round(-7, 2, oracle.RM_TOWARDS_ZERO) == -1


def test_mbqm_matches_definition():
    rng = np.random.default_rng(1)
    for _ in range(2000):
        x = int(rng.integers(-2**23, 2**23))
        m = int(rng.integers(2**30, 2**31))
        s = int(rng.integers(0, 21))
        a = oracle.rshift_round(x * m, 31, oracle.RM_HALF_UP)
        want = oracle.rshift_round(a, s, oracle.RM_HALF_AWAY) if s else a
        assert oracle.mbqm(x, m, -s) == want
    # saturation between the two shifts, and the int32 left shift
    assert oracle.mbqm(-2**31, -2**31, 0) == 2**31 - 1
    assert oracle.mbqm(2**30, 2**31 - 1, 1) == -(2**31 - 1)          # x << shift wraps in int32
    assert oracle.mbqm(-2**29, 2**31 - 1, 1) == -2**30 + 1


def _hist_cases():
    z = np.load(os.path.join(G, "calib_hist.npz"))
    names = sorted({k.split("/")[1] for k in z.files if k.startswith("single/")})
    return z, names


def test_histogram_matches_reference():
    z, names = _hist_cases()
    assert names
    for name in names:
        x = z[f"single/{name}/x"]
        abs_max = max(abs(np.min(x)), abs(np.max(x)))
        for bins in (2048, 777):
            h, w = oracle.histogram(x, abs_max, bins)
            assert np.array_equal(h, z[f"single/{name}/{bins}/hist"]), (name, bins)
            assert np.float32(w).tobytes() == z[f"single/{name}/{bins}/width"].tobytes()


@pytest.mark.parametrize("name", ["grow", "zero_then", "reset"])
def test_streaming_histogram_matches_reference(name):
    z = np.load(os.path.join(G, "calib_hist.npz"))
    n = int(z[f"stream/{name}/n"])
    samples = [z[f"stream/{name}/x{i}"] for i in range(n)]
    st = oracle.StreamingHistogram(2048)
    for a in samples:
        st.update(a)
    assert len(st.hist) == len(z[f"stream/{name}/hist"])
    assert np.array_equal(st.hist, z[f"stream/{name}/hist"])
    for key, val in (("width", st.width), ("th", st.th), ("min", st.min), ("max", st.max)):
        assert np.float32(val).tobytes() == z[f"stream/{name}/{key}"].tobytes(), key
    # the order-free restatement: sum of zero-extended per-sample histograms with the scheduled (th, bins)
    mins = np.minimum.accumulate([np.min(a) for a in samples])
    maxs = np.maximum.accumulate([np.max(a) for a in samples])
    absv = np.maximum(np.abs(mins), np.abs(maxs)).astype(np.float32)
    ok = [np.abs(a).max() >= 1e-8 for a in samples]
    sched = oracle.bin_schedule(absv, ok)
    last_reset = max([i for i, s in enumerate(sched) if s[2]] + [0])
    final_bins = [s for s in sched if s[0] is not None][-1][1]
    total = np.zeros(final_bins, np.int32)
    for i, (a, (th, nb, _)) in enumerate(zip(samples, sched)):
        if th is None or i < last_reset:
            continue
        oracle.histogram(a, th, nb, into=total)
    assert np.array_equal(total, z[f"stream/{name}/hist"])


def _kld_names():
    z = np.load(os.path.join(G, "calib_kld.npz"))
    return z, sorted({k.split("/")[0] for k in z.files})


def test_kld_matches_reference_golden():
    z, names = _kld_names()
    assert len(names) >= 8
    for name in names:
        h, w = oracle.fold_for_kld(z[f"{name}/hist"], z[f"{name}/width"])
        assert len(h) == int(z[f"{name}/folded_len"])
        assert np.float32(w).tobytes() == z[f"{name}/folded_width"].tobytes()
        th = oracle.kl_diversity_hist(h, w)
        assert th.tobytes() == z[f"{name}/threshold"].tobytes(), (name, th, z[f"{name}/threshold"])


@pytest.mark.skipif(not oracle.ref_kld_available(), reason="compiled reference KLD not present")
def test_kld_matches_compiled_reference_random():
    rng = np.random.default_rng(7)
    for t in range(12):
        bins = int(rng.choice([128, 2048, 2176, 4096, 16384]))
        scale = float(rng.uniform(0.3, 3))
        x = (rng.standard_normal(50000) * scale).astype(np.float32)
        if t % 3 == 0:
            x = np.maximum(x, 0)
        h, w = oracle.histogram(x, np.abs(x).max(), bins)
        assert oracle.kl_diversity_hist(h, w).tobytes() == oracle.ref_kl_diversity_hist(h, w).tobytes()
