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


@pytest.mark.skipif(not oracle.ref_mathutils_available(), reason="compiled reference MathUtils functions not present")
def test_requant_arithmetic_matches_compiled_reference():
    """to_int, RightShiftRound, MultiplyByQuantizedMultiplier and applyMultiplierAndRShift of the oracle against the
    reference's own functions (MathUtils.cpp:179-213,:474-562) on edge values and random draws."""
    R = oracle.ref_mathutils()
    rng = np.random.default_rng(11)
    rmodes = [oracle.RM_HALF_AWAY, oracle.RM_HALF_UP, oracle.RM_HALF_DOWN, oracle.RM_HALF_EVEN, oracle.RM_TOWARDS_ZERO,
              oracle.RM_UP, oracle.RM_DOWN]
    # to_int on halves, near-halves and random floats
    vals = [0.0, 0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 0.49999997, -0.49999997, 1e6 + 0.5, -1e6 - 0.5, 123456.75]
    vals += list((rng.standard_normal(300) * 1000).astype(np.float32))
    for rm in rmodes:
        for v in vals:
            assert oracle.to_int(v, rm) == R.ref_to_int_f32(float(np.float32(v)), rm), (v, rm)
    # RightShiftRound: every mode the function knows, shifts 0..63 and negative (left) shifts, ties included
    srcs = [0, 1, -1, 3, -3, 5, -5, 6, -6, 2**31 - 1, -2**31, 2**40 + 2**20, -(2**40) - 2**20, 2**62, -(2**62)]
    srcs += [int(v) for v in rng.integers(-2**50, 2**50, 200)]
    for rm in rmodes:
        for s in list(range(0, 64)) + [-1, -3]:
            for x in srcs:
                if s < 0 and abs(x) >= 2**58:
                    continue   # the left shift would overflow int64 (undefined in the reference too)
                assert oracle.rshift_round(x, s, rm) == R.ref_rshift_round(x, s, rm), (x, s, rm)
    # MultiplyByQuantizedMultiplier: TFLite multipliers, right and (small) left shifts
    for _ in range(4000):
        x = int(rng.integers(-2**24, 2**24))
        m = int(rng.integers(2**30, 2**31))
        sh = int(rng.integers(-31, 3))
        if sh > 0 and abs(x) >= 2**28:
            continue
        for rm in (oracle.RM_HALF_AWAY, oracle.RM_HALF_UP):
            assert oracle.mbqm(x, m, sh, rm) == R.ref_mbqm(x, m, sh, rm), (x, m, sh, rm)
    # applyMultiplierAndRShift: every requant mode, both chip families
    for _ in range(4000):
        v = int(rng.integers(-2**24, 2**24))
        for qm in (oracle.QM_MULTIPLIER_SHIFT, oracle.QM_ONLY_SHIFT, oracle.QM_QDM, oracle.QM_TFLITE, oracle.QM_TFLITE_LSHIFT):
            for cv in (0, 1):
                if qm == oracle.QM_MULTIPLIER_SHIFT:
                    m, s = (int(rng.integers(1, 2**15)), int(rng.integers(0, 31)))
                    if cv:
                        m, s = int(rng.integers(1, 2**12)), int(rng.integers(0, 20))   # float path: keep v*m exact in fp32
                        v2 = int(rng.integers(-2**11, 2**11))
                    else:
                        v2 = v
                elif qm == oracle.QM_ONLY_SHIFT:
                    m, s, v2 = 1, int(rng.integers(0, 31)), v
                else:
                    m, v2 = int(rng.integers(2**30, 2**31)), v
                    s = int(rng.integers(0, 31)) if cv else -int(rng.integers(0, 31))   # CV18xx negates the attribute
                rm = oracle.RM_HALF_AWAY if (cv or qm != oracle.QM_MULTIPLIER_SHIFT) else oracle.RM_HALF_UP
                got = oracle.apply_multiplier_rshift(v2, m, s, qm, rm, bool(cv))
                assert got == R.ref_apply_multiplier_rshift(v2, m, s, qm, rm, cv), (v2, m, s, qm, rm, cv)


@pytest.mark.skipif(not oracle.ref_float16_available(), reason="compiled reference Float16.cpp not present")
def test_bf16_conversion_matches_compiled_reference():
    """The oracle's BF16 rounding against the reference's own f32_to_bf16 (lib/Support/Float16.cpp, BM168x branch) on
    random bit patterns (normals, denormals, infinities, NaNs) and the edges of every case."""
    R = oracle.ref_float16()
    rng = np.random.default_rng(0)
    edge = [0, 0x80000000, 0x7f800000, 0xff800000, 0x7fc00000, 0x7f800001, 0x00000001, 0x007fffff, 0x007f8000, 0x007f7fff,
            0x807f8000, 0x807f7fff, 0x3f808000, 0x3f818000, 0x3f807fff, 0x3f808001, 0x7f7fffff, 0x7f7f8000, 0x7f7f7fff,
            0x00800000, 0x00808000]
    bits = np.concatenate([rng.integers(0, 2**32, 60000, dtype=np.uint64).astype(np.uint32), np.array(edge, dtype=np.uint32)])
    f = oracle.lib().orc_f32_to_bf16_bits
    for v, b in zip(bits.view(np.float32), bits):
        assert int(f(float(v))) == int(R.ref_f32_to_bf16(float(v))), hex(int(b))
    for b in list(range(0, 1 << 16, 7)) + [0x7f80, 0xff80, 0x7fc0, 0x0001, 0x8001]:
        got = oracle.bf16_bits_to_f32(np.array([b], dtype=np.uint16))[0]
        want = np.float32(R.ref_bf16_to_f32(b))
        assert got.tobytes() == want.tobytes() or (np.isnan(got) and np.isnan(want)), hex(b)


@pytest.mark.skipif(not oracle.ref_float16_available(), reason="compiled reference Float16.cpp not present")
def test_f16_conversion_matches_compiled_reference():
    """The oracle's F16 rounding against the reference's own f32_to_f16 / f16_to_f32 (lib/Support/Float16.cpp:763-786):
    random bit patterns whose magnitude fp16 can express or nearly so, the subnormal band, ties, overflow to infinity,
    infinities, NaNs, zeros, fp32 denormals; and every fp16 pattern back to fp32.  (Inputs below 2^-63 make the
    reference shift by 64 bits or more, which C leaves undefined: not compared.)"""
    R = oracle.ref_float16()
    rng = np.random.default_rng(1)
    exps = rng.integers(127 - 40, 127 + 18, 60000).astype(np.uint32)       # 2^-40 .. 2^17
    bits = (rng.integers(0, 2, 60000).astype(np.uint32) << 31) | (exps << 23) | rng.integers(0, 1 << 23, 60000).astype(np.uint32)
    edge = [0, 0x80000000, 0x7f800000, 0xff800000, 0x7fc00000, 0x7f800001, 0x00000001, 0x007fffff, 0x477fe000, 0x477ff000,
            0x477fefff, 0x477ff001, 0xc77ff000, 0x47800000, 0x38800000, 0x387fffff, 0x387fe000, 0x33800000, 0x33000000,
            0x33000001, 0x32ffffff, 0x3c001000, 0x3c003000, 0x3c000fff, 0x3c001001, 0x7f7fffff, 0xb3000001]
    bits = np.concatenate([bits, np.array(edge, dtype=np.uint32)])
    f = oracle.lib().orc_f32_to_f16_bits
    for v, b in zip(bits.view(np.float32), bits):
        assert int(f(float(v))) == int(R.ref_f32_to_f16(float(v))) & 0xffff, hex(int(b))
    # and numpy's IEEE conversion agrees on everything but the NaN pattern: what the kernels' hardware rounding computes
    finite = bits.view(np.float32)[np.isfinite(bits.view(np.float32))]
    with np.errstate(over="ignore"):
        assert np.array_equal(oracle.f32_to_f16_bits(finite[:5000]), finite[:5000].astype(np.float16).view(np.uint16))
    g = oracle.lib().orc_f16_bits_to_f32
    for h in range(1 << 16):
        got, want = np.float32(g(h)), np.float32(R.ref_f16_to_f32(h))
        assert got.tobytes() == want.tobytes() or (np.isnan(got) and np.isnan(want)), hex(h)


def test_top_fp32_oracle_against_onednn():
    """The fp32 Top-dialect restatements (convolution, pooling) against torch's CPU operators, which call oneDNN - the
    library top::ConvOp / top::MaxPoolOp / top::AvgPoolOp call (lib/Support/Dnnl/Conv.cpp, Pool.cpp)."""
    torch = pytest.importorskip("torch")
    F = torch.nn.functional
    rng = np.random.default_rng(0)
    x = rng.standard_normal((2, 8, 9, 11)).astype(np.float32)
    w = rng.standard_normal((12, 4, 3, 3)).astype(np.float32)
    b = rng.standard_normal(12).astype(np.float32)
    got = oracle.top_conv2d_f32(x, w, b, stride=(2, 1), pads=(1, 1, 2, 2), dilation=(1, 2), groups=2, do_relu=True, relu_limit=3.0)
    ref = F.conv2d(F.pad(torch.from_numpy(x), (2, 2, 1, 1)), torch.from_numpy(w), torch.from_numpy(b), stride=(2, 1),
                   dilation=(1, 2), groups=2).clamp(0, 3).numpy()
    assert got.shape == ref.shape and np.allclose(got, ref, rtol=1e-5, atol=1e-5)
    t = torch.from_numpy(x)
    assert np.array_equal(oracle.top_pool2d_f32(x, kernel=(3, 3), stride=(2, 2), pads=(1, 1, 1, 1), is_max=True),
                          F.max_pool2d(t, 3, 2, 1).numpy())
    for cip in (True, False):
        assert np.allclose(oracle.top_pool2d_f32(x, kernel=(3, 3), stride=(2, 2), pads=(1, 1, 1, 1), is_max=False, count_include_pad=cip),
                           F.avg_pool2d(t, 3, 2, 1, count_include_pad=cip).numpy(), rtol=1e-6, atol=1e-6)
