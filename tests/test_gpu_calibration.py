"""Calibration kernels on the GPU: histogram counts bit-exact against the oracle and the reference's golden
vectors, KLD thresholds identical to the reference's."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import oracle
import tpu_mlir_b200._lib as L
from tpu_mlir_b200.calibration import CaliMathB200, ShardedCalibrator, bin_schedule, kld_threshold_host

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def m():
    return CaliMathB200()


def test_minmax(m):
    rng = np.random.default_rng(0)
    for shape in [(1, 1), (1, 7), (5, 1000), (3, 802816), (64, 4097)]:
        x = rng.standard_normal(shape).astype(np.float32) * rng.uniform(0.1, 5)
        got = m.minmax(torch.from_numpy(x).cuda(), samples=shape[0]).cpu().numpy()
        assert np.array_equal(got[:, 0], x.min(axis=1)) and np.array_equal(got[:, 1], x.max(axis=1))
    # unaligned view (the vector path needs 16-byte alignment)
    base = torch.from_numpy(rng.standard_normal(10001).astype(np.float32)).cuda()
    got = m.minmax(base[1:], samples=1).cpu().numpy()
    assert got[0, 0] == base[1:].min().item() and got[0, 1] == base[1:].max().item()


def test_histogram_matches_reference_golden(m):
    z = np.load(os.path.join(G, "calib_hist.npz"))
    names = sorted({k.split("/")[1] for k in z.files if k.startswith("single/")})
    for name in names:
        x = z[f"single/{name}/x"]
        abs_max = max(abs(np.min(x)), abs(np.max(x)))
        for bins in (2048, 777):
            h, w = m.histogram(x, abs_max, bins)
            assert np.array_equal(h, z[f"single/{name}/{bins}/hist"]), (name, bins)
            assert np.float32(w).tobytes() == z[f"single/{name}/{bins}/width"].tobytes()


@pytest.mark.parametrize("bins", [2, 128, 2048, 6206, 49152, 50000, 300000, 2000000])
def test_histogram_matches_oracle_many_bin_counts(m, bins):
    """Includes bin counts where numpy's float32 bin edges move the top bins, and sizes beyond shared memory."""
    rng = np.random.default_rng(bins)
    x = (rng.standard_normal(200000) * 2).astype(np.float32)
    x[::17] = 0
    x[5] = np.abs(x).max()          # the abs-max itself lands in the last bin
    abs_max = np.float32(np.abs(x).max())
    want, _ = oracle.histogram(x, abs_max, bins)
    got, _ = m.histogram(x, abs_max, bins)
    assert np.array_equal(got, want)
    # a threshold below the data range: values beyond the last bin are dropped
    want, _ = oracle.histogram(x, abs_max / 3, bins)
    got, _ = m.histogram(x, abs_max / 3, bins)
    assert np.array_equal(got, want) and got.sum() < np.count_nonzero(x)


def test_histogram_quotient_is_exact_for_many_widths(m):
    """The kernel forms t / width from a reciprocal and two FMAs; the counts must equal float32 division for widths of
    every magnitude, values on bin boundaries, and the widths (significand all ones) that take the dividing path."""
    rng = np.random.default_rng(99)
    bins = 2048
    for i in range(48):
        if i < 40:
            th = np.float32(10.0 ** rng.uniform(-20, 20) * rng.uniform(1, 10))
        else:   # width = th / 2047 with an all-ones significand: th = width * 2047 rounded, then checked
            w = np.nextafter(np.float32(2.0 ** rng.integers(-10, 10)), np.float32(0))
            th = np.float32(w * np.float32(bins - 1))
        width = np.float32(th) / np.float32(bins - 1)
        k = rng.integers(0, bins, 60000).astype(np.float32)
        # values at and just around the rounding boundaries (k +- 0.5) * width, plus random ones
        x = np.concatenate([(k + np.float32(0.5)) * width, np.nextafter((k + np.float32(0.5)) * width, np.float32(0)),
                            np.nextafter((k + np.float32(0.5)) * width, np.float32(np.inf)),
                            rng.uniform(0, float(th), 60000).astype(np.float32)]).astype(np.float32)
        x *= rng.choice(np.array([-1, 1], np.float32), x.size)
        want, _ = oracle.histogram(x, th, bins)
        got, _ = m.histogram(x, th, bins)
        assert np.array_equal(got, want), (i, float(th))


def test_histogram_batch_with_schedule(m):
    rng = np.random.default_rng(3)
    S, n = 9, 5000
    x = (rng.standard_normal((S, n)) * rng.uniform(0.2, 4, size=(S, 1))).astype(np.float32)
    x[4] = 0
    sc = bin_schedule(x.min(axis=1), x.max(axis=1))
    hist = torch.zeros(sc.final_bins, dtype=torch.int32, device="cuda")
    m.histogram_into(hist, torch.from_numpy(x).cuda(), sc.th, sc.nbins)
    st = oracle.StreamingHistogram()
    for s in range(S):
        st.update(x[s])
    assert np.array_equal(hist.cpu().numpy(), st.hist)
    assert sc.width.tobytes() == np.float32(st.width).tobytes()


@pytest.mark.parametrize("name", ["grow", "zero_then", "reset"])
def test_combine_histogram_protocol_matches_reference(m, name):
    """The reference's math_impl protocol driven the way kld_calibrator.py:462-476 drives it."""
    z = np.load(os.path.join(G, "calib_hist.npz"))
    n = int(z[f"stream/{name}/n"])
    mn, mx, state = float("inf"), float("-inf"), None
    for i in range(n):
        a = z[f"stream/{name}/x{i}"]
        mn, mx = min(np.min(a), mn), max(np.max(a), mx)
        av = max(abs(mn), abs(mx))
        if np.abs(a).max() < 1e-8:
            continue
        act = m.prepare(a)
        if state is None:
            h, w = m.histogram(act, av, 2048)
            state = (h, w, mn, mx, av)
        else:
            state = m.combine_histogram(state, act, mn, mx, av, 2048)
    assert np.array_equal(state[0], z[f"stream/{name}/hist"])
    assert np.float32(state[1]).tobytes() == z[f"stream/{name}/width"].tobytes()
    assert np.float32(state[4]).tobytes() == z[f"stream/{name}/th"].tobytes()


def test_kld_matches_reference_golden(m):
    z = np.load(os.path.join(G, "calib_kld.npz"))
    names = sorted({k.split("/")[0] for k in z.files})
    hists = [torch.from_numpy(z[f"{n}/hist"]).cuda() for n in names]
    widths = [z[f"{n}/width"] for n in names]
    th, kl = m.find_thresholds(hists, widths, return_kl=True)
    for i, n in enumerate(names):
        want = z[f"{n}/threshold"]
        # the per-candidate KL values differ from the CPU's only through log10; report the margin on failure
        hf, wf = oracle.fold_for_kld(z[f"{n}/hist"], z[f"{n}/width"])
        _, kl_cpu = oracle.kl_diversity_hist(hf, wf, return_kl=True)
        k = len(kl_cpu)
        gap = np.sort(kl_cpu)[:2]
        assert th[i].tobytes() == want.tobytes(), (n, th[i], want, "two smallest KL on CPU:", gap,
                                                   "max |KL gpu - cpu|:", np.abs(kl[i][:k] - kl_cpu).max())
        assert np.allclose(kl[i][:k], kl_cpu, rtol=1e-5, atol=1e-7)


def test_reference_symbol_kl_diversity_hist():
    z = np.load(os.path.join(G, "calib_kld.npz"))
    for n in ("normal2048", "sparse", "huge_counts"):
        hf, wf = oracle.fold_for_kld(z[f"{n}/hist"], z[f"{n}/width"])
        assert kld_threshold_host(hf, wf).tobytes() == z[f"{n}/threshold"].tobytes()


def test_kld_random_against_oracle(m):
    rng = np.random.default_rng(5)
    hists, widths, want = [], [], []
    for t in range(10):
        bins = int(rng.choice([128, 2048, 2300, 5000, 16384]))
        x = (rng.standard_normal(60000) * rng.uniform(0.3, 3)).astype(np.float32)
        if t % 2:
            x = np.maximum(x, 0)
        h, w = oracle.histogram(x, np.abs(x).max(), bins)
        hf, wf = oracle.fold_for_kld(h, w)
        hists.append(torch.from_numpy(h).cuda())
        widths.append(w)
        want.append(oracle.kl_diversity_hist(hf, wf))
    got = m.find_thresholds(hists, widths)
    assert np.array_equal(got, np.array(want, dtype=np.float32))


@pytest.mark.parametrize("cache_bytes", [None, 0, 4 * 2 * 4 * 33 * 17 * 4 + 64],
                         ids=["whole_shard_kept", "second_forward", "first_batch_kept"])
def test_sharded_calibrator_single_gpu_matches_streaming_oracle(m, cache_bytes):
    """The three ways the second pass gets its activations: one region per tensor holding the whole shard (one kernel
    launch per tensor), nothing kept (the network runs again, as in the reference), and a kept prefix of the batches."""
    rng = np.random.default_rng(8)
    x = torch.from_numpy((rng.standard_normal((10, 4, 33, 17)) * rng.uniform(0.5, 2.5, size=(10, 1, 1, 1)))
                         .astype(np.float32)).cuda()

    def forward(b):
        return {"conv": torch.nn.functional.avg_pool2d(b, 3, 1, 1), "relu": torch.relu(b)}

    cal = ShardedCalibrator(forward, math=m)
    res = cal.run([x[0:4], x[4:8], x[8:10]], samples_per_rank=10, cache_bytes=cache_bytes)
    assert cal.cached_bytes == {None: 10 * 2 * 4 * 33 * 17 * 4, 0: 0}.get(cache_bytes, 4 * 2 * 4 * 33 * 17 * 4)
    for name in ("conv", "relu"):
        st = oracle.StreamingHistogram()
        for i in range(10):
            st.update(forward(x[i:i + 1])[name].cpu().numpy())
        assert np.array_equal(cal.histograms[name].cpu().numpy(), st.hist)
        hf, wf = oracle.fold_for_kld(st.hist, st.width)
        assert np.float32(res[name].kl).tobytes() == oracle.kl_diversity_hist(hf, wf).tobytes()
