"""CPU tests of the calibration host logic: the (threshold, bins) schedule against the reference's golden
streaming histograms, and the sharded driver on 2 gloo ranks with the oracle standing in for the kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from tpu_mlir_b200.calibration import ShardedCalibrator, bin_schedule, table_threshold

G = os.path.join(os.path.dirname(__file__), "golden")


class OracleMath:
    """The kernels' interface served by the CPU oracle (tests only)."""

    def minmax(self, x, samples=1):
        a = x.reshape(samples, -1)
        return torch.stack([a.min(dim=1).values, a.max(dim=1).values], dim=1)

    def histogram_into(self, hist, x, th, nbins):
        a = x.reshape(len(th), -1).numpy()
        h = hist.numpy()
        for s in range(len(th)):
            if nbins[s]:
                oracle.histogram(a[s], th[s], int(nbins[s]), into=h)

    def find_thresholds(self, hists, widths, dst_bins=128):
        out = []
        for h, w in zip(hists, widths):
            hf, wf = oracle.fold_for_kld(h.numpy(), np.float32(w), dst_bins)
            out.append(oracle.kl_diversity_hist(hf, wf, dst_bins))
        return np.array(out, dtype=np.float32)


@pytest.mark.parametrize("name", ["grow", "zero_then", "reset"])
def test_schedule_reproduces_reference_stream(name):
    z = np.load(os.path.join(G, "calib_hist.npz"))
    n = int(z[f"stream/{name}/n"])
    samples = [z[f"stream/{name}/x{i}"] for i in range(n)]
    sc = bin_schedule([s.min() for s in samples], [s.max() for s in samples])
    want = z[f"stream/{name}/hist"]
    assert sc.final_bins == len(want)
    assert sc.width.tobytes() == z[f"stream/{name}/width"].tobytes()
    assert sc.min.tobytes() == z[f"stream/{name}/min"].tobytes() and sc.max.tobytes() == z[f"stream/{name}/max"].tobytes()
    total = np.zeros(sc.final_bins, np.int32)
    for a, th, nb in zip(samples, sc.th, sc.nbins):
        if nb:
            oracle.histogram(a, th, int(nb), into=total)
    assert np.array_equal(total, want)


def test_schedule_edge_cases():
    sc = bin_schedule([], [])
    assert sc.final_bins == 0
    sc = bin_schedule([0.0, 0.0], [0.0, 0.0])
    assert sc.final_bins == 0 and not sc.nbins.any()
    sc = bin_schedule([-1.0, -0.5, -3.0], [0.5, 0.2, 1.0])
    assert sc.nbins[0] == 2048 and sc.nbins[1] == 2048 and sc.nbins[2] > 2048 and sc.final_bins == sc.nbins[2]
    assert table_threshold(5.0, 3.0) == 3.0 and table_threshold(0.0, 3.0) == 1e-5


def _forward(batch):
    x = batch
    return {"a": torch.relu(x) * 2.0, "b": x * x - 1.0, "zero": torch.zeros_like(x[:, :4])}


def _make_samples(total):
    rng = np.random.default_rng(99)
    scales = rng.uniform(0.5, 3.0, size=total).astype(np.float32)
    return torch.from_numpy((rng.standard_normal((total, 3000)).astype(np.float32)) * scales[:, None])


def _single_process_reference(samples):
    res = {}
    for name in ("a", "b", "zero"):
        st = oracle.StreamingHistogram(2048)
        for i in range(samples.shape[0]):
            st.update(_forward(samples[i:i + 1])[name].numpy())
        if st.hist is None:
            res[name] = (None, None, None)
            continue
        hf, wf = oracle.fold_for_kld(st.hist, st.width)
        res[name] = (st.hist, st.width, oracle.kl_diversity_hist(hf, wf))
    return res


def _worker(rank, world, port, total, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    samples = _make_samples(total)
    per = total // world
    mine = samples[rank * per:(rank + 1) * per]
    batches = [mine[i:i + 3] for i in range(0, per, 3)]
    cal = ShardedCalibrator(_forward, math=OracleMath(), dist=dist)
    res = cal.run(batches, samples_per_rank=per)
    shard_dir = os.environ.get("B200Q_TEST_SHARD_DIR")
    if shard_dir:
        from tpu_mlir_b200.calibration import save_shard
        save_shard(cal, os.path.join(shard_dir, f"shard{rank}.npz"))
    if rank == 0:
        q.put({n: (cal.histograms[n].numpy().copy(), r.width, r.kl, r.bins, r.threshold) for n, r in res.items()})
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_calibrator_two_ranks_matches_streaming_reference(tmp_path, monkeypatch):
    monkeypatch.setenv("B200Q_TEST_SHARD_DIR", str(tmp_path))
    total, world = 12, 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, total, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    want = _single_process_reference(_make_samples(total))
    for name in ("a", "b"):
        hist, width, kl = want[name]
        g_hist, g_width, g_kl, g_bins, g_th = got[name]
        assert g_bins == len(hist) and np.array_equal(g_hist, hist), name
        assert np.float32(g_width).tobytes() == np.float32(width).tobytes()
        assert np.float32(g_kl).tobytes() == np.float32(kl).tobytes()
    assert got["zero"][3] == 0 and got["zero"][4] == 1e-5
    # the per-rank shard files re-merge to the same result without the ranks; a missing shard is refused
    from tpu_mlir_b200.calibration import merge_shards
    merged = merge_shards([str(tmp_path / "shard1.npz"), str(tmp_path / "shard0.npz")], math=OracleMath())
    for name in ("a", "b", "zero"):
        assert merged[name].bins == got[name][3] and np.float32(merged[name].kl).tobytes() == np.float32(got[name][2]).tobytes()
        assert merged[name].threshold == got[name][4]
    with pytest.raises(ValueError):
        merge_shards([str(tmp_path / "shard0.npz")], math=OracleMath())


def test_single_process_path():
    samples = _make_samples(6)
    cal = ShardedCalibrator(_forward, math=OracleMath(), dist=None)
    res = cal.run([samples[0:4], samples[4:6]], samples_per_rank=6)
    want = _single_process_reference(samples)
    assert np.array_equal(cal.histograms["b"].numpy(), want["b"][0])
    assert np.float32(res["b"].kl).tobytes() == np.float32(want["b"][2]).tobytes()


def test_bin_schedule_many_equals_the_scalar_recurrence():
    """The per-tensor recurrence vectorised over tensors (what the sharded calibrator runs on every rank) against the
    scalar form, including tensors that never contribute, all-zero samples, no growth, and a reset past 8M bins."""
    from tpu_mlir_b200.calibration import bin_schedule, bin_schedule_many
    rng = np.random.default_rng(0)
    T, S = 24, 300
    smax = np.abs(rng.standard_normal((T, S)).astype(np.float32)) * rng.uniform(0.1, 30, (T, 1)).astype(np.float32)
    smin = -np.abs(rng.standard_normal((T, S)).astype(np.float32)) * rng.uniform(0, 30, (T, 1)).astype(np.float32)
    smin[3] = 0
    smax[5, :10] = 0
    smin[5, :10] = 0
    smax[7], smin[7] = 1, -1
    smax[7, 0], smin[7, 0], smax[7, 150] = 1e-6, 0, 5000.0
    smax[8], smin[8] = np.float32(2.5), np.float32(-1)
    smax[9], smin[9] = 0, 0
    many = bin_schedule_many(smin, smax)
    for t in range(T):
        a, b = bin_schedule(smin[t], smax[t]), many[t]
        assert np.array_equal(a.th, b.th) and np.array_equal(a.nbins, b.nbins), t
        assert a.final_bins == b.final_bins and a.width.tobytes() == b.width.tobytes(), t
        assert (a.min.tobytes(), a.max.tobytes(), a.abs_max.tobytes()) == (b.min.tobytes(), b.max.tobytes(), b.abs_max.tobytes()), t
    assert many[7].nbins[149] == 0 and many[7].nbins[150] == 2048 and many[7].final_bins == 2048 and many[9].final_bins == 0
