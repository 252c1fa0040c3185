"""Activation calibration on the GPU: running min/max, streaming histogram and KLD threshold per tensor.

Mirrors the statistics half of the reference's ``ActivationCalibrator``
(python/calibration/kld_calibrator.py:364-477 ``process_statistic``, :321-347 ``find_threshold``) and its math
object (python/calibration/cali_math.py:27-143).  Two things differ in form, not in result:

* ``CaliMathB200`` offers the reference's ``prepare / histogram / combine_histogram`` protocol, computed by the
  kernels in libb200q.so.
* ``ShardedCalibrator`` runs the same statistics over samples that are sharded across ranks.  The reference's
  streaming histogram depends on the sample order only through the running abs-max (cali_math.py:82-103 keeps
  old counts in their bins when it grows the histogram), so it equals the sum over samples of per-sample
  histograms taken with a (threshold, bins) schedule derived from the per-sample min/max alone.  Pass 1 gathers
  the min/max of every sample (all-gather), every rank derives the identical schedule on the host, pass 2
  histograms the local samples into a buffer of the final size, one all-reduce (sum, int32) merges the ranks.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Sequence

import numpy as np

from . import _lib as L

MAX_GROWN_BINS = 8000000   # cali_math.py:96
MAX_KLD_BINS = 64 * 2048   # kld_calibrator.py:338
ALL_ZERO_EPS = 1e-8        # kld_calibrator.py:395


# ----------------------------------------------------------------------------------------------- host logic
@dataclass
class Schedule:
    """What each sample contributes to one tensor's histogram, and the final histogram geometry."""
    th: np.ndarray          # float32 [S] threshold used for sample s (0 where it contributes nothing)
    nbins: np.ndarray       # int32 [S] bins used for sample s (0 = skipped)
    final_bins: int         # length of the final histogram (0 if no sample contributed)
    width: np.float32       # bin width handed to the KLD search
    min: np.float32
    max: np.float32
    abs_max: np.float32


def bin_schedule(sample_min: Sequence[float], sample_max: Sequence[float], bin_num: int = 2048) -> Schedule:
    """Replays process_statistic + combine_histogram (kld_calibrator.py:391-398,:462-476; cali_math.py:82-103)
    on the per-sample (min, max) of one tensor, in sample order, in float32 like the reference."""
    smin = np.asarray(sample_min, dtype=np.float32)
    smax = np.asarray(sample_max, dtype=np.float32)
    S = len(smin)
    th_s = np.zeros(S, np.float32)
    nb_s = np.zeros(S, np.int32)
    run_min, run_max = float("inf"), float("-inf")
    th: Optional[np.float32] = None
    nb = 0
    width = np.float32(0)
    last_reset = 0
    for i in range(S):
        run_min = min(smin[i], run_min)
        run_max = max(smax[i], run_max)
        abs_value = max(abs(run_min), abs(run_max))
        if max(abs(smin[i]), abs(smax[i])) < ALL_ZERO_EPS:      # np.abs(activation).max() < 1e-8: no histogram
            continue
        if th is None:
            th, nb = np.float32(abs_value), bin_num
            width = np.float32(th / (nb - 1))
        elif abs_value > th:
            old_step = np.float32(th / nb)
            inc = int((np.float32(abs_value) - th) // old_step + 1)
            if inc + nb > MAX_GROWN_BINS:
                th, nb = np.float32(abs_value), bin_num          # starts over with this sample only
                last_reset = i
            else:
                th = np.float32(inc * old_step + th)
                nb = inc + nb
            width = np.float32(th / (nb - 1))
        th_s[i], nb_s[i] = th, nb
    nb_s[:last_reset] = 0
    th_s[:last_reset] = 0
    amax = np.float32(max(abs(run_min), abs(run_max))) if S else np.float32(0)
    return Schedule(th=th_s, nbins=nb_s, final_bins=int(nb), width=np.float32(width), min=np.float32(run_min),
                    max=np.float32(run_max), abs_max=amax)


def bin_schedule_many(sample_min: np.ndarray, sample_max: np.ndarray, bin_num: int = 2048) -> List[Schedule]:
    """``bin_schedule`` for T tensors at once: ``sample_min / sample_max`` are float32 [T, S], the results are identical
    to the scalar form (tested).  The recurrence cannot be reordered, but its state (threshold, bin count) only changes
    at a sample that raises a tensor's running absolute maximum (or starts it): the running extrema of all samples are
    accumulated in one pass, the recurrence's step runs only at the columns where some tensor's running maximum
    rises - one set of numpy operations over the T tensors, in the same float32 arithmetic as the scalar form - and the
    columns in between are filled from the unchanged state.  With thousands of samples and tens of tensors this keeps
    the host out of the calibration's critical path (every rank computes the same schedule)."""
    smin = np.ascontiguousarray(sample_min, dtype=np.float32)
    smax = np.ascontiguousarray(sample_max, dtype=np.float32)
    T, S = smin.shape
    th_s = np.zeros((T, S), np.float32)
    nb_s = np.zeros((T, S), np.int32)
    run_min = np.full(T, np.inf, np.float32)
    run_max = np.full(T, -np.inf, np.float32)
    th = np.zeros(T, np.float32)
    nb = np.zeros(T, np.int64)
    started = np.zeros(T, bool)
    width = np.zeros(T, np.float32)
    last_reset = np.zeros(T, np.int64)
    one = np.float32(1)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        if S:
            run_min_all = np.minimum.accumulate(smin, axis=1)
            run_max_all = np.maximum.accumulate(smax, axis=1)
            abs_all = np.maximum(np.abs(run_min_all), np.abs(run_max_all))
            live_all = ~(np.maximum(np.abs(smin), np.abs(smax)) < np.float32(ALL_ZERO_EPS))
            rises = np.ones(S, bool)
            rises[1:] = (abs_all[:, 1:] > abs_all[:, :-1]).any(axis=0) | (abs_all[:, 1:] != abs_all[:, 1:]).any(axis=0)
            run_min, run_max = run_min_all[:, -1].copy(), run_max_all[:, -1].copy()
            events = np.flatnonzero(rises)
        else:
            events = np.zeros(0, np.int64)
        filled = 0          # columns [0, filled) of th_s / nb_s are final
        k = 0
        forced = -1         # a column that must run although no maximum rises there (see `pending`)
        while True:
            nxt = int(events[k]) if k < events.size else S
            if 0 <= forced < nxt:
                i = forced
            elif nxt < S:
                i = nxt
                k += 1
            else:
                break
            forced = -1
            if i > filled:   # the state did not change in [filled, i)
                lv = live_all[:, filled:i]
                th_s[:, filled:i] = np.where(lv, th[:, None], 0)
                nb_s[:, filled:i] = np.where(lv, nb[:, None], 0)
            abs_value = abs_all[:, i]
            live = live_all[:, i]
            first = live & ~started
            grow = live & started & (abs_value > th)
            if first.any():
                th = np.where(first, abs_value, th)
                nb = np.where(first, bin_num, nb)
                started |= first
            if grow.any():
                old_step = th / nb.astype(np.float32)
                inc = (np.floor_divide(abs_value - th, old_step) + one)
                inc = np.where(grow & np.isfinite(inc), inc, 0).astype(np.int64)
                reset = grow & (inc + nb > MAX_GROWN_BINS)
                ext = grow & ~reset
                th = np.where(ext, inc.astype(np.float32) * old_step + th, th)
                nb = np.where(ext, inc + nb, nb)
                th = np.where(reset, abs_value, th)
                nb = np.where(reset, bin_num, nb)
                last_reset = np.where(reset, i, last_reset)
            upd = first | grow
            if upd.any():
                width = np.where(upd, th / (nb - 1).astype(np.float32), width)
            th_s[:, i] = np.where(live, th, 0)
            nb_s[:, i] = np.where(live, nb, 0)
            filled = i + 1
            # float32 rounding can leave a grown threshold a hair below the maximum it grew for; the scalar form then
            # grows again at the tensor's next live sample even though no maximum rises there: run the next column too
            if i + 1 < S and (started & (abs_value > th)).any():
                forced = i + 1
        if S > filled:
            lv = live_all[:, filled:S]
            th_s[:, filled:S] = np.where(lv, th[:, None], 0)
            nb_s[:, filled:S] = np.where(lv, nb[:, None], 0)
    out = []
    for t in range(T):
        lr = int(last_reset[t])
        th_s[t, :lr] = 0
        nb_s[t, :lr] = 0
        amax = np.float32(max(abs(run_min[t]), abs(run_max[t]))) if S else np.float32(0)
        out.append(Schedule(th=th_s[t], nbins=nb_s[t], final_bins=int(nb[t]), width=np.float32(width[t]),
                            min=np.float32(run_min[t]) if S else np.float32(np.inf),
                            max=np.float32(run_max[t]) if S else np.float32(-np.inf), abs_max=amax))
    return out


def table_threshold(kl: float, abs_max: float) -> float:
    """calibration_result.canonicalize (python/calibration/utils.py:53-69) and the 1e-5 floor of
    dump_cali_table (kld_calibrator.py:848-851)."""
    th = min(float(kl), float(abs_max))
    return th if th > 1e-5 else 1e-5


# ----------------------------------------------------------------------------------------------- GPU math
class CaliMathB200:
    """The reference's math_impl protocol (cali_math.py:27-143: prepare / histogram / combine_histogram) on the
    GPU.  Arrays passed to ``prepare`` stay on the device; histograms come back as int32 numpy arrays."""

    def __init__(self, device: Optional[int] = None):
        import torch
        self.torch = torch
        if not torch.cuda.is_available():
            raise L.B200QError(L.ERR_NO_DEVICE, "CaliMathB200 needs a CUDA device (there is no CPU fallback)")
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None else device)
        self.ctx = C.c_void_p()
        L.check(L.lib().b200q_calib_create(C.byref(self.ctx)))

    def __del__(self):
        try:
            if self.ctx:
                L.lib().b200q_calib_destroy(C.byref(self.ctx))
        except Exception:
            pass

    # -- device helpers
    def _dev(self, a):
        t = self.torch
        if isinstance(a, t.Tensor):
            return a.to(self.device, dtype=t.float32).contiguous()
        return t.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(self.device)

    def _stream(self):
        return C.c_void_p(self.torch.cuda.current_stream(self.device).cuda_stream)

    def prepare(self, array):
        return self._dev(array)

    def minmax(self, x, samples: int = 1):
        """Per-sample (min, max) of a device tensor viewed as [samples, -1]; returns a device tensor [samples, 2]."""
        x = self._dev(x)
        n = x.numel() // samples
        out = self.torch.empty((samples, 2), dtype=self.torch.float32, device=self.device)
        L.check(L.lib().b200q_calib_minmax(self.ctx, C.c_void_p(x.data_ptr()), n, samples,
                                           C.c_void_p(out.data_ptr()), self._stream()))
        return out

    def histogram_into(self, hist, x, th: np.ndarray, nbins: np.ndarray):
        """hist (device int32) += per-sample histograms of x viewed as [len(th), -1]."""
        x = self._dev(x)
        S = len(th)
        th = np.ascontiguousarray(th, dtype=np.float32)
        nbins = np.ascontiguousarray(nbins, dtype=np.int32)
        L.check(L.lib().b200q_calib_histogram(self.ctx, C.c_void_p(x.data_ptr()), x.numel() // S, S,
                                              th.ctypes.data_as(C.POINTER(C.c_float)),
                                              nbins.ctypes.data_as(C.POINTER(C.c_int32)),
                                              C.c_void_p(hist.data_ptr()), hist.numel(), self._stream()))

    def histogram(self, ndarray, abs_max, bin_num: int = 2048):
        """CaliMathCpu.histogram (cali_math.py:68-80): returns (int32 counts, float32 width)."""
        hist = self.torch.zeros(bin_num, dtype=self.torch.int32, device=self.device)
        abs_max = np.float32(abs_max)
        self.histogram_into(hist, self._dev(ndarray).reshape(-1), np.array([abs_max]), np.array([bin_num]))
        return hist.cpu().numpy(), np.float32(abs_max / np.float32(bin_num - 1))

    def combine_histogram(self, old_hist, arr, new_min, new_max, new_th, bin_num: int = 2048):
        """CaliMathCpu.combine_histogram (cali_math.py:82-103) with the histogram taken on the GPU."""
        (old, old_edges, old_min, old_max, old_th) = old_hist
        if new_th <= old_th:
            hist, _ = self.histogram(arr, old_th, len(old))
            return (old + hist, old_edges, min(old_min, new_min), max(old_max, new_max), old_th)
        old_bins = len(old)
        old_step = old_th / old_bins
        inc = int((new_th - old_th) // old_step + 1)
        new_bins = inc + old_bins
        if new_bins > MAX_GROWN_BINS:
            hist, edges = self.histogram(arr, new_th, bin_num)
            return (hist, edges, min(old_min, new_min), max(old_max, new_max), new_th)
        new_th = inc * old_step + old_th
        hist, edges = self.histogram(arr, new_th, new_bins)
        hist[0:old_bins] += old
        return (hist, edges, min(old_min, new_min), max(old_max, new_max), new_th)

    def find_thresholds(self, hists, widths, dst_bins: int = 128, return_kl: bool = False):
        """find_threshold (kld_calibrator.py:321-347) for a list of device int32 histograms."""
        T = len(hists)
        ptrs = (C.c_void_p * T)(*[h.data_ptr() for h in hists])
        nb = (C.c_int64 * T)(*[h.numel() for h in hists])
        w = (C.c_float * T)(*[float(np.float32(x)) for x in widths])
        out = (C.c_float * T)()
        kl = (C.c_float * (T * 1024))() if return_kl else None
        L.check(L.lib().b200q_calib_find_thresholds(self.ctx, T, ptrs, nb, w, dst_bins, out, kl, self._stream()))
        th = np.frombuffer(out, dtype=np.float32).copy()
        if return_kl:
            return th, np.frombuffer(kl, dtype=np.float32).reshape(T, 1024).copy()
        return th


def kld_threshold_host(hist: np.ndarray, width, dst_bins: int = 128) -> np.float32:
    """BaseKldCalibrator.kld_threshold (kld_calibrator.py:55-59) through the reference's own C symbol, served
    by libb200q.so."""
    h = np.ascontiguousarray(hist, dtype=np.int32)
    return np.float32(L.lib().kl_diversity_hist(h.ctypes.data_as(C.POINTER(C.c_int)), C.c_float(float(width)),
                                                C.c_longlong(h.size), C.c_longlong(dst_bins)))


# ----------------------------------------------------------------------------------------------- sharded driver
@dataclass
class TensorResult:
    name: str
    min: float
    max: float
    abs_max: float
    bins: int
    width: float
    kl: float
    threshold: float     # what the calibration table would hold (min(kl, abs_max), floor 1e-5)


class ShardedCalibrator:
    """Statistics + KLD thresholds for the activations of a forward function, samples sharded across ranks.

    ``forward(batch) -> dict name -> device float32 tensor [B, ...]`` produces every activation of interest for a
    batch of samples; ``shard`` is the local contiguous range of the global sample order.  ``math`` defaults to
    the GPU implementation; ``dist`` is a torch.distributed-like module (None = single process).
    """

    def __init__(self, forward: Callable, math=None, dist=None, bin_num: int = 2048, dst_bins: int = 128):
        self.forward = forward
        self.math = math if math is not None else CaliMathB200()
        self.dist = dist if (dist is not None and dist.is_initialized() and dist.get_world_size() > 1) else None
        self.bin_num = bin_num
        self.dst_bins = dst_bins

    def _world(self):
        return (self.dist.get_rank(), self.dist.get_world_size()) if self.dist else (0, 1)

    def run(self, batches: Iterable, samples_per_rank: int, cache_bytes: Optional[int] = None) -> Dict[str, TensorResult]:
        """``batches`` must be re-iterable (it is walked twice) and cover exactly ``samples_per_rank`` local
        samples in order; rank r holds global samples [r*samples_per_rank, (r+1)*samples_per_rank).

        The activations of the first pass stay on the device for the second pass while they fit in ``cache_bytes``
        (default: the device memory that is free when the run starts less 24 GB); batches past that budget are
        forwarded a second time, as the reference does for every batch (kld_calibrator.py:629-760 runs the network
        once for min/max and once more for the histograms).  ``self.timings`` holds the seconds spent per phase."""
        import time
        import torch
        rank, world = self._world()
        m = self.math
        tm: Dict[str, float] = {}
        cuda = torch.cuda.is_available()

        def lap(key, t0):
            if cuda:
                torch.cuda.synchronize()
            tm[key] = tm.get(key, 0.0) + time.perf_counter() - t0
            return time.perf_counter()

        if cache_bytes is None:
            # what the driver has free plus what torch's allocator holds without using (blocks of an earlier run), less
            # 24 GB for the forward
            idle = torch.cuda.memory_reserved() - torch.cuda.memory_allocated() if cuda else 0
            cache_bytes = max(0, torch.cuda.mem_get_info()[0] + idle - (24 << 30)) if cuda else 0
        # ---- pass 1: per-sample min/max of every tensor
        t0 = time.perf_counter()
        names: List[str] = []
        local: Dict[str, List] = {}
        cache: List[Optional[Dict]] = []
        held = 0
        # The kept activations are copied into a few large slabs: holding the forward's own tensors would make the
        # allocator ask the driver for fresh memory on every batch (slow once peer access is enabled by NCCL), while a
        # copy costs a fraction of the forward and lets the forward reuse its blocks.
        SLAB = 4 << 30
        slabs: List = []
        slab_off = 0

        def keep(acts):
            nonlocal slab_off
            out = {}
            for n in names:
                a = acts[n]
                if not a.is_cuda or a.dtype != torch.float32 or not a.is_contiguous():
                    out[n] = a
                    continue
                nbytes = (a.numel() * 4 + 255) & ~255
                if not slabs or slab_off + nbytes > slabs[-1].numel():
                    ta = time.perf_counter()
                    slabs.append(torch.empty(max(SLAB, nbytes), dtype=torch.uint8, device=a.device))
                    tm["cache_alloc"] = tm.get("cache_alloc", 0.0) + time.perf_counter() - ta
                    slab_off = 0
                v = slabs[-1][slab_off:slab_off + a.numel() * 4].view(torch.float32).view(a.shape)
                v.copy_(a)
                slab_off += nbytes
                out[n] = v
            return out

        # When the activations of the WHOLE shard fit, every tensor gets one region [samples, ...] and the kernels run
        # once per tensor over all its samples (at most CHUNK samples per launch) instead of once per tensor and batch:
        # 2 x 73 launches for ResNet-50 instead of 2 x 73 per batch, whose fixed cost (not their bytes) set the pace.
        CHUNK = 1024
        store: Optional[Dict] = None
        filled = 0
        for batch in batches:
            acts = self.forward(batch)
            if not names:
                names = list(acts.keys())
                local = {n: [] for n in names}
                per_sample = sum(acts[n][0].numel() * 4 for n in names)
                if all(acts[n].is_cuda and acts[n].dtype == torch.float32 for n in names) and per_sample * samples_per_rank <= cache_bytes:
                    ta = time.perf_counter()
                    store = {n: torch.empty((samples_per_rank,) + tuple(acts[n].shape[1:]), dtype=torch.float32, device=acts[n].device)
                             for n in names}
                    tm["cache_alloc"] = time.perf_counter() - ta
                    held = per_sample * samples_per_rank
            if store is not None:
                B = acts[names[0]].shape[0]
                for n in names:
                    store[n][filled:filled + B].copy_(acts[n])
                filled += B
                cache.append(None)
                del acts
                continue
            for n in names:
                a = acts[n]
                local[n].append(m.minmax(a, samples=a.shape[0]))
            need = sum(acts[n].numel() * acts[n].element_size() for n in names)
            if held + need <= cache_bytes and (not cache or cache[-1] is not None):
                cache.append(keep(acts))
                held += need
            else:
                cache.append(None)
            del acts
        if store is not None:
            assert filled == samples_per_rank, "batches do not cover samples_per_rank samples"
            for n in names:
                for c0 in range(0, samples_per_rank, CHUNK):
                    c1 = min(c0 + CHUNK, samples_per_rank)
                    local[n].append(m.minmax(store[n][c0:c1], samples=c1 - c0))
        mm_local = torch.stack([torch.cat(local[n], dim=0) for n in names])            # [T, S_local, 2]
        assert mm_local.shape[1] == samples_per_rank, "batches do not cover samples_per_rank samples"
        t0 = lap("pass1_forward_minmax", t0)
        if self.dist:
            gathered = [torch.empty_like(mm_local) for _ in range(world)]
            self.dist.all_gather(gathered, mm_local.contiguous())
            mm_all = torch.cat(gathered, dim=1)                                          # rank-major = sample order
        else:
            mm_all = mm_local
        mm_all = mm_all.cpu().numpy()
        t0 = lap("gather_minmax", t0)
        # ---- identical schedule on every rank
        sched = dict(zip(names, bin_schedule_many(mm_all[:, :, 0], mm_all[:, :, 1], self.bin_num)))
        t0 = lap("bin_schedule", t0)
        # ---- pass 2: histograms of the local samples into final-size buffers (one flat allocation)
        sizes = [max(sched[n].final_bins, 1) for n in names]
        offs = np.concatenate(([0], np.cumsum(sizes)))
        flat = torch.zeros(int(offs[-1]), dtype=torch.int32, device=mm_local.device)
        views = {n: flat[int(offs[t]):int(offs[t + 1])] for t, n in enumerate(names)}
        s0 = rank * samples_per_rank
        done = 0
        if store is not None:
            for n in names:
                sc = sched[n]
                for c0 in range(0, samples_per_rank, CHUNK):
                    c1 = min(c0 + CHUNK, samples_per_rank)
                    if sc.final_bins and sc.nbins[s0 + c0:s0 + c1].any():
                        m.histogram_into(views[n], store[n][c0:c1], sc.th[s0 + c0:s0 + c1], sc.nbins[s0 + c0:s0 + c1])
        for bi, batch in enumerate(batches if store is None else []):
            acts = cache[bi] if cache[bi] is not None else self.forward(batch)
            cache[bi] = None
            for n in names:
                a = acts[n]
                B = a.shape[0]
                sc = sched[n]
                lo = s0 + done
                if sc.final_bins and sc.nbins[lo:lo + B].any():
                    m.histogram_into(views[n], a, sc.th[lo:lo + B], sc.nbins[lo:lo + B])
            done += next(iter(acts.values())).shape[0]
            del acts
        store = None
        t0 = lap("pass2_histograms", t0)
        # this rank's own contribution, kept for save_shard (the all-reduce below overwrites `flat` with the sum)
        self._shard = dict(names=list(names), minmax=mm_local.cpu().numpy(), hist=flat.cpu().numpy().copy(), sizes=np.asarray(sizes, np.int64),
                           rank=rank, world=world, samples_per_rank=int(samples_per_rank), bin_num=int(self.bin_num))
        self.allreduce_bytes = int(flat.numel() * 4) if self.dist else 0
        self.cached_bytes = int(held)
        if self.dist:
            self.dist.all_reduce(flat)                                                   # sum of int32 counts
        t0 = lap("allreduce_histograms", t0)
        # ---- KLD
        live = [n for n in names if sched[n].final_bins]
        kl = m.find_thresholds([views[n] for n in live], [sched[n].width for n in live], self.dst_bins) if live else []
        out: Dict[str, TensorResult] = {}
        for n in names:
            sc = sched[n]
            k = float(kl[live.index(n)]) if n in live else 0.0
            out[n] = TensorResult(name=n, min=float(sc.min), max=float(sc.max), abs_max=float(sc.abs_max),
                                  bins=sc.final_bins, width=float(sc.width), kl=k,
                                  threshold=table_threshold(k, sc.abs_max) if n in live else 1e-5)
        lap("kld", t0)
        self.timings = tm
        self.histograms = {n: views[n] for n in names}
        return out


def save_shard(calibrator: ShardedCalibrator, path: str) -> None:
    """Persist this rank's part of a finished ``run``: its per-sample (min, max) pairs and its local histograms (before
    the all-reduce), so that a calibration can be re-merged without the ranks, or one shard recomputed after a failure
    (the reference keeps only the final table, kld_calibrator.py:804-884)."""
    sh = calibrator._shard
    np.savez(path, names=np.array(sh["names"]), minmax=sh["minmax"], hist=sh["hist"], sizes=sh["sizes"],
             meta=np.array([sh["rank"], sh["world"], sh["samples_per_rank"], sh["bin_num"]], np.int64))


def merge_shards(paths: Sequence[str], math=None, dst_bins: int = 128) -> Dict[str, TensorResult]:
    """Rebuild the result of a sharded run from the files ``save_shard`` wrote, one per rank: the bin schedule is
    recomputed from all ranks' (min, max) pairs in rank order, the int32 histograms are summed (what the all-reduce
    does) and the thresholds searched again.  Raises if a shard is missing or was histogrammed under another schedule
    (e.g. recomputed with different samples)."""
    import torch
    shards = sorted((dict(np.load(p)) for p in paths), key=lambda d: int(d["meta"][0]))
    world = int(shards[0]["meta"][1])
    if [int(d["meta"][0]) for d in shards] != list(range(world)):
        raise ValueError(f"need one shard per rank 0..{world - 1}, got ranks {[int(d['meta'][0]) for d in shards]}")
    names = [str(n) for n in shards[0]["names"]]
    bin_num = int(shards[0]["meta"][3])
    for d in shards:
        if [str(n) for n in d["names"]] != names or int(d["meta"][3]) != bin_num or int(d["meta"][2]) != int(shards[0]["meta"][2]):
            raise ValueError("shards disagree on tensors, samples per rank or bin count")
    mm_all = np.concatenate([d["minmax"] for d in shards], axis=1)
    sched = bin_schedule_many(mm_all[:, :, 0], mm_all[:, :, 1], bin_num)
    sizes = np.array([max(sc.final_bins, 1) for sc in sched], np.int64)
    for d in shards:
        if not np.array_equal(d["sizes"], sizes):
            raise ValueError("a shard's histograms were built under a different bin schedule: recompute it with the same samples")
    flat = np.sum([d["hist"].astype(np.int64) for d in shards], axis=0).astype(np.int32)
    offs = np.concatenate(([0], np.cumsum(sizes)))
    m = math if math is not None else CaliMathB200()
    dev = "cuda" if isinstance(m, CaliMathB200) else "cpu"
    tflat = torch.from_numpy(flat).to(dev)
    views = [tflat[int(offs[t]):int(offs[t + 1])] for t in range(len(names))]
    live = [t for t, sc in enumerate(sched) if sc.final_bins]
    kl = m.find_thresholds([views[t] for t in live], [sched[t].width for t in live], dst_bins) if live else []
    out: Dict[str, TensorResult] = {}
    for t, n in enumerate(names):
        sc = sched[t]
        k = float(kl[live.index(t)]) if t in live else 0.0
        out[n] = TensorResult(name=n, min=float(sc.min), max=float(sc.max), abs_max=float(sc.abs_max), bins=sc.final_bins,
                              width=float(sc.width), kl=k, threshold=table_threshold(k, sc.abs_max) if t in live else 1e-5)
    return out


def dump_cali_table(path: str, results: Dict[str, TensorResult], *, order: Optional[List[str]] = None, mlir_file: str = "",
                    num_samples: int = 0, tune_num: int = 0, histogram_bin_num: int = 2048) -> None:
    """Write the results of ``ShardedCalibrator.run`` as a calibration table in the reference's text format
    (kld_calibrator.py:804-884): tensors in graph order, ``threshold min max`` with seven decimals."""
    from .cali_table import write_cali_table
    names = order if order is not None else list(results.keys())
    rows = [(n, float(results[n].threshold), float(results[n].min), float(results[n].max)) for n in names if n in results]
    write_cali_table(path, rows, mlir_file=mlir_file, method="use_kl", histogram_bin_num=histogram_bin_num,
                     num_samples=num_samples, tune_num=tune_num)
