#!/usr/bin/env python3
"""Benchmark of the quantized-inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N=1): BASELINE config 1, one tpu.Conv2D INT8 layer: x s8 NCHW [32,256,56,56], filter s8
[256,256,3,3], stride 1, pad 1, bias, per-channel QDM requant (multiplier in [2^30,2^31), rshift in [8,20],
half away from zero), fused ReLU, s8 NCHW output.  One step = one pass of that layer over the batch.
With N > 1 (torchrun, one rank per GPU) every rank runs its own batch of the same layer (no data-path
collective; weak scaling) and rank 0 reports the whole-job aggregate.

Printed JSON line: `value` = device-resident TOPS (one CUDA-event pair around R repeats of the K steps of the
device-face call, R chosen so that the region lasts about 0.6 s; inputs rotated through more buffers than L2 holds);
`e2e` = the same metric through the operator face with pinned HOST float buffers, copies included; `roofline` = the
tensor-core kernel alone against the kind::i8 tensor-pipe peak measured in the same run; `cpu_baseline` = the
reference's arithmetic route (fp32 oneDNN convolution + requant loop) on the host cores; `extras` = the other
workloads of the metric: ResNet-50 INT8 inference and calibration with their work sharded over the ranks (every N),
and at N=1 the single-kernel lines (INT8 GEMM, 1x1 conv, A16MatMul decode and prefill, histogram and min/max), each
with its own roofline.  `--impl reference` times only the CPU route, on the full workload, with all host threads.
`--workload X` prints the lines of one extra alone.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CFG = dict(N=32, C=256, H=56, W=56, OC=256, KH=3, KW=3)
WORKLOAD = "tpu.Conv2D int8 NCHW n32 c256 56x56 oc256 k3 s1 p1 relu, per-channel QDM requant (BASELINE config 1)"
OPS_PER_STEP = 2.0 * CFG["N"] * CFG["OC"] * CFG["H"] * CFG["W"] * CFG["C"] * CFG["KH"] * CFG["KW"]
# DRAM traffic of one launch of the convolution kernel, from one ncu capture of this workload: 28.38 MB read (the
# bordered image and the filters, once) + 0.03 MB written while the kernel runs (its 25.7 MB output is still in
# L2 when it ends and is written back afterwards)
CONV_DRAM_BYTES_PER_LAUNCH = 28_233_728 + 11_264
METRIC, UNIT = "int8 conv TOPS", "TOPS"
# identical in both arms
CONFIG = dict(workload=WORKLOAD,
              l2="GPU arm: 6 input/output sets used round-robin (308 MB > L2), no flush kernel; CPU arm: not applicable")
TIMED_REGION_S = 0.6


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(bf16_tflops=float(d["bf16_tflops"]), hbm_gbs=float(d["hbm_gbs"]), source="measured")
    return dict(bf16_tflops=1590.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the benchmark runs.  Samples are time-stamped;
    stop(t0, t1) reports the ones that fall inside the timed region [t0, t1] (wall clock), and falls back to
    every sample taken under load (warm-up included) when the region was shorter than the sampling period."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self, t0=None, t1=None):
        import datetime
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(f[1]), float(f[2]), float(f[3]), [nm for nm, v in zip(names, f[4:8]) if v.lower().startswith("active")]))
            except ValueError:
                continue
        inside = [r for r in rows if t0 is not None and t0 <= r[0] <= t1]
        window = "timed region"
        if len(inside) < 3:
            # shorter than the sampling period: use the samples under load (power well above idle), warm-up included
            pmax = max([r[3] for r in rows], default=0.0)
            inside = [r for r in rows if r[3] >= 0.5 * pmax] or rows
            window = "whole run under load (timed region shorter than the sampling period)"
        sm = [r[1] for r in inside]
        reasons = sorted({x for r in inside for x in r[4]})
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=max([r[2] for r in inside], default=None),
                    reasons=reasons, samples=len(sm), window=window)


def cpu_route(c, n_images, threads):
    """The reference's CPU arithmetic for this layer on the first n_images images; returns (seconds, output)."""
    import oracle
    x = c["x"][:n_images]
    kw = dict(pads=(1, 1, 1, 1), do_relu=True, qmode=oracle.QM_QDM, is_cv18xx=True, mult=c["mult"], rshift=c["rshift"],
              threads=threads)
    oracle.conv2d_int8_fp32_path(x[:1], c["w"], c["bias"], **kw)   # warm the primitive cache
    t0 = time.perf_counter()
    out = oracle.conv2d_int8_fp32_path(x, c["w"], c["bias"], **kw)
    return time.perf_counter() - t0, out


def run_reference(args):
    """--impl reference: the CPU interpreter's arithmetic route, full workload per step, all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from tpu_mlir_b200 import synth
    import oracle
    c = synth.conv2d_int8(seed=1, **CFG)
    threads = os.cpu_count() or 1
    kw = dict(pads=(1, 1, 1, 1), do_relu=True, qmode=oracle.QM_QDM, is_cv18xx=True, mult=c["mult"], rshift=c["rshift"],
              threads=threads)
    for _ in range(max(args.warmup, 1)):
        oracle.conv2d_int8_fp32_path(c["x"], c["w"], c["bias"], **kw)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.conv2d_int8_fp32_path(c["x"], c["w"], c["bias"], **kw)
    dt = (time.perf_counter() - t0) / args.steps
    tops = OPS_PER_STEP / dt / 1e12
    line = dict(impl="reference", metric=METRIC, value=tops, unit=UNIT, n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=dt * 1e3, higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype="f32 (integer-valued, as the reference interpreter computes)", data="synthetic",
                config=CONFIG,
                cpu_baseline=dict(value=tops, unit=UNIT, cores=threads, kind="port",
                                  sample="full batch of 32 images per step; fp32 oneDNN convolution (torch CPU) + requant loop"),
                e2e=dict(value=tops, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))
    return 0


def _time_steps(fn, steps, warmup):
    """Milliseconds per call of fn(i): `steps` calls back to back inside ONE CUDA-event pair on the current stream
    (a pair per call would add several microseconds of launch gaps to kernels this short).  fn(i) rotates through
    enough buffer sets that no call finds its inputs in L2."""
    import torch
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / steps


def _time_steps_graph(fn, steps, warmup):
    """Milliseconds per call of fn(i, stream) with the `steps` calls captured ONCE into a CUDA graph and replayed: for
    kernels of ~10 us the Python/ctypes launch path (not the GPU) would otherwise set the pace."""
    import torch
    side = torch.cuda.Stream()
    sp = C.c_void_p(side.cuda_stream)
    with torch.cuda.stream(side):
        for i in range(warmup):
            fn(i, sp)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for i in range(steps):
            fn(i, sp)
    g.replay()   # one untimed replay: graph upload
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / steps


def tensor_peak(kind, pair, seconds):
    """TOPS (kind 0: kind::i8) or TFLOP/s (kind 1: bf16) of the tensor pipe with operands resident in shared memory,
    from b200q_probe_tensor_peak: launches of ~25 ms each, back to back for about `seconds`."""
    import tpu_mlir_b200._lib as L
    lib = L.lib()
    ms, ops = C.c_double(), C.c_double()
    kblocks = 80000     # ~25 ms per launch at full clocks
    L.check(lib.b200q_probe_tensor_peak(kind, pair, kblocks, 2, C.byref(ms), C.byref(ops), None))
    launches = max(1, int(round(seconds * 1e3 / (ms.value / 2))))
    L.check(lib.b200q_probe_tensor_peak(kind, pair, kblocks, launches, C.byref(ms), C.byref(ops), None))
    return ops.value / (ms.value * 1e-3) / 1e12, ms.value


def tensor_peaks(sustained=True):
    """The probe's figures for kind::i8: burst (about 50 ms after idle) and sustained (2 s back to back, the last
    figure under the power cap), single-CTA and CTA-pair form, and the bf16 figure beside MEASURED_PEAKS' cuBLAS one."""
    out = {}
    out["i8_burst"], _ = tensor_peak(0, 0, 0.05)
    out["i8_pair_burst"], _ = tensor_peak(0, 1, 0.05)
    out["bf16_burst"], _ = tensor_peak(1, 0, 0.05)
    if sustained:
        out["i8_pair_sustained"], ms = tensor_peak(0, 1, 2.0)
        out["sustained_ms"] = ms
    out["unit"] = "TOPS (bf16: TFLOP/s)"
    out["source"] = ("b200q_probe_tensor_peak: tcgen05.mma 128x256 (pair: 256x256) x 32 bytes of K on tiles resident in "
                     "shared memory, every SM, timed with CUDA events")
    return out


def kernel_lines(workload, steps, warmup, a16_m=(1, 2, 4, 8, 16, 32, 128, 2048)):
    """Single-kernel lines, device resident, each against its roofline (N=1 only)."""
    import torch
    import tpu_mlir_b200._lib as L
    from tpu_mlir_b200 import synth
    lib = L.lib()
    peaks = measured_peaks()
    P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    lines = []
    if workload == "gemm":
        M = N = K = 8192
        a = torch.randint(-128, 128, (M, K), dtype=torch.int8, device="cuda")
        b = torch.randint(-128, 128, (N, K), dtype=torch.int8, device="cuda")
        out = torch.empty((M, N), dtype=torch.int8, device="cuda")
        rng = np.random.default_rng(0)
        mult, rshift = synth.qdm_params(rng, N)
        keep = [torch.from_numpy(v.astype(np.int32)).cuda() for v in
                (rng.integers(-2**16, 2**16, N), mult, -rshift)]
        e = L.Epilogue(dialect=L.RQ_QDM, round_mode=L.ROUND_HALF_AWAY_FROM_ZERO, per_channel=1, out_zp=0,
                       relu=L.RELU_NONE, out_dtype=L.DT_I8, scale=0.0, bias=keep[0].data_ptr(),
                       multiplier=keep[1].data_ptr(), shift=keep[2].data_ptr())
        st = torch.zeros(1, dtype=torch.int32, device="cuda")

        def go(i):
            L.check(lib.b200q_gemm_i8_dev(P(a), L.DT_I8, P(b), L.DT_I8, M, N, K, C.byref(e), P(out), P(st),
                                          L.ALGO_TENSOR_CORE, None))
        mean_ms = _time_steps(go, min(steps, 200), warmup)
        assert int(st.item()) == 0
        tops = 2.0 * M * N * K / (mean_ms * 1e-3) / 1e12
        peak, _ = tensor_peak(0, 1, 0.05)
        lines.append(dict(metric="int8 matmul TOPS", value=tops, unit="TOPS", ms_per_step=mean_ms,
                          config=dict(workload="int8 GEMM 8192x8192x8192, per-channel QDM requant, s8 out",
                                      l2="operands + output = 192 MB > L2"),
                          roofline=dict(bound="tensor", achieved=tops, peak=peak, unit="TOPS", frac=tops / peak,
                                        traffic=None, peak_basis="kind::i8 CTA-pair probe of this run (burst)",
                                        frac_of_2x_bf16=tops / (2 * peaks["bf16_tflops"]))))
    elif workload == "conv1x1":
        # the short-K layer of a bottleneck block (ResNet-50 layer1 conv3), channels-last in and out: the product is
        # bound by its output stream, not by the tensor pipe
        from tpu_mlir_b200.ops import Conv2DOp
        N, Cin, H, W, OC = 256, 64, 56, 56, 256
        rng = np.random.default_rng(0)
        op = Conv2DOp(input_shape=(N, Cin, H, W), oc=OC, kernel_shape=(1, 1), pads=(0, 0, 0, 0), do_relu=True,
                      input_dtype=L.DT_U8, out_dtype=L.DT_U8, quant_mode=L.QM_MULTIPLIER_SHIFT,
                      multiplier=rng.integers(5000, 30000, OC), rshift=rng.integers(18, 26, OC))
        d = op.desc     # (the op owns the arrays the descriptor points to)
        x = torch.randint(0, 255, (N, H, W, Cin), dtype=torch.uint8, device="cuda")
        w = torch.randint(-64, 64, (OC, Cin, 1, 1), dtype=torch.int8, device="cuda")
        bias = torch.randint(-4096, 4096, (OC,), dtype=torch.int32, device="cuda")
        y = torch.empty((N, H, W, OC), dtype=torch.uint8, device="cuda")
        h = C.c_void_p()
        L.check(lib.b200q_conv2d_dev_create(C.byref(d), P(w), P(bias), C.byref(h)))
        mean_ms = _time_steps(lambda i: L.check(lib.b200q_conv2d_dev_run_layout(h, P(x), L.LAYOUT_NHWC, P(y), L.LAYOUT_NHWC,
                                                                                 None)), min(steps, 200), warmup)
        L.check(lib.b200q_conv2d_dev_status(h, None))
        lib.b200q_conv2d_dev_destroy(C.byref(h))
        nbytes = x.numel() + y.numel() + w.numel()
        gbs = nbytes / (mean_ms * 1e-3) / 1e9
        lines.append(dict(metric="int8 1x1 conv GB/s", value=gbs, unit="GB/s", ms_per_step=mean_ms,
                          config=dict(workload="tpu.Conv2D int8 channels-last n256 c64 56x56 oc256 k1, per-channel "
                                               "MultiplierShift requant + ReLU, u8 out (transposed product)",
                                      l2="input + output = 257 MB > L2", bytes_per_call=int(nbytes),
                                      tops=2.0 * N * H * W * OC * Cin / (mean_ms * 1e-3) / 1e12),
                          roofline=dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s",
                                        frac=gbs / peaks["hbm_gbs"], traffic=None,
                                        peak_basis=f"{peaks['source']} copy bandwidth")))
    elif workload == "dwconv":
        # a depthwise 3x3 layer of a mobile network (MobileNetV2 block, 384 channels at 28x28), NCHW: the CUDA-core patch kernel
        from tpu_mlir_b200.ops import Conv2DOp
        N, Cc, H, W = 256, 384, 28, 28
        rng = np.random.default_rng(0)
        op = Conv2DOp(input_shape=(N, Cc, H, W), oc=Cc, kernel_shape=(3, 3), pads=(1, 1, 1, 1), group=Cc, do_relu=True,
                      quant_mode=L.QM_MULTIPLIER_SHIFT, multiplier=rng.integers(5000, 30000, Cc), rshift=rng.integers(14, 20, Cc))
        x = torch.randint(-128, 128, (N, Cc, H, W), dtype=torch.int8, device="cuda")
        w = torch.randint(-64, 64, (Cc, 1, 3, 3), dtype=torch.int8, device="cuda")
        bias = torch.randint(-4096, 4096, (Cc,), dtype=torch.int32, device="cuda")
        y = torch.empty((N, Cc, H, W), dtype=torch.int8, device="cuda")
        h = C.c_void_p()
        L.check(lib.b200q_conv2d_dev_create(C.byref(op.desc), P(w), P(bias), C.byref(h)))
        mean_ms = _time_steps(lambda i: L.check(lib.b200q_conv2d_dev_run(h, P(x), P(y), None)), min(steps, 100), warmup)
        L.check(lib.b200q_conv2d_dev_status(h, None))
        lib.b200q_conv2d_dev_destroy(C.byref(h))
        nbytes = x.numel() + y.numel() + w.numel()
        gbs = nbytes / (mean_ms * 1e-3) / 1e9
        lines.append(dict(metric="int8 depthwise conv GB/s", value=gbs, unit="GB/s", ms_per_step=mean_ms,
                          config=dict(workload="tpu.Conv2D int8 depthwise NCHW n256 c384 28x28 k3 s1 p1, per-channel MultiplierShift "
                                               "requant + ReLU (CUDA-core patch kernel)",
                                      l2="input + output = 154 MB > L2", bytes_per_call=int(nbytes)),
                          roofline=dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s",
                                        frac=gbs / peaks["hbm_gbs"], traffic=None,
                                        peak_basis=f"{peaks['source']} copy bandwidth")))
    elif workload == "a16":
        # one MLP layer of a 7B decoder through the handle API (tensors stay the caller's); every M reads the packed
        # weights (24.7 MB) from 8 weight sets used round-robin so that no call finds them in L2
        NS = 8
        c0 = synth.a16_w4(seed=2, M=1)
        sets = [tuple(torch.from_numpy(c0[k]).cuda() for k in ("wq", "scale", "zp")) for _ in range(NS)]
        wq, sc, zp = sets[0]
        hs = []
        for w_, s_, z_ in sets:
            h = C.c_void_p()
            L.check(lib.b200q_a16_dev_create(P(w_), P(s_), P(z_), None, 11008, 4096, 64, C.byref(h)))
            hs.append(h)
        packed = wq.numel() + sc.numel() * 2 + zp.numel()
        for M in a16_m:
            x = torch.from_numpy(synth.a16_w4(seed=2, M=M)["x"]).cuda()
            y = torch.empty((M, 11008), dtype=torch.uint16, device="cuda")

            def go(i, stream, x=x, y=y, M=M):
                L.check(lib.b200q_a16_dev_run(hs[i % NS], P(x), P(y), M, stream))
            for h in hs:        # the first call of a handle at a new M may allocate: not inside a graph capture
                L.check(lib.b200q_a16_dev_run(h, P(x), P(y), M, None))
            torch.cuda.synchronize()
            calls = 200 if M <= 128 else 48
            mean_ms = _time_steps_graph(go, calls, warmup)
            for h in hs:
                L.check(lib.b200q_a16_dev_status(h, None))
            nbytes = packed + x.numel() * 2 + y.numel() * 2
            gbs = nbytes / (mean_ms * 1e-3) / 1e9
            tf = 2.0 * M * 11008 * 4096 / (mean_ms * 1e-3) / 1e12
            hbm = dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s", frac=gbs / peaks["hbm_gbs"],
                       traffic=None, peak_basis=f"{peaks['source']} copy bandwidth")
            tensor = dict(bound="tensor", achieved=tf, peak=peaks["bf16_tflops"], unit="TFLOP/s",
                          frac=tf / peaks["bf16_tflops"], traffic=None, peak_basis=f"{peaks['source']} dense bf16 (burst)")
            # the two bounds cross where 2*M*N*K / bf16 peak = packed bytes / HBM peak: M ~ 33 for this layer
            bound_is_hbm = nbytes / (peaks["hbm_gbs"] * 1e9) >= 2.0 * M * 11008 * 4096 / (peaks["bf16_tflops"] * 1e12)
            route = ("decode kernel (one token: CUDA cores, weights straight from global memory)" if M == 1 else
                     "decode kernel, resident form (the block's weight slice in shared memory, mma.sync)" if M <= 8 else
                     "two launches of the resident decode kernel (8 tokens each)" if M <= 16 else
                     "bf16 copy of the weight kept in the handle (90 MB) + bf16 tensor-core GEMM" if M >= 64 else
                     "fused kernel: packed weights by TMA, dequantised in registers into tensor memory, tcgen05 kind::f16")
            lines.append(dict(metric="A16MatMul w4bf16 " + ("GB/s" if bound_is_hbm else "TFLOP/s"),
                              value=gbs if bound_is_hbm else tf, unit="GB/s" if bound_is_hbm else "TFLOP/s",
                              ms_per_step=mean_ms,
                              config=dict(workload=f"A16MatMul w4bf16 N=11008 K=4096 group 64, M={M}", route=route,
                                          l2="8 weight sets used round-robin (198 MB packed > L2)",
                                          bytes_per_call=int(nbytes), gbs=gbs, tflops=tf,
                                          timing=f"{calls} calls captured in one CUDA graph, replayed inside one event pair"),
                              roofline=hbm if bound_is_hbm else tensor))
        for h in hs:
            lib.b200q_a16_dev_destroy(C.byref(h))
    elif workload == "hist":
        from tpu_mlir_b200.calibration import CaliMathB200
        m = CaliMathB200()
        S, n = 64, 64 * 112 * 112
        x = torch.randn((S, n), dtype=torch.float32, device="cuda")
        mm = m.minmax(x, samples=S).cpu().numpy()
        th = np.maximum(np.abs(mm[:, 0]), np.abs(mm[:, 1])).astype(np.float32)
        th[:] = th.max()
        nb = np.full(S, 2048, np.int32)
        hist = torch.zeros(2048, dtype=torch.int32, device="cuda")
        mean_h = _time_steps(lambda i: m.histogram_into(hist, x, th, nb), min(steps, 200), warmup)
        mean_m = _time_steps(lambda i: m.minmax(x, samples=S), min(steps, 200), warmup)
        for name, ms in (("calibration histogram GB/s", mean_h), ("calibration min/max GB/s", mean_m)):
            gbs = x.numel() * 4 / (ms * 1e-3) / 1e9
            lines.append(dict(metric=name, value=gbs, unit="GB/s", ms_per_step=ms,
                              config=dict(workload="64 samples x 64x112x112 float32 (largest ResNet-50 activation), "
                                                   "2048 bins", l2="input 205 MB > L2"),
                              roofline=dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s",
                                            frac=gbs / peaks["hbm_gbs"], traffic=None,
                                            peak_basis=f"{peaks['source']} copy bandwidth (read-only kernel)")))
    elif workload == "top":
        # fp32 Top-dialect forward (calibration's float graph): one 3x3 convolution and the whole ResNet-50 forward.
        # The bound is the CUDA cores' fp32 FMA rate: SMs x 128 lanes x 2 flop x the SM clock sampled during the run.
        from tpu_mlir_b200 import resnet50
        n, ic, hw, oc = 64, 128, 28, 128
        x = torch.randn(n, ic, hw, hw, device="cuda")
        w = torch.randn(oc, ic, 3, 3, device="cuda")
        b = torch.randn(oc, device="cuda")
        d = L.TopConvDesc(n=n, ic=ic, ih=hw, iw=hw, oc=oc, kh=3, kw=3, sh=1, sw=1, dh=1, dw=1, pht=1, phb=1, pwl=1, pwr=1,
                          groups=1, with_bias=1, do_relu=1, relu_limit=-1.0)
        h = C.c_void_p()
        L.check(lib.b200q_top_conv2d_dev_create(C.byref(d), P(w), P(b), C.byref(h)))
        y = torch.empty(n, oc, hw, hw, device="cuda")
        sampler = ClockSampler(torch.cuda.current_device())
        sampler.start()
        mean_c = _time_steps(lambda i: L.check(lib.b200q_top_conv2d_dev_run(h, P(x), P(y), n, None)), min(steps, 200), warmup)
        lib.b200q_top_conv2d_dev_destroy(C.byref(h))
        ops = resnet50.build_fp32()
        fwd = resnet50.Fp32Forward(ops, torch.device("cuda"))
        xb = torch.randn(64, 3, 224, 224, device="cuda")
        mean_f = _time_steps(lambda i: fwd(xb), 10, 3)
        clocks = sampler.stop()
        sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        mhz = float(clocks.get("sm_mhz") or clocks.get("sm_max_mhz") or 1965.0)
        peak = sms * 128 * 2 * mhz * 1e6 / 1e12
        tf_c = 2.0 * n * oc * hw * hw * ic * 9 / (mean_c * 1e-3) / 1e12
        flop_img = sum(2.0 * np.prod(fwd.shape[o["name"]]) * np.prod(o["w"].shape[1:]) for o in ops if o["type"] == "conv")
        tf_f = 64 * flop_img / (mean_f * 1e-3) / 1e12
        basis = f"{sms} SMs x 128 fp32 lanes x 2 flop x {mhz:.0f} MHz (median SM clock sampled during the run)"
        lines.append(dict(metric="fp32 conv TFLOP/s", value=tf_c, unit="TFLOP/s", ms_per_step=mean_c, dtype="f32", clocks=clocks,
                          config=dict(workload="top.Conv fp32 NCHW n64 c128 28x28 oc128 k3 s1 p1 relu (ResNet-50 layer2)",
                                      l2="input 25.7 MB + output 25.7 MB, L2-resident: the kernel is FMA-bound"),
                          roofline=dict(bound="fp32 fma", achieved=tf_c, peak=peak, unit="TFLOP/s", frac=tf_c / peak, traffic=None,
                                        peak_basis=basis)))
        lines.append(dict(metric="ResNet-50 fp32 forward img/s", value=64 / (mean_f * 1e-3), unit="img/s", ms_per_step=mean_f,
                          steps=10, dtype="f32",
                          config=dict(workload="ResNet-50 fp32 Top-dialect forward, batch 64, every activation kept (the calibration "
                                               "forward): 53 convolutions, pooling, adds, fc on this library's kernels"),
                          roofline=dict(bound="fp32 fma", achieved=tf_f, peak=peak, unit="TFLOP/s", frac=tf_f / peak, traffic=None,
                                        peak_basis=basis)))
    elif workload == "peak":
        lines.append(dict(metric="tensor-pipe peak", **tensor_peaks()))
    else:
        raise ValueError(workload)
    return lines


class Ranks:
    """The process layout the launcher gave this run: one rank per GPU over NCCL, or a single process."""

    def __init__(self):
        import torch
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist

    def barrier(self):
        import torch
        if self.dist:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, values):
        import torch
        t = torch.tensor(list(values), dtype=torch.float64, device=self.dev)
        if self.dist:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t]

    def min_over_ranks(self, value):
        import torch
        t = torch.tensor([value], dtype=torch.float64, device=self.dev)
        if self.dist:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return float(t[0])

    def close(self):
        if self.dist:
            self.dist.destroy_process_group()


def resnet50_line(R, steps, warmup, check=True):
    """BASELINE config 3: INT8 ResNet-50 inference, global batch 256 sharded 256/N per rank (no data-path collective).
    Device-resident and host-buffer img/s; the int8 logits of the first two images of every rank's shard are compared
    bit for bit with the CPU oracle's walk of the same graph, and the SHA-256 of all 256x1000 logits (rank order) is
    reported: it does not depend on N."""
    import hashlib
    import torch
    from tpu_mlir_b200 import resnet50, synth
    from tpu_mlir_b200.module import module
    GLOBAL_BATCH = int(os.environ.get("B200Q_RESNET_BATCH", "256"))     # BASELINE config 3: 256
    per = GLOBAL_BATCH // R.world
    ops = resnet50.build_fp32(seed=3)
    cal_images = torch.from_numpy(synth.calibration_images(seed=4, count=64)).to(R.dev)
    table = resnet50.self_calibration_table(ops, cal_images, batch=16)          # every rank derives the same table
    del cal_images
    graph, weights = resnet50.lower_int8(ops, table, batch=per)
    m = module(channels_last=os.environ.get("B200Q_RESNET_LAYOUT", "nhwc") == "nhwc",
               cuda_graph=os.environ.get("B200Q_RESNET_GRAPH", "1") == "1",
               fuse_residual_add=os.environ.get("B200Q_RESNET_FUSE_ADD", "0") == "1")
    m.load(graph, weights)
    n_fused = len(m._fused_adds)
    x_h = torch.from_numpy(synth.calibration_images(seed=5, count=per, start=R.rank * per)).pin_memory()
    m.set_tensor("input", x_h)
    for _ in range(warmup):
        m.invoke(fixed_to_float=False)
    R.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        m.invoke(fixed_to_float=False)
    e1.record()
    e1.synchronize()
    total_ms = e0.elapsed_time(e1)
    R.barrier()
    # end to end: pinned host images in, int8 logits out, every step
    e2e_steps = max(3, steps // 4)
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        m.set_tensor("input", x_h)
        m.invoke(fixed_to_float=False)
        logits = m.tensors["fc"].cpu()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    total_ms, e2e_s = R.max_over_ranks([total_ms, e2e_s])
    # parity and digest (outside the timed regions)
    mine = m.tensors["fc"].reshape(per, -1).contiguous()
    if R.dist:
        parts = [torch.empty_like(mine) for _ in range(R.world)]
        R.dist.all_gather(parts, mine)
        all_logits = torch.cat(parts, dim=0)
    else:
        all_logits = mine
    digest = hashlib.sha256(all_logits.cpu().numpy().tobytes()).hexdigest()
    parity = "not checked"
    if check:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import oracle_graph
        torch.set_num_threads(max(1, (os.cpu_count() or 1) // R.world))
        g2, w2 = resnet50.lower_int8(ops, table, batch=min(2, per))
        want = oracle_graph.run(g2, w2, {"input": x_h[:min(2, per)].numpy()})["fc"]
        ok = bool(np.array_equal(want.reshape(min(2, per), -1), mine[:min(2, per)].cpu().numpy()))
        ok_all = R.min_over_ranks(1.0 if ok else 0.0) == 1.0
        parity = (f"int8 logits of the first {min(2, per)} images of each of the {R.world} shards equal the CPU oracle's bit for bit"
                  if ok_all else "MISMATCH against the CPU oracle")
    del m
    torch.cuda.empty_cache()
    if R.rank != 0:
        return None
    return dict(metric="ResNet-50 int8 img/s", value=GLOBAL_BATCH * steps / (total_ms * 1e-3), unit="img/s",
                ms_per_step=total_ms / steps, steps=steps, warmup=warmup, scaling="strong", n_gpus=R.world,
                config=dict(workload=f"ResNet-50 INT8 symmetric (random init, calibrated on 64 synthetic images), "
                                     f"global batch {GLOBAL_BATCH} of 3x224x224, batch sharded over the ranks",
                            per_gpu_batch=per, ops_in_graph=len(graph["ops"]), residual_adds_fused=n_fused,
                            kernels_per_step=len(graph["ops"]) - n_fused),
                parity=parity, logits_sha256=digest,
                e2e=dict(value=GLOBAL_BATCH * e2e_steps / e2e_s, unit="img/s", steps=e2e_steps,
                         h2d_bytes_per_step=int(x_h.numel() * 4), d2h_bytes_per_step=int(logits.numel())))


def calibration_line(R, total=None):
    """BASELINE config 4: calibration of ResNet-50 on 2048 synthetic samples sharded 2048/N per rank: fp32 forward
    (torch), per-sample min/max, all-gather, streaming histograms, one all-reduce of the int32 counts, KLD."""
    import hashlib
    import torch
    from tpu_mlir_b200 import resnet50, synth
    from tpu_mlir_b200.calibration import ShardedCalibrator
    TOTAL = total or int(os.environ.get("B200Q_CALIB_SAMPLES", "2048"))
    per = TOTAL // R.world
    ops = resnet50.build_fp32(seed=3)
    images = torch.from_numpy(synth.calibration_images(seed=4, count=per, start=R.rank * per)).to(R.dev)
    fwd = resnet50.Fp32Forward(ops, R.dev)
    cal = ShardedCalibrator(fwd, dist=R.dist)
    CB = int(os.environ.get("B200Q_CALIB_BATCH", "64"))      # samples per forward call (the same at every N)
    batches = [images[i:i + CB] for i in range(0, per, CB)]
    if per >= 2 * CB:
        cal.run(batches[:2], samples_per_rank=2 * CB)      # warm-up: NCCL channels, allocator
    R.barrier()
    t0 = time.perf_counter()
    res = cal.run(batches, samples_per_rank=per)
    R.barrier()
    dt = time.perf_counter() - t0
    (dt,) = R.max_over_ranks([dt])
    phases = R.max_over_ranks([cal.timings[k] for k in sorted(cal.timings)])
    if R.rank != 0:
        return None
    digest = hashlib.sha256("".join(f"{n} {r.threshold:.7f} {r.min:.7f} {r.max:.7f}\n" for n, r in res.items()).encode()).hexdigest()
    return dict(metric="calibration samples/s", value=TOTAL / dt, unit="samples/s", ms_per_step=dt * 1e3, steps=1,
                scaling="strong", n_gpus=R.world, table_sha256=digest,
                config=dict(workload=f"ResNet-50 fp32 forward (own full-fp32 Top-dialect kernels) + min/max, streaming histogram (2048 bins) and KLD on "
                                     f"{len(res)} tensors, {TOTAL} synthetic samples sharded over the ranks",
                            tensors=len(res), samples_per_rank=per, forward_batch=CB,
                            allreduce_bytes=cal.allreduce_bytes, allgather_bytes=int(len(res) * per * 8 * R.world) if R.dist else 0,
                            activations_kept_on_device_bytes=cal.cached_bytes,
                            phase_seconds_max_over_ranks=dict(zip(sorted(cal.timings), phases))))


def guarded(fn, *a, **k):
    """An extra never takes the headline down with it."""
    try:
        return fn(*a, **k)
    except Exception as e:      # noqa: BLE001
        return dict(error=f"{type(e).__name__}: {e}"[:400])


def headline(args, R):
    import torch
    import tpu_mlir_b200._lib as L
    from tpu_mlir_b200 import synth
    from tpu_mlir_b200.ops import Conv2DOp, InferenceParameter
    world, rank = R.world, R.rank
    lib = L.lib()

    c = synth.conv2d_int8(seed=1 + rank, **CFG) if rank else synth.conv2d_int8(seed=1, **CFG)
    op = Conv2DOp(input_shape=c["x"].shape, oc=CFG["OC"], kernel_shape=(3, 3), pads=(1, 1, 1, 1), do_relu=True,
                  quant_mode=L.QM_QDM, is_cv18xx=True, multiplier=c["mult"], rshift=c["rshift"],
                  algo=L.ALGO_TENSOR_CORE)
    stream = torch.cuda.Stream()
    sptr = C.c_void_p(stream.cuda_stream)
    w_d = torch.from_numpy(c["w"]).cuda()
    b_d = torch.from_numpy(c["bias"]).cuda()
    # NSETS input/output pairs used round-robin: a step's tensors were last touched NSETS steps (> 300 MB of
    # traffic, L2 is 126 MB) earlier, so every step reads its input from HBM without a flush kernel in between
    NSETS = 6
    x_sets = [torch.from_numpy(c["x"]).cuda() for _ in range(NSETS)]
    y_sets = [torch.empty(op.out_shape, dtype=torch.int8, device="cuda") for _ in range(NSETS)]
    h = C.c_void_p()
    L.check(lib.b200q_conv2d_dev_create(C.byref(op.desc), C.c_void_p(w_d.data_ptr()), C.c_void_p(b_d.data_ptr()),
                                        C.byref(h)))
    xp = [C.c_void_p(t.data_ptr()) for t in x_sets]
    yp = [C.c_void_p(t.data_ptr()) for t in y_sets]
    run = lib.b200q_conv2d_dev_run

    def step_device(i):
        rc = run(h, xp[i % NSETS], yp[i % NSETS], sptr)
        if rc:
            L.check(rc)

    K = args.steps
    sampler = ClockSampler(R.local_rank)
    if rank == 0:
        sampler.start()
    with torch.cuda.stream(stream):
        for i in range(args.warmup):
            step_device(i)
        L.check(lib.b200q_conv2d_dev_status(h, sptr))
        # how many repeats of the K steps make the timed region last TIMED_REGION_S: from 50 steps timed on the side
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record(stream)
        for i in range(50):
            step_device(i)
        p1.record(stream)
        p1.synchronize()
        est_ms = p0.elapsed_time(p1) / 50
        (est_ms,) = R.max_over_ranks([est_ms])
        repeats = max(1, int(np.ceil(TIMED_REGION_S * 1e3 / (K * est_ms))))
        R.barrier()
        t_wall0 = time.time()
        # pass 1, the timed region: the K steps, `repeats` times, as a user runs them (no events between the kernels,
        # so the convolution kernel launches as a programmatic dependent of its layout kernel)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(K * repeats):
            step_device(i)
        e1.record(stream)
        e1.synchronize()
        t_wall1 = time.time()
        L.check(lib.b200q_conv2d_dev_status(h, sptr))
        R.barrier()
        total_ms = e0.elapsed_time(e1)
        # pass 2, the same steps with the library recording events around each kernel: the per-kernel durations
        # behind `roofline` (the events serialise the two kernels, so their sum is a little above a step of pass 1)
        prof_steps = K * min(repeats, 25)
        L.check(lib.b200q_conv2d_dev_set_profiling(h, 1))
        for i in range(prof_steps):
            step_device(i)
        stream.synchronize()
        L.check(lib.b200q_conv2d_dev_status(h, sptr))
        R.barrier()
        clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
        runs, lay, ker = C.c_int64(), C.c_double(), C.c_double()
        L.check(lib.b200q_conv2d_dev_profile(h, C.byref(runs), C.byref(lay), C.byref(ker)))
        layout_ms, k_ms = lay.value / runs.value, ker.value / runs.value
        L.check(lib.b200q_conv2d_dev_set_profiling(h, 0))
    timed_steps = K * repeats
    gpu_launches = 2 * timed_steps

    # ---- end to end through the operator face: pinned host float buffers, copies inside the timed region
    e2e = None
    if not args.skip_e2e:
        x_h = torch.from_numpy(c["x"]).to(torch.float32).pin_memory()
        w_h = torch.from_numpy(c["w"]).to(torch.float32)
        bias_h = torch.from_numpy(c["bias"]).to(torch.float32)
        y_h = torch.empty(op.out_shape, dtype=torch.float32).pin_memory()
        p = InferenceParameter(inputs=[x_h.numpy(), w_h.numpy(), bias_h.numpy()], outputs=[y_h.numpy()])
        op.init(p)
        for _ in range(3):
            op.inference(p)
        e2e_steps = max(K, 100)
        R.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            op.inference(p)          # synchronous: H2D, layout, conv, D2H
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        op.deinit(p)
        same = bool(np.array_equal(y_h.numpy(), y_sets[0].cpu().numpy().astype(np.float32)))
        if not same:
            raise SystemExit("operator face and device face disagree")
        e2e = dict(s=e2e_s, steps=e2e_steps, h2d=int(x_h.numel() * 4), d2h=int(y_h.numel() * 4))
        gpu_launches += 3 * 8 * e2e_steps  # per piece of the batch (8 pieces): f32->bordered layout, conv, int8->f32
        del x_h, y_h

    total_ms, e2e_s = R.max_over_ranks([total_ms, e2e["s"] if e2e else 0.0])
    line = None
    if rank == 0:
        peaks = measured_peaks()
        probe = guarded(tensor_peaks)
        two_bf16 = 2.0 * peaks["bf16_tflops"]
        int8_peak = probe.get("i8_pair_burst") or two_bf16
        value = world * OPS_PER_STEP * timed_steps / (total_ms * 1e-3) / 1e12
        achieved = OPS_PER_STEP / (k_ms * 1e-3) / 1e12
        line = dict(metric=METRIC, value=value, unit=UNIT, n_gpus=world, steps=K, warmup=args.warmup,
                    ms_per_step=total_ms / timed_steps, higher_is_better=True, scaling="weak", vs_baseline=None,
                    dtype="s8 x s8 -> s32 accumulate -> s8", data="synthetic", config=CONFIG,
                    timing=dict(repeats=repeats, timed_steps=timed_steps, timed_region_ms=total_ms,
                                note="the K steps run `repeats` times inside ONE CUDA-event pair so that the region is long "
                                     "enough for the clock sampler; ms_per_step = region / (K x repeats)",
                                per_step_kernels=dict(layout_ms=layout_ms, conv_ms=k_ms, steps=prof_steps,
                                                      source="a second pass of the same steps with CUDA events "
                                                             "recorded around each kernel")),
                    roofline=dict(bound="tensor", achieved=achieved, peak=int8_peak, unit="TOPS",
                                  frac=achieved / int8_peak, traffic=CONV_DRAM_BYTES_PER_LAUNCH,
                                  traffic_source="ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of "
                                                 "this workload's convolution kernel",
                                  peak_basis="kind::i8 tensor-pipe probe of this run, CTA pairs, burst "
                                             "(tcgen05.mma on tiles resident in shared memory)" if "i8_pair_burst" in probe
                                             else f"2 x {peaks['source']} dense bf16 (probe failed: {probe.get('error')})",
                                  peak_2x_bf16=two_bf16, frac_of_2x_bf16=achieved / two_bf16,
                                  frac_of_sustained=achieved / probe["i8_pair_sustained"] if "i8_pair_sustained" in probe else None,
                                  probe=probe),
                    clocks=clocks, gpu_launches=gpu_launches)
        if e2e:
            line["e2e"] = dict(value=world * OPS_PER_STEP * e2e["steps"] / e2e_s / 1e12, unit=UNIT,
                               h2d_bytes_per_step=e2e["h2d"], d2h_bytes_per_step=e2e["d2h"],
                               ms_per_step=e2e_s / e2e["steps"] * 1e3, steps=e2e["steps"],
                               api="b200q_conv2d_inference (host float32 buffers, pinned)")
        if not args.skip_cpu:
            n_img = 8
            threads = os.cpu_count() or 1
            secs, out = cpu_route(c, n_img, threads)
            if not np.array_equal(out, y_sets[0][:n_img].cpu().numpy()):
                raise SystemExit("GPU result differs from the CPU route on the sampled images")
            line["cpu_baseline"] = dict(value=OPS_PER_STEP * n_img / CFG["N"] / secs / 1e12, unit=UNIT, cores=threads,
                                        kind="port", sample=f"first {n_img} of 32 images, fp32 oneDNN conv + requant "
                                                            f"loop, {secs:.3f} s")
    lib.b200q_conv2d_dev_destroy(C.byref(h))
    del x_sets, y_sets
    torch.cuda.empty_cache()
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="conv",
                    choices=["conv", "gemm", "conv1x1", "dwconv", "a16", "hist", "top", "peak", "resnet50", "calib"],
                    help="conv = the benchmark contract (BASELINE config 1) with every other workload under `extras`; "
                         "any other value prints that workload's lines alone")
    ap.add_argument("--no-extras", action="store_true", help="headline only")
    ap.add_argument("--a16-m", default="1,2,4,8,16,32,128,2048", help="token counts of --workload a16 (profiling runs pick one)")
    ap.add_argument("--skip-cpu", action="store_true", help="skip the CPU legs (profiling runs)")
    ap.add_argument("--skip-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference(args)
    R = Ranks()
    common = dict(higher_is_better=True, data="synthetic")

    def emit(ln):
        if R.rank == 0 and ln:
            ln.update({k: v for k, v in common.items() if k not in ln})
            print(json.dumps(ln), flush=True)

    if args.workload == "resnet50":
        emit(resnet50_line(R, max(args.steps, 20), args.warmup, check=not args.skip_cpu))
    elif args.workload == "calib":
        emit(calibration_line(R))
    elif args.workload != "conv":
        if R.world != 1:
            raise SystemExit("the single-kernel workloads run on one GPU")
        for ln in kernel_lines(args.workload, args.steps, args.warmup, tuple(int(v) for v in args.a16_m.split(","))):
            ln.update(n_gpus=1, steps=ln.get("steps", args.steps), warmup=args.warmup)
            emit(ln)
    else:
        line = headline(args, R)
        if not args.no_extras:
            extras = {}
            t0 = time.time()
            r = guarded(resnet50_line, R, 100, 5, not args.skip_cpu)
            c = guarded(calibration_line, R)
            if R.rank == 0:
                extras["resnet50"], extras["calibration"] = r, c
                if R.world == 1:
                    for wl in ("gemm", "conv1x1", "dwconv", "a16", "hist", "top"):
                        extras[wl] = guarded(kernel_lines, wl, 100, 5)
                extras["seconds"] = time.time() - t0
                line["extras"] = extras
        emit(line)
    R.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
