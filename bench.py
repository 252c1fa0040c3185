#!/usr/bin/env python3
"""Benchmark of the quantized-inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N=1): BASELINE config 1, one tpu.Conv2D INT8 layer: x s8 NCHW [32,256,56,56], filter s8
[256,256,3,3], stride 1, pad 1, bias, per-channel QDM requant (multiplier in [2^30,2^31), rshift in [8,20],
half away from zero), fused ReLU, s8 NCHW output.  One step = one pass of that layer over the batch.
With N > 1 (torchrun, one rank per GPU) every rank runs its own batch of the same layer (no data-path
collective; weak scaling) and rank 0 reports the whole-job aggregate.

Printed JSON line: `value` = device-resident TOPS (one CUDA-event pair around all K steps of the device-face
call, inputs rotated through more buffers than L2 holds); `e2e` = the same metric through the operator face with pinned HOST float buffers, copies
included; `roofline` = the tensor-core kernel alone against the dense INT8 peak; `cpu_baseline` = the
reference's arithmetic route (fp32 oneDNN convolution + requant loop) on the host cores.
`--impl reference` times only that CPU route, on the full workload, with all host threads.
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
                config=dict(workload=WORKLOAD, route="fp32 oneDNN convolution (torch CPU) + requant loop"),
                cpu_baseline=dict(value=tops, unit=UNIT, cores=threads, kind="port",
                                  sample="full batch of 32 images per step"),
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


def run_kernel_workload(args):
    """Secondary lines (not the benchmark contract): one kernel each, device resident, against its roofline."""
    import torch
    import tpu_mlir_b200._lib as L
    from tpu_mlir_b200 import synth
    lib = L.lib()
    torch.cuda.set_device(0)
    peaks = measured_peaks()
    P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    lines = []
    if args.workload == "gemm":
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
        mean_ms = _time_steps(go, args.steps, args.warmup)
        assert int(st.item()) == 0
        tops = 2.0 * M * N * K / (mean_ms * 1e-3) / 1e12
        peak = 2 * peaks["bf16_tflops"]
        lines.append(dict(metric="int8 matmul TOPS", value=tops, unit="TOPS", ms_per_step=mean_ms,
                          config=dict(workload="int8 GEMM 8192x8192x8192, per-channel QDM requant, s8 out",
                                      l2="operands + output = 192 MB > L2"),
                          roofline=dict(bound="tensor", achieved=tops, peak=peak, unit="TOPS", frac=tops / peak,
                                        traffic=None, peak_basis=f"2 x {peaks['source']} dense bf16")))
    elif args.workload == "conv1x1":
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
                                                                                 None)), args.steps, args.warmup)
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
    elif args.workload == "a16":
        for M in (1, 2, 4, 8):
            c = synth.a16_w4(seed=2, M=M)
            NS = 8   # 8 copies of the weight set (198 MB > L2) used round-robin, one handle each (decode keeps them resident)
            x = torch.from_numpy(c["x"]).cuda()
            sets = [tuple(torch.from_numpy(c[k]).cuda() for k in ("wq", "scale", "zp")) for _ in range(NS)]
            wq, sc, zp = sets[0]
            y = torch.empty((M, 11008), dtype=torch.uint16, device="cuda")
            hs = []
            for w_, s_, z_ in sets:
                h = C.c_void_p()
                L.check(lib.b200q_a16_dev_create(P(w_), P(s_), P(z_), None, 11008, 4096, 64, C.byref(h)))
                hs.append(h)

            def go(i, stream):
                L.check(lib.b200q_a16_dev_run(hs[i % NS], P(x), P(y), M, stream))
            mean_ms = _time_steps_graph(go, min(args.steps, 200), args.warmup)
            for h in hs:
                L.check(lib.b200q_a16_dev_status(h, None))
                lib.b200q_a16_dev_destroy(C.byref(h))
            nbytes = wq.numel() + sc.numel() * 2 + zp.numel() + x.numel() * 2 + y.numel() * 2
            gbs = nbytes / (mean_ms * 1e-3) / 1e9
            lines.append(dict(metric="w4bf16 GEMV GB/s", value=gbs, unit="GB/s", ms_per_step=mean_ms,
                              config=dict(workload=f"A16MatMul w4bf16 N=11008 K=4096 group 64, M={M}",
                                          l2="8 weight sets used round-robin (198 MB > L2)", bytes_per_call=int(nbytes),
                                          timing="200 calls captured in one CUDA graph, replayed inside one event pair"),
                              roofline=dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s",
                                            frac=gbs / peaks["hbm_gbs"], traffic=None,
                                            peak_basis=f"{peaks['source']} copy bandwidth")))
        # prefill shapes of the same layer through the handle API: the weight is dequantised to bf16 once (when the
        # handle first sees M > 8), every call is one bf16 tensor-core GEMM
        for M in (16, 128, 2048):
            c = synth.a16_w4(seed=2, M=M)
            x, wq, sc, zp = (torch.from_numpy(c[k]).cuda() for k in ("x", "wq", "scale", "zp"))
            y = torch.empty((M, 11008), dtype=torch.uint16, device="cuda")
            h = C.c_void_p()
            L.check(lib.b200q_a16_dev_create(P(wq), P(sc), P(zp), None, 11008, 4096, 64, C.byref(h)))

            def go(i, stream, h=h, x=x, y=y, M=M):
                L.check(lib.b200q_a16_dev_run(h, P(x), P(y), M, stream))
            mean_ms = _time_steps_graph(go, min(args.steps, 100), args.warmup)
            L.check(lib.b200q_a16_dev_status(h, None))
            lib.b200q_a16_dev_destroy(C.byref(h))
            tf = 2.0 * M * 11008 * 4096 / (mean_ms * 1e-3) / 1e12
            lines.append(dict(metric="w4bf16 prefill TFLOP/s", value=tf, unit="TFLOP/s", ms_per_step=mean_ms,
                              config=dict(workload=f"A16MatMul w4bf16 N=11008 K=4096 group 64, M={M} (bf16 weight resident, 90 MB)",
                                          l2="the 90 MB weight is re-read from L2/HBM by every call",
                                          timing="100 calls captured in one CUDA graph, replayed inside one event pair"),
                              roofline=dict(bound="tensor", achieved=tf, peak=peaks["bf16_tflops"], unit="TFLOP/s",
                                            frac=tf / peaks["bf16_tflops"], traffic=None,
                                            peak_basis=f"{peaks['source']} dense bf16")))
    else:
        from tpu_mlir_b200.calibration import CaliMathB200
        m = CaliMathB200()
        S, n = 64, 64 * 112 * 112
        x = torch.randn((S, n), dtype=torch.float32, device="cuda")
        mm = m.minmax(x, samples=S).cpu().numpy()
        th = np.maximum(np.abs(mm[:, 0]), np.abs(mm[:, 1])).astype(np.float32)
        th[:] = th.max()
        nb = np.full(S, 2048, np.int32)
        hist = torch.zeros(2048, dtype=torch.int32, device="cuda")
        mean_h = _time_steps(lambda i: m.histogram_into(hist, x, th, nb), args.steps, args.warmup)
        mean_m = _time_steps(lambda i: m.minmax(x, samples=S), args.steps, args.warmup)
        for name, ms in (("calibration histogram GB/s", mean_h), ("calibration min/max GB/s", mean_m)):
            gbs = x.numel() * 4 / (ms * 1e-3) / 1e9
            lines.append(dict(metric=name, value=gbs, unit="GB/s", ms_per_step=ms,
                              config=dict(workload="64 samples x 64x112x112 float32 (largest ResNet-50 activation), "
                                                   "2048 bins", l2="input 205 MB > L2"),
                              roofline=dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s",
                                            frac=gbs / peaks["hbm_gbs"], traffic=None,
                                            peak_basis=f"{peaks['source']} copy bandwidth (read-only kernel)")))
    for ln in lines:
        ln.update(n_gpus=1, steps=args.steps, warmup=args.warmup, higher_is_better=True, data="synthetic")
        print(json.dumps(ln))
    return 0


def run_network_workload(args):
    """Whole-network lines (BASELINE configs 3 and 4): INT8 ResNet-50 inference img/s with the batch sharded over
    the ranks, and calibration samples/s with the samples sharded and one NCCL all-reduce of the histograms."""
    import torch
    import torch.distributed as dist
    from tpu_mlir_b200 import resnet50, synth
    from tpu_mlir_b200.module import module
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    ops = resnet50.build_fp32(seed=3)
    line = None
    if args.workload == "resnet50":
        GLOBAL_BATCH = 256
        per = GLOBAL_BATCH // world
        cal_images = torch.from_numpy(synth.calibration_images(seed=4, count=64)).to(dev)
        table = resnet50.self_calibration_table(ops, cal_images, batch=16)          # every rank derives the same table
        graph, weights = resnet50.lower_int8(ops, table, batch=per)
        m = module(channels_last=os.environ.get("B200Q_RESNET_LAYOUT", "nhwc") == "nhwc",
                   cuda_graph=os.environ.get("B200Q_RESNET_GRAPH", "1") == "1")
        m.load(graph, weights)
        x_h = torch.from_numpy(synth.calibration_images(seed=5, count=per, start=rank * per)).pin_memory()
        m.set_tensor("input", x_h)
        for _ in range(args.warmup):
            m.invoke()
        barrier()
        ms = []
        for _ in range(args.steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            m.invoke()
            e1.record()
            e1.synchronize()
            ms.append(e0.elapsed_time(e1))
        barrier()
        total_ms = float(np.sum(ms))
        # end to end: pinned host images in, int8 logits out, every step
        t0 = time.perf_counter()
        for _ in range(args.steps):
            m.set_tensor("input", x_h)
            m.invoke()
            logits = m.tensors["fc"].cpu()
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        t = torch.tensor([total_ms, e2e_s], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            line = dict(metric="ResNet-50 int8 img/s", value=GLOBAL_BATCH * args.steps / (float(t[0]) * 1e-3), unit="img/s",
                        ms_per_step=float(t[0]) / args.steps, scaling="strong",
                        config=dict(workload="ResNet-50 INT8 symmetric (random init, calibrated on 64 synthetic images), "
                                             "global batch 256 of 3x224x224, batch sharded over the ranks",
                                    per_gpu_batch=per, kernels_per_step=len(graph["ops"])),
                        e2e=dict(value=GLOBAL_BATCH * args.steps / float(t[1]), unit="img/s",
                                 h2d_bytes_per_step=int(x_h.numel() * 4), d2h_bytes_per_step=int(logits.numel())))
    else:
        TOTAL = int(os.environ.get("B200Q_CALIB_SAMPLES", "2048"))
        per = TOTAL // world
        from tpu_mlir_b200.calibration import ShardedCalibrator
        images = torch.from_numpy(synth.calibration_images(seed=4, count=per, start=rank * per)).to(dev)
        fwd = resnet50.Fp32Forward(ops, dev)
        cal = ShardedCalibrator(fwd, dist=dist if world > 1 else None)
        batches = [images[i:i + 32] for i in range(0, per, 32)]
        cal.run(batches[:2], samples_per_rank=min(64, per)) if per >= 64 else None     # warm-up
        barrier()
        t0 = time.perf_counter()
        res = cal.run(batches, samples_per_rank=per)
        barrier()
        dt = time.perf_counter() - t0
        t = torch.tensor([dt], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            import hashlib
            digest = hashlib.sha256("".join(f"{n} {r.threshold:.7f} {r.min:.7f} {r.max:.7f}\n" for n, r in res.items()).encode()).hexdigest()
            line = dict(metric="calibration samples/s", value=TOTAL / float(t[0]), unit="samples/s", ms_per_step=float(t[0]) * 1e3,
                        scaling="strong",
                        config=dict(workload=f"ResNet-50 fp32 forward (torch) x2 passes + min/max, streaming histogram (2048 bins) "
                                             f"and KLD on {len(res)} tensors, {TOTAL} synthetic samples sharded over the ranks",
                                    table_sha256=digest, tensors=len(res)))
    if rank == 0 and line:
        line.update(n_gpus=world, steps=args.steps, warmup=args.warmup, higher_is_better=True, data="synthetic")
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="conv", choices=["conv", "gemm", "conv1x1", "a16", "hist", "resnet50", "calib"],
                    help="conv = the benchmark contract (BASELINE config 1); the others time one more kernel each")
    ap.add_argument("--skip-cpu", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    ap.add_argument("--skip-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference(args)
    if args.workload in ("resnet50", "calib"):
        return run_network_workload(args)
    if args.workload != "conv":
        return run_kernel_workload(args)

    import torch
    import torch.distributed as dist
    import tpu_mlir_b200._lib as L
    from tpu_mlir_b200 import synth
    from tpu_mlir_b200.ops import Conv2DOp, InferenceParameter

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
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
    x_d, y_d = x_sets[0], y_sets[0]
    h = C.c_void_p()
    L.check(lib.b200q_conv2d_dev_create(C.byref(op.desc), C.c_void_p(w_d.data_ptr()), C.c_void_p(b_d.data_ptr()),
                                        C.byref(h)))

    def step_device(i):
        L.check(lib.b200q_conv2d_dev_run(h, C.c_void_p(x_sets[i % NSETS].data_ptr()),
                                         C.c_void_p(y_sets[i % NSETS].data_ptr()), sptr))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    with torch.cuda.stream(stream):
        for i in range(args.warmup):
            step_device(i)
        L.check(lib.b200q_conv2d_dev_status(h, sptr))
        barrier()
        t_wall0 = time.time()
        # pass 1, the timed region: K steps as a user runs them (no events between the kernels, so the convolution
        # kernel launches as a programmatic dependent of its layout kernel)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(args.steps):
            step_device(i)
        e1.record(stream)
        e1.synchronize()
        L.check(lib.b200q_conv2d_dev_status(h, sptr))
        barrier()
        step_ms = [e0.elapsed_time(e1)]
        # pass 2, the same K steps with the library recording events around each kernel: the per-kernel durations
        # behind `roofline` (the events serialise the two kernels, so their sum is a little above a step of pass 1)
        L.check(lib.b200q_conv2d_dev_set_profiling(h, 1))
        for i in range(args.steps):
            step_device(i)
        stream.synchronize()
        L.check(lib.b200q_conv2d_dev_status(h, sptr))
        barrier()
        clocks = sampler.stop(t_wall0, time.time()) if rank == 0 else None
        runs, lay, ker = C.c_int64(), C.c_double(), C.c_double()
        L.check(lib.b200q_conv2d_dev_profile(h, C.byref(runs), C.byref(lay), C.byref(ker)))
        layout_ms, kernel_ms = [lay.value / runs.value], [ker.value / runs.value]
        L.check(lib.b200q_conv2d_dev_set_profiling(h, 0))
        y_d = y_sets[(args.steps - 1) % NSETS]
    total_ms = float(np.sum(step_ms))
    gpu_launches = 2 * args.steps

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
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            op.inference(p)          # synchronous: H2D, layout, conv, D2H
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        op.deinit(p)
        same = bool(np.array_equal(y_h.numpy(), y_d.cpu().numpy().astype(np.float32)))
        if not same:
            raise SystemExit("operator face and device face disagree")
        e2e = dict(s=e2e_s, h2d=int(x_h.numel() * 4), d2h=int(y_h.numel() * 4))
        gpu_launches += 3 * 8 * args.steps  # per piece of the batch (8 pieces): f32->bordered layout, conv, int8->f32

    # ---- aggregate over ranks (max time)
    t = torch.tensor([total_ms, e2e["s"] if e2e else 0.0], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_s = float(t[0]), float(t[1])

    if rank == 0:
        peaks = measured_peaks()
        int8_peak = 2.0 * peaks["bf16_tflops"]
        value = world * OPS_PER_STEP * args.steps / (total_ms * 1e-3) / 1e12
        k_ms = float(np.mean(kernel_ms))
        achieved = OPS_PER_STEP / (k_ms * 1e-3) / 1e12
        line = dict(metric=METRIC, value=value, unit=UNIT, n_gpus=world, steps=args.steps, warmup=args.warmup,
                    ms_per_step=total_ms / args.steps, higher_is_better=True, scaling="weak", vs_baseline=None,
                    dtype="s8 x s8 -> s32 accumulate -> s8", data="synthetic",
                    config=dict(workload=WORKLOAD, l2="6 input/output sets used round-robin (308 MB > L2), no flush kernel",
                                per_step_kernels=dict(layout_ms=float(np.mean(layout_ms)), conv_ms=k_ms,
                                                      source="a second pass of the same K steps with CUDA events "
                                                             "recorded around each kernel")),
                    roofline=dict(bound="tensor", achieved=achieved, peak=int8_peak, unit="TOPS",
                                  frac=achieved / int8_peak, traffic=CONV_DRAM_BYTES_PER_LAUNCH,
                                  traffic_source="ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch "
                                                 "(profiles/igemm_i8_conv_config1.md)",
                                  peak_basis=f"2 x {peaks['source']} dense bf16 ({peaks['bf16_tflops']} TFLOP/s); "
                                             "no measured INT8 figure exists"),
                    clocks=clocks, gpu_launches=gpu_launches)
        if e2e:
            line["e2e"] = dict(value=world * OPS_PER_STEP * args.steps / e2e_s / 1e12, unit=UNIT,
                               h2d_bytes_per_step=e2e["h2d"], d2h_bytes_per_step=e2e["d2h"],
                               ms_per_step=e2e_s / args.steps * 1e3,
                               api="b200q_conv2d_inference (host float32 buffers, pinned)")
        if not args.skip_cpu and world >= 1:
            n_img = 8
            threads = os.cpu_count() or 1
            secs, out = cpu_route(c, n_img, threads)
            if not np.array_equal(out, y_d[:n_img].cpu().numpy()):
                raise SystemExit("GPU result differs from the CPU route on the sampled images")
            line["cpu_baseline"] = dict(value=OPS_PER_STEP * n_img / CFG["N"] / secs / 1e12, unit=UNIT, cores=threads,
                                        kind="port", sample=f"first {n_img} of 32 images, fp32 oneDNN conv + requant "
                                                            f"loop, {secs:.3f} s")
        print(json.dumps(line))
    lib.b200q_conv2d_dev_destroy(C.byref(h))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
