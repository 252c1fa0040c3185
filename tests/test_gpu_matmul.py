"""INT8 MatMul parity on the GPU: every kernel result must equal the CPU oracle bit for bit."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import tpu_mlir_b200._lib as L
from tpu_mlir_b200 import synth
from tpu_mlir_b200.ops import InferenceParameter, MatMulOp

from gpu_util import Guarded, NP_OF_DT, TORCH_OF_NP, dev, dt_of, empty_dev, make_epilogue, ptr

pytestmark = pytest.mark.gpu


def run_gemm_dev(A, B_kn, epi_kwargs, algo):
    M, K = A.shape
    N = B_kn.shape[1]
    e, keep = make_epilogue(**epi_kwargs)
    a_d, b_d = dev(A), dev(np.ascontiguousarray(B_kn.T))
    # canary bytes around the output: a store past a ragged edge of the last tile fails the test
    guard = Guarded((M, N), TORCH_OF_NP[np.dtype(NP_OF_DT[epi_kwargs.get("out_dtype", L.DT_I8)])])
    out = guard.view
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    L.check(L.lib().b200q_gemm_i8_dev(ptr(a_d), dt_of(A), ptr(b_d), dt_of(B_kn), M, N, K, C.byref(e), ptr(out),
                                      ptr(status), algo, None))
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"kernel wait timed out at site {int(status.item())}"
    guard.check()
    return out.cpu().numpy()


@pytest.mark.parametrize("algo", [L.ALGO_TENSOR_CORE, L.ALGO_CUDA_CORE])
def test_config0_qdm_per_channel(algo):
    """BASELINE config 0: 512x1024x1024, per-channel QDM requant, half away from zero."""
    c = synth.matmul_int8(seed=0)
    # oracle: int32 MatMul followed by per-channel RequantIntAxis in TFLite mode with full-width multipliers
    acc, viol = oracle.matmul_int8(c["A"], c["B"], c["bias"], out_dt=oracle.DT_I32, return_violations=True)
    assert viol == 0
    quant3 = np.stack([c["mult"], -c["rshift"], np.zeros_like(c["mult"])], axis=1)
    # RequantIntAxis wants the channel on axis 1: view [M,N] as [M,N,1]
    want = oracle.requant_int_axis(acc.reshape(acc.shape[0], acc.shape[1], 1), quant3, qmode=oracle.QM_TFLITE,
                                   rmode=oracle.RM_HALF_AWAY, out_dt=oracle.DT_I8).reshape(acc.shape)
    got = run_gemm_dev(c["A"], c["B"], dict(dialect=L.RQ_QDM, round_mode=L.ROUND_HALF_AWAY_FROM_ZERO, mult=c["mult"],
                                            shift=-c["rshift"], bias=c["bias"]), algo)
    assert np.array_equal(got, want)


DIALECTS = [
    dict(dialect=L.RQ_MULTIPLIER_SHIFT, round_mode=L.ROUND_HALF_UP),
    dict(dialect=L.RQ_MULTIPLIER_SHIFT, round_mode=L.ROUND_HALF_TO_EVEN),
    dict(dialect=L.RQ_QDM, round_mode=L.ROUND_HALF_AWAY_FROM_ZERO),
    dict(dialect=L.RQ_QDM, round_mode=L.ROUND_HALF_UP),
    dict(dialect=L.RQ_MULTIPLIER_SHIFT_F32, round_mode=L.ROUND_HALF_AWAY_FROM_ZERO),
    dict(dialect=L.RQ_ONLY_SHIFT, round_mode=L.ROUND_HALF_UP),
    dict(dialect=L.RQ_ONLY_SHIFT, round_mode=L.ROUND_TOWARDS_ZERO),
]


def oracle_requant(acc, dialect, round_mode, mult, shift, out_zp, relu_after, out_dt):
    """Elementwise oracle for one device-face dialect (per channel = last axis)."""
    out = np.empty(acc.shape, dtype=np.int64)
    for n in range(acc.shape[1]):
        for m in range(acc.shape[0]):
            a = int(acc[m, n])
            if dialect == L.RQ_MULTIPLIER_SHIFT:
                v = oracle.apply_multiplier_rshift(a, mult[n], shift[n], oracle.QM_MULTIPLIER_SHIFT, round_mode, False)
            elif dialect == L.RQ_QDM:
                v = oracle.mbqm(a, mult[n], shift[n], round_mode)
            elif dialect == L.RQ_MULTIPLIER_SHIFT_F32:
                v = oracle.apply_multiplier_rshift(a, mult[n], shift[n], oracle.QM_MULTIPLIER_SHIFT, round_mode, True)
            else:
                v = oracle.apply_multiplier_rshift(a, 1, shift[n], oracle.QM_ONLY_SHIFT, round_mode, False)
            v += out_zp
            if relu_after and v < out_zp:
                v = out_zp
            out[m, n] = oracle.saturate(v, out_dt)
    return out


@pytest.mark.parametrize("algo", [L.ALGO_TENSOR_CORE, L.ALGO_CUDA_CORE])
@pytest.mark.parametrize("case", range(len(DIALECTS)))
def test_requant_dialects_small(algo, case):
    d = DIALECTS[case]
    rng = np.random.default_rng(100 + case)
    M, K, N = 70, 48, 40            # ragged against the 128 x 64 tile on purpose
    A = rng.integers(0, 256, size=(M, K), dtype=np.uint8)
    B = rng.integers(-128, 128, size=(K, N), dtype=np.int8)
    bias = rng.integers(-3000, 3000, size=N, dtype=np.int32)
    if d["dialect"] == L.RQ_QDM:
        mult = rng.integers(2**30, 2**31, size=N)
        shift = -rng.integers(0, 12, size=N)
        shift[:3] = [1, 2, 0]       # left shifts too
    elif d["dialect"] == L.RQ_MULTIPLIER_SHIFT:
        mult = rng.integers(-3000, 30000, size=N)
        shift = rng.integers(8, 26, size=N)
        shift[:3] = [0, -2, 40]     # no shift, left shift, long shift
    elif d["dialect"] == L.RQ_MULTIPLIER_SHIFT_F32:
        mult = rng.integers(1, 20000, size=N)
        shift = rng.integers(8, 25, size=N)
    else:
        mult = np.ones(N, dtype=np.int64)
        shift = rng.integers(4, 12, size=N)
    acc = oracle.matmul_int8(A, B, bias, out_dt=oracle.DT_I32)
    for out_dt, zp, relu in ((L.DT_I8, 3, L.RELU_NONE), (L.DT_U8, 0, L.RELU_AFTER_REQUANT), (L.DT_I16, -5, L.RELU_NONE)):
        want = oracle_requant(acc, d["dialect"], d["round_mode"], mult, shift, zp, relu == L.RELU_AFTER_REQUANT, out_dt)
        got = run_gemm_dev(A, B, dict(dialect=d["dialect"], round_mode=d["round_mode"], mult=mult, shift=shift,
                                      bias=bias, out_zp=zp, relu=relu, out_dtype=out_dt), algo)
        assert np.array_equal(got.astype(np.int64), want), (d, out_dt)


# the last shape has enough 128-row tiles for the CTA-pair (256-row tile) form of the tensor-core kernel, ragged in M, K and N
@pytest.mark.parametrize("shape", [(1, 16, 8), (129, 272, 257), (300, 1040, 96), (128, 128, 64), (5, 4096, 1000),
                                   (38437, 272, 300)])
def test_ragged_shapes_tensor_core(shape):
    M, K, N = shape
    rng = np.random.default_rng(M * 7 + N)
    A = rng.integers(-128, 128, size=(M, K), dtype=np.int8)
    B = rng.integers(-128, 128, size=(K, N), dtype=np.int8)
    bias = rng.integers(-2**16, 2**16, size=N, dtype=np.int32)
    mult, rshift = synth.qdm_params(rng, N)
    want = oracle.matmul_int8(A, B, bias, out_dt=oracle.DT_I32)
    got = run_gemm_dev(A, B, dict(dialect=L.RQ_NONE, round_mode=0, bias=bias, out_dtype=L.DT_I32), L.ALGO_TENSOR_CORE)
    assert np.array_equal(got, want)
    got = run_gemm_dev(A, B, dict(dialect=L.RQ_QDM, round_mode=L.ROUND_HALF_AWAY_FROM_ZERO, mult=mult, shift=-rshift,
                                  bias=bias, relu=L.RELU_BEFORE_REQUANT), L.ALGO_TENSOR_CORE)
    quant3 = np.stack([mult, -rshift, np.zeros_like(mult)], axis=1)
    relu_acc = np.maximum(want, 0)
    ref = oracle.requant_int_axis(relu_acc.reshape(M, N, 1), quant3, qmode=oracle.QM_TFLITE, rmode=oracle.RM_HALF_AWAY,
                                  out_dt=oracle.DT_I8).reshape(M, N)
    assert np.array_equal(got, ref)


def test_unsigned_by_unsigned_extreme_accumulators():
    """u8 x u8 products reach 65025: the folded epilogue forms must size their accumulator bound from the operand
    signedness.  All-255 operands, a large multiplier and a small shift drive every intermediate to its limit; half of
    the columns use a mild pair so that unsaturated values are checked too."""
    M, K, N = 128, 2048, 128
    A = np.full((M, K), 255, np.uint8)
    B = np.full((K, N), 255, np.uint8)
    B[:, ::3] = np.random.default_rng(1).integers(0, 256, (K, len(range(0, N, 3))), dtype=np.uint8)
    mult = np.where(np.arange(N) % 2 == 0, 30000, 3).astype(np.int64)
    shift = np.where(np.arange(N) % 2 == 0, 3, 21).astype(np.int64)
    acc = A.astype(np.int64) @ B.astype(np.int64)
    for out_dt, odt in ((L.DT_I8, oracle.DT_I8), (L.DT_U8, oracle.DT_U8)):
        want = oracle_requant(acc, L.RQ_MULTIPLIER_SHIFT, L.ROUND_HALF_UP, mult, shift, 0, False, odt)
        got = run_gemm_dev(A, B, dict(dialect=L.RQ_MULTIPLIER_SHIFT, round_mode=L.ROUND_HALF_UP, mult=mult, shift=shift, out_dtype=out_dt),
                           L.ALGO_TENSOR_CORE)
        assert np.array_equal(got.astype(np.int64), want) and len(np.unique(want)) > 5, out_dt


# ------------------------------------------------------------------ operator face (host float buffers)
def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


@pytest.mark.parametrize("right_transpose", [False, True])
def test_operator_face_fuse_rq_per_channel(right_transpose):
    """tpu.MatMul, MultiplierShift with fuse_rq: per-channel multiplier in operand 3, one common rshift."""
    rng = np.random.default_rng(5)
    M, K, N = 96, 256, 200
    A = rng.integers(0, 256, size=(M, K), dtype=np.uint8)
    B = rng.integers(-128, 128, size=(K, N), dtype=np.int8)
    bias = rng.integers(-2**15, 2**15, size=N, dtype=np.int32)
    multi = rng.integers(2**20, 2**27, size=N).astype(np.int64)      # loses low bits in the float operand
    rshift = 30
    multi_seen = oracle.through_f32(multi)
    want = oracle.matmul_int8(A, B, bias, do_relu=True, qmode=oracle.QM_MULTIPLIER_SHIFT, fuse_rq=True,
                              mult=multi_seen, rshift=[rshift], out_zp=0, out_dt=oracle.DT_U8)
    op = MatMulOp(M=M, K=K, N=N, with_bias=True, do_relu=True, right_transpose=right_transpose,
                  input_dtype=L.DT_U8, out_dtype=L.DT_U8, quant_mode=L.QM_MULTIPLIER_SHIFT, fuse_rq=True,
                  multipliers=[1], rshifts=[rshift])
    out = np.zeros((M, N), np.float32)
    p = InferenceParameter(inputs=[f32(A), f32(B.T if right_transpose else B), f32(bias), f32(multi), None],
                           outputs=[out])
    op.init(p)
    op.inference(p)
    op.inference(p)              # second call uses the resident weights
    op.deinit(p)
    assert np.array_equal(out, want.astype(np.float32))
    # like the reference, inference also works without a prior init
    out2 = np.zeros_like(out)
    p2 = InferenceParameter(inputs=p.inputs, outputs=[out2])
    op.inference(p2)
    assert np.array_equal(out2, out)


@pytest.mark.parametrize("qmode,cv18xx", [(L.QM_TFLITE, False), (L.QM_MULTIPLIER_SHIFT, False), (L.QM_QDM, True),
                                          (L.QM_MULTIPLIER_SHIFT, True), (L.QM_ONLY_SCALE, False)])
def test_operator_face_per_tensor_modes(qmode, cv18xx):
    rng = np.random.default_rng(11 + qmode)
    batch, M, K, N = 3, 20, 64, 48
    A = rng.integers(-128, 128, size=(batch, M, K), dtype=np.int8)
    B = rng.integers(-128, 128, size=(K, N), dtype=np.int8)
    bias = rng.integers(-1000, 1000, size=N, dtype=np.int32)
    if qmode == L.QM_MULTIPLIER_SHIFT:
        mult, rs = [177], [14]
    else:
        mult, rs = [1518500250], [7]
    if cv18xx:
        mult, rs = mult * batch, [rs[0] + i for i in range(batch)]
    kw = dict(qmode=qmode, is_cv18xx=cv18xx, mult=mult, rshift=rs, out_zp=0 if cv18xx else 2, only_scale=0.0123)
    want = np.stack([oracle.matmul_int8(A[b], B, bias, **{**kw, "mult": mult[b:b + 1] if cv18xx else mult,
                                                          "rshift": rs[b:b + 1] if cv18xx else rs})
                     for b in range(batch)])
    op = MatMulOp(batch=batch, M=M, K=K, N=N, with_bias=True, quant_mode=qmode, is_cv18xx=cv18xx, multipliers=mult,
                  rshifts=rs, out_zp=0 if cv18xx else 2, out_scale=0.0123)
    out = np.zeros((batch, M, N), np.float32)
    p = InferenceParameter(inputs=[f32(A), f32(B), f32(bias)], outputs=[out])
    op.inference(p)
    assert np.array_equal(out, want.astype(np.float32))


def test_operator_face_zero_points_and_batched_right():
    rng = np.random.default_rng(3)
    batch, M, K, N = 2, 17, 40, 24
    A = rng.integers(0, 256, size=(batch, M, K), dtype=np.uint8)
    B = rng.integers(-128, 128, size=(batch, K, N), dtype=np.int8)
    want = oracle.matmul_int8(A, B, None, input_zp=7, right_zp=-3, qmode=oracle.QM_MULTIPLIER_SHIFT, mult=[3], rshift=[9],
                              out_zp=1)
    op = MatMulOp(batch=batch, M=M, K=K, N=N, right_batched=True, right_is_weight=False, input_zp=7, right_zp=-3,
                  input_dtype=L.DT_U8, multipliers=[3], rshifts=[9], out_zp=1)
    out = np.zeros((batch, M, N), np.float32)
    op.inference(InferenceParameter(inputs=[f32(A), f32(B)], outputs=[out]))
    assert np.array_equal(out, want.astype(np.float32))


@pytest.mark.parametrize("lt,ot", [(True, False), (False, True), (True, True)])
@pytest.mark.parametrize("batch,right_batched", [(1, False), (3, True), (2, False)])
def test_operator_face_left_and_output_transpose(lt, ot, batch, right_batched):
    """left_transpose: inputs[0] holds [batch][K][M]; output_transpose: outputs[0] holds [batch][N][M]
    (MatMul.cpp:24-135; lib/Support/Dnnl/MatMul.cpp:182-186,:229-238 transpose around the product)."""
    rng = np.random.default_rng(31 + batch)
    M, K, N = 45, 96, 40
    A = rng.integers(-128, 128, size=(batch, M, K), dtype=np.int8)
    B = rng.integers(-128, 128, size=(batch, K, N) if right_batched else (K, N), dtype=np.int8)
    bias = rng.integers(-2**12, 2**12, size=N, dtype=np.int32)
    want = np.stack([oracle.matmul_int8(A[b], B[b] if right_batched else B, bias, qmode=oracle.QM_MULTIPLIER_SHIFT, mult=[5], rshift=[11])
                     for b in range(batch)])
    op = MatMulOp(batch=batch, M=M, K=K, N=N, with_bias=True, left_transpose=lt, output_transpose=ot, right_batched=right_batched,
                  right_is_weight=not right_batched, multipliers=[5], rshifts=[11])
    a_in = np.ascontiguousarray(A.transpose(0, 2, 1)) if lt else A
    out = np.zeros((batch, N, M) if ot else (batch, M, N), np.float32)
    op.inference(InferenceParameter(inputs=[f32(a_in), f32(B), f32(bias)], outputs=[out]))
    got = out.transpose(0, 2, 1) if ot else out
    assert np.array_equal(got, want.astype(np.float32)) and len(np.unique(want)) > 50


@pytest.mark.parametrize("lt,rt,ot", [(True, True, True), (False, True, True), (True, False, False), (False, False, True)])
def test_operator_face_hdim_is_batch(lt, rt, ot):
    """hdim_is_batch (MatMul.cpp:58-104; lib/Support/Dnnl/MatMul.cpp:172-241): batch x batch_low products; a transposed
    operand holds batch_low between its matrix dimensions, (B0, M, B1, K) x (B0, K, B1, N) = (B0, M, B1, N), and is put in
    batch-major order by tensor_hc_transpose; an operand without its flag already is."""
    rng = np.random.default_rng(41)
    B0, B1, M, K, N = 2, 3, 37, 64, 48
    A = rng.integers(-128, 128, size=(B0, B1, M, K), dtype=np.int8)
    Bm = rng.integers(-128, 128, size=(B0, B1, K, N), dtype=np.int8)
    want = np.stack([np.stack([oracle.matmul_int8(A[i, j], Bm[i, j], None, qmode=oracle.QM_MULTIPLIER_SHIFT, mult=[7], rshift=[12], out_zp=-2,
                                                  do_relu=True) for j in range(B1)]) for i in range(B0)])
    op = MatMulOp(batch=B0, batch_low=B1, M=M, K=K, N=N, hdim_is_batch=True, left_transpose=lt, right_transpose=rt, output_transpose=ot,
                  right_batched=True, right_is_weight=False, do_relu=True, multipliers=[7], rshifts=[12], out_zp=-2)
    a_in = np.ascontiguousarray(A.transpose(0, 2, 1, 3)) if lt else A
    b_in = np.ascontiguousarray(Bm.transpose(0, 2, 1, 3)) if rt else Bm
    out = np.zeros((B0, M, B1, N) if ot else (B0, B1, M, N), np.float32)
    op.inference(InferenceParameter(inputs=[f32(a_in), f32(b_in)], outputs=[out]))
    got = out.transpose(0, 2, 1, 3) if ot else out
    assert np.array_equal(got, want.astype(np.float32)) and len(np.unique(want)) > 50


def test_empty_and_errors():
    op = MatMulOp(M=0, K=16, N=8, multipliers=[1], rshifts=[0])
    out = np.zeros((0, 8), np.float32)
    op.inference(InferenceParameter(inputs=[np.zeros((0, 16), np.float32), np.zeros((16, 8), np.float32)], outputs=[out]))
    op = MatMulOp(M=4, K=16, N=8, hdim_is_batch=True, multipliers=[1], rshifts=[0])      # needs a batched right operand
    with pytest.raises(L.B200QError) as ei:
        op.inference(InferenceParameter(inputs=[np.zeros((4, 16), np.float32), np.zeros((16, 8), np.float32)],
                                        outputs=[np.zeros((4, 8), np.float32)]))
    assert ei.value.code == L.ERR_INVALID
    op = MatMulOp(M=4, K=16, N=8, quant_mode=L.QM_QDM, multipliers=[1], rshifts=[0])
    with pytest.raises(L.B200QError) as ei:
        op.inference(InferenceParameter(inputs=[np.zeros((4, 16), np.float32), np.zeros((16, 8), np.float32)],
                                        outputs=[np.zeros((4, 8), np.float32)]))
    assert ei.value.code == L.ERR_UNSUPPORTED


@pytest.mark.parametrize("shape", [(128, 128, 256), (4864, 2048, 128)], ids=["one_tile", "cta_pairs"])
def test_a_wait_that_runs_out_is_reported_and_the_next_launch_is_exact(shape):
    """Failure detection without a fault: every stage's barrier is told to expect 16 bytes more than the stage's loads
    deliver, so the consumer's bounded wait runs out after 1 ms.  The kernel ends by itself with the wait site in its
    status word, and the same launch without the aid is bit exact afterwards."""
    M, N, K = shape
    rng = np.random.default_rng(77)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    B = rng.integers(-128, 128, (K, N), dtype=np.int8)
    mult, rshift = synth.qdm_params(rng, N)
    e, keep = make_epilogue(dialect=L.RQ_QDM, round_mode=L.ROUND_HALF_AWAY_FROM_ZERO, mult=mult, shift=-rshift)
    a_d, b_d = dev(A), dev(np.ascontiguousarray(B.T))
    out = empty_dev((M, N), L.DT_I8)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib = L.lib()

    def launch():
        L.check(lib.b200q_gemm_i8_dev(ptr(a_d), L.DT_I8, ptr(b_d), L.DT_I8, M, N, K, C.byref(e), ptr(out), ptr(status),
                                      L.ALGO_TENSOR_CORE, None))
        torch.cuda.synchronize()
        return int(status.item())

    lib.b200q_debug_set_wait_fault(16, 1_000_000)
    try:
        site = launch()
    finally:
        lib.b200q_debug_set_wait_fault(0, 0)
    assert site in (1, 2, 3, 4), site          # a wait site of the pipeline, most often 3: the MMA warp's wait for a stage
    status.zero_()
    assert launch() == 0
    acc = A.astype(np.int32) @ B.astype(np.int32)
    want = oracle.requant_int_axis(acc.reshape(M, N, 1), np.stack([mult, -rshift, np.zeros_like(mult)], axis=1),
                                   qmode=oracle.QM_TFLITE, rmode=oracle.RM_HALF_AWAY, out_dt=oracle.DT_I8).reshape(M, N)
    assert np.array_equal(out.cpu().numpy(), want)


def test_operator_face_reports_the_timeout_code():
    rng = np.random.default_rng(6)
    A = rng.integers(-128, 128, (128, 256), dtype=np.int8)
    B = rng.integers(-128, 128, (256, 128), dtype=np.int8)
    want = oracle.matmul_int8(A, B, None, qmode=oracle.QM_MULTIPLIER_SHIFT, mult=[3], rshift=[12])
    op = MatMulOp(M=128, K=256, N=128, multipliers=[3], rshifts=[12], algo=L.ALGO_TENSOR_CORE)
    y = np.zeros((128, 128), np.float32)
    p = InferenceParameter(inputs=[f32(A), f32(B)], outputs=[y])
    op.init(p)
    lib = L.lib()
    lib.b200q_debug_set_wait_fault(16, 1_000_000)
    try:
        with pytest.raises(L.B200QError) as ei:
            op.inference(p)
    finally:
        lib.b200q_debug_set_wait_fault(0, 0)
    assert ei.value.code == L.ERR_TIMEOUT
    op.inference(p)          # the context is intact: the next call succeeds and is exact
    op.deinit(p)
    assert np.array_equal(y, want.astype(np.float32))


def test_tensor_pipe_probe_reports_a_plausible_peak():
    ms, ops = C.c_double(), C.c_double()
    for kind, pair, lo, hi in ((0, 0, 1500, 5000), (0, 1, 1500, 5000), (1, 0, 800, 2500)):
        L.check(L.lib().b200q_probe_tensor_peak(kind, pair, 8000, 4, C.byref(ms), C.byref(ops), None))
        t = ops.value / (ms.value * 1e-3) / 1e12
        assert lo < t < hi, (kind, pair, t)
