"""A16MatMul w4bf16 on the GPU against the oracle's restatement of the interpreter (tolerance, not bit parity:
the reference's fp32 GEMM has no fixed summation order)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import tpu_mlir_b200._lib as L
from tpu_mlir_b200 import synth
from tpu_mlir_b200.ops import A16MatMulOp, InferenceParameter

from gpu_util import dev, ptr

pytestmark = pytest.mark.gpu


def check(y_bits, ref_bits):
    """|y - y_ref| <= 1e-2 * max(|y_ref|, 1e-2 * rms(y_ref)): relative 1e-2 with a floor for outputs near zero."""
    y, r = oracle.bf16_bits_to_f32(y_bits).astype(np.float64), oracle.bf16_bits_to_f32(ref_bits).astype(np.float64)
    rms = np.sqrt(np.mean(r * r))
    tol = 1e-2 * np.maximum(np.abs(r), 1e-2 * rms)
    bad = np.abs(y - r) > tol
    assert not bad.any(), (int(bad.sum()), float(np.abs(y - r).max()), float(rms))


def run_dev(c, M, N, K, group, bias=None):
    x, wq, sc, zp = dev(c["x"]), dev(c["wq"]), dev(c["scale"]), dev(c["zp"])
    b = dev(bias) if bias is not None else None
    y = torch.empty((M, N), dtype=torch.uint16, device="cuda")
    L.check(L.lib().b200q_a16_w4_dev(ptr(x), ptr(wq), ptr(sc), ptr(zp), ptr(b), ptr(y), M, N, K, group, None, None))
    torch.cuda.synchronize()
    return y.cpu().numpy()


@pytest.mark.parametrize("M", [1, 2, 5, 8, 16])
def test_llama_mlp_shape(M):
    """BASELINE config 2: N=11008, K=4096, group 64 (decode shapes; M=16 exercises the token slicing)."""
    c = synth.a16_w4(seed=2, M=M)
    ref = oracle.a16matmul_w4(c["x"], c["wq"], c["scale"], c["zp"], group=64)
    check(run_dev(c, M, 11008, 4096, 64), ref)


@pytest.mark.parametrize("case", [dict(M=1, K=64, N=16, g=64), dict(M=3, K=256, N=40, g=128), dict(M=8, K=1024, N=17, g=64),
                                  dict(M=4, K=192, N=100, g=64),
                                  # one or two tokens take the CUDA-core kernel (K <= 16384): ragged lane/row splits
                                  dict(M=2, K=11008, N=50, g=128), dict(M=1, K=8192, N=33, g=64),
                                  dict(M=2, K=12288, N=20, g=256),
                                  # groups of 32, several slices per lane, rows fewer than row lanes
                                  dict(M=1, K=96, N=7, g=32), dict(M=2, K=160, N=9, g=32), dict(M=1, K=32768, N=5, g=128),
                                  dict(M=2, K=20480, N=3, g=64), dict(M=1, K=4096, N=1200, g=64)])
def test_small_and_ragged_shapes_with_bias(case):
    c = synth.a16_w4(seed=7, M=case["M"], K=case["K"], N=case["N"], group=case["g"])
    bias = np.random.default_rng(1).standard_normal(case["N"]).astype(np.float32)
    ref = oracle.a16matmul_w4(c["x"], c["wq"], c["scale"], c["zp"], bias, group=case["g"])
    check(run_dev(c, case["M"], case["N"], case["K"], case["g"], bias), ref)


def test_operator_face():
    M, K, N, g = 4, 512, 96, 64
    c = synth.a16_w4(seed=9, M=M, K=K, N=N, group=g)
    ref = oracle.a16matmul_w4(c["x"], c["wq"], c["scale"], c["zp"], group=g)
    f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32)  # noqa: E731
    op = A16MatMulOp(M=M, K=K, N=N, q_group_size=g)
    out = np.zeros((M, N), np.float32)
    p = InferenceParameter(inputs=[oracle.bf16_bits_to_f32(c["x"]), f32(c["wq"]), oracle.bf16_bits_to_f32(c["scale"]),
                                   f32(c["zp"]), None], outputs=[out])
    op.init(p)
    op.inference(p)
    op.inference(p)
    op.deinit(p)
    check(oracle.f32_to_bf16_bits_fast(out), ref)
    assert np.array_equal(oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits_fast(out)), out), "output is bf16-representable"


def test_unsupported_is_reported():
    # a group size that is not a multiple of 32 has no kernel
    op = A16MatMulOp(M=1, K=96, N=16, q_group_size=48)
    with pytest.raises(L.B200QError) as ei:
        op.inference(InferenceParameter(inputs=[np.zeros((1, 96), np.float32), np.zeros((16, 48), np.float32),
                                                np.zeros(32, np.float32), np.zeros(32, np.float32), None],
                                        outputs=[np.zeros((1, 16), np.float32)]))
    assert ei.value.code == L.ERR_UNSUPPORTED


def check_prefill(y_bits, ref_f32):
    """Prefill rounds the dequantised weight to bf16 before the tensor-core GEMM (2^-9 relative per weight, which
    shows up as ~1e-3 * rms(y) of absolute noise), so the floor of the relative bound is rms(y_ref) itself, and
    both sides are rounded to bf16 afterwards, which can add one bf16 ulp:
    |y - y_ref| <= 1e-2 * max(|y_ref|, rms(y_ref)) + ulp_bf16(y_ref)."""
    y = oracle.bf16_bits_to_f32(y_bits).astype(np.float64)
    r = np.asarray(ref_f32, dtype=np.float64)
    rms = np.sqrt(np.mean(r * r))
    ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(r), 1e-30))) - 7)
    bad = np.abs(y - r) > 1e-2 * np.maximum(np.abs(r), rms) + ulp
    assert not bad.any(), (int(bad.sum()), float(np.abs(y - r).max()), float(rms))
    assert float(np.sqrt(np.mean((y - r) ** 2))) < 3e-3 * rms


def run_handle(c, M, N, K, group, bias=None):
    x, wq, sc, zp = dev(c["x"]), dev(c["wq"]), dev(c["scale"]), dev(c["zp"])
    b = dev(bias) if bias is not None else None
    y = torch.empty((M, N), dtype=torch.uint16, device="cuda")
    h = C.c_void_p()
    lib = L.lib()
    L.check(lib.b200q_a16_dev_create(ptr(wq), ptr(sc), ptr(zp), ptr(b), N, K, group, C.byref(h)))
    for _ in range(2):     # the second run reuses the dequantised weight kept in the handle
        L.check(lib.b200q_a16_dev_run(h, ptr(x), ptr(y), M, None))
    L.check(lib.b200q_a16_dev_status(h, None))
    lib.b200q_a16_dev_destroy(C.byref(h))
    return y.cpu().numpy()


@pytest.mark.parametrize("M", [16, 128])
def test_prefill_llama_mlp_shape_against_oracle(M):
    c = synth.a16_w4(seed=2, M=M)
    ref = oracle.bf16_bits_to_f32(oracle.a16matmul_w4(c["x"], c["wq"], c["scale"], c["zp"], group=64))
    check_prefill(run_handle(c, M, 11008, 4096, 64), ref)


def test_prefill_2048_tokens_against_fp32_matmul():
    """BASELINE config 2 at M=2048: the fp32 reference is the oracle's dequantised weight times x in fp32 (torch)."""
    M = 2048
    c = synth.a16_w4(seed=2, M=M)
    W = torch.from_numpy(oracle.a16_dequant_w4(c["wq"], c["scale"], c["zp"], group=64)).cuda()
    x = torch.from_numpy(oracle.bf16_bits_to_f32(c["x"])).cuda()
    torch.backends.cuda.matmul.allow_tf32 = False
    ref = (x @ W.T).cpu().numpy()
    check_prefill(run_handle(c, M, 11008, 4096, 64), ref)


def test_prefill_ragged_with_bias():
    M, K, N, g = 37, 320, 200, 64
    c = synth.a16_w4(seed=5, M=M, K=K, N=N, group=g)
    bias = np.random.default_rng(2).standard_normal(N).astype(np.float32)
    ref = oracle.bf16_bits_to_f32(oracle.a16matmul_w4(c["x"], c["wq"], c["scale"], c["zp"], bias, group=g))
    check_prefill(run_handle(c, M, N, K, g, bias), ref)
