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
                                  dict(M=2, K=20480, N=3, g=64), dict(M=1, K=4096, N=1200, g=64),
                                  # long rows: the activations of 3 to 8 tokens and two weight stages do not fit in shared memory,
                                  # so K runs as two or three ranges whose fp32 partial sums meet in a workspace
                                  dict(M=5, K=11008, N=130, g=64), dict(M=8, K=11008, N=4096, g=64), dict(M=8, K=12288, N=40, g=128),
                                  dict(M=8, K=16512, N=33, g=64), dict(M=3, K=11008, N=17, g=128)])
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


def check_f32(y_bits, ref_f32):
    """The plain bound of `check` against an fp32 reference: |y - y_ref| <= 1e-2 * max(|y_ref|, 1e-2 * rms(y_ref)),
    after rounding the reference to bf16 like the reference's own output."""
    check(y_bits, oracle.f32_to_bf16_bits_fast(np.asarray(ref_f32, dtype=np.float32)))


def check_rounded_weight(y_bits, ref_f32):
    """The route that keeps a bf16 copy of the dequantised weight (b200q_a16_set_route(3), and the handle's choice from
    64 tokens on) rounds W to bf16 (2^-9 relative per weight, ~1e-3 * rms(y) of absolute noise), which the reference
    does not; its bound has rms(y_ref) as the floor and one bf16 ulp for the output rounding on both sides:
    |y - y_ref| <= 1e-2 * max(|y_ref|, rms(y_ref)) + ulp_bf16(y_ref)."""
    y = oracle.bf16_bits_to_f32(y_bits).astype(np.float64)
    r = np.asarray(ref_f32, dtype=np.float64)
    rms = np.sqrt(np.mean(r * r))
    ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(r), 1e-30))) - 7)
    bad = np.abs(y - r) > 1e-2 * np.maximum(np.abs(r), rms) + ulp
    assert not bad.any(), (int(bad.sum()), float(np.abs(y - r).max()), float(rms))
    assert float(np.sqrt(np.mean((y - r) ** 2))) < 3e-3 * rms


@pytest.fixture
def route():
    """Selects the kernel behind b200q_a16_* for one test and restores the default."""
    lib = L.lib()

    def set_route(r):
        lib.b200q_a16_set_route(r)
    yield set_route
    lib.b200q_a16_set_route(0)


def run_handle(c, M, N, K, group, bias=None):
    x, wq, sc, zp = dev(c["x"]), dev(c["wq"]), dev(c["scale"]), dev(c["zp"])
    b = dev(bias) if bias is not None else None
    y = torch.empty((M, N), dtype=torch.uint16, device="cuda")
    h = C.c_void_p()
    lib = L.lib()
    L.check(lib.b200q_a16_dev_create(ptr(wq), ptr(sc), ptr(zp), ptr(b), N, K, group, C.byref(h)))
    for _ in range(2):     # the second run reuses what the handle keeps
        L.check(lib.b200q_a16_dev_run(h, ptr(x), ptr(y), M, None))
    L.check(lib.b200q_a16_dev_status(h, None))
    lib.b200q_a16_dev_destroy(C.byref(h))
    return y.cpu().numpy()


@pytest.mark.parametrize("M", [16, 48, 128])
def test_prefill_llama_mlp_shape_against_oracle(M):
    """Default routes of the handle API above 8 tokens: below 64 tokens the fused-dequantisation tensor-core kernel, held
    to the plain bound; from 64 tokens the bf16 copy of the weight, held to the bound that allows for its rounding."""
    c = synth.a16_w4(seed=2, M=M)
    if M < 64:
        ref = oracle.a16matmul_w4(c["x"], c["wq"], c["scale"], c["zp"], group=64)
        check(run_handle(c, M, 11008, 4096, 64), ref)
    else:
        W = oracle.a16_dequant_w4(c["wq"], c["scale"], c["zp"], group=64)
        ref = oracle.bf16_bits_to_f32(c["x"]).astype(np.float32) @ W.T
        check_rounded_weight(run_handle(c, M, 11008, 4096, 64), ref)


def test_stateless_call_never_rounds_the_weight():
    """b200q_a16_w4_dev has no handle to keep a copy in: every M above 8 takes the fused kernel, plain bound."""
    c = synth.a16_w4(seed=3, M=128, K=4096, N=2048)
    ref = oracle.a16matmul_w4(c["x"], c["wq"], c["scale"], c["zp"], group=64)
    check(run_dev(c, 128, 2048, 4096, 64), ref)


@pytest.mark.parametrize("M", [1, 2, 3, 4, 7, 8, 33, 300])
def test_tensor_core_kernel_every_token_count(route, M):
    """The fused kernel forced for every M (few-token form up to 4 tokens, token tiles of 32 / 64 / 128 above)."""
    route(2)
    c = synth.a16_w4(seed=11, M=M, K=4096, N=1000, group=64)
    bias = np.random.default_rng(3).standard_normal(1000).astype(np.float32)
    ref = oracle.a16matmul_w4(c["x"], c["wq"], c["scale"], c["zp"], bias, group=64)
    check(run_dev(c, M, 1000, 4096, 64, bias), ref)


@pytest.mark.parametrize("case", [dict(M=1, K=64, N=16, g=64), dict(M=4, K=192, N=100, g=64), dict(M=9, K=256, N=128, g=64),
                                  dict(M=2, K=11008, N=130, g=64), dict(M=33, K=11008, N=130, g=64),
                                  dict(M=100, K=4096, N=384, g=128), dict(M=40, K=2048, N=17, g=256),
                                  # groups of two / four / eight k-blocks with narrow token tiles: fewer MMA issuers in use
                                  dict(M=20, K=4096, N=700, g=128), dict(M=12, K=2048, N=300, g=256), dict(M=50, K=1024, N=260, g=512),
                                  dict(M=24, K=4160, N=200, g=64),
                                  dict(M=3, K=8192, N=300, g=128)])
def test_tensor_core_kernel_shapes(route, case):
    """Ragged rows, K that is not a multiple of a raw stage (256), groups of 128 and 256, many groups per row."""
    route(2)
    c = synth.a16_w4(seed=13, M=case["M"], K=case["K"], N=case["N"], group=case["g"])
    ref = oracle.a16matmul_w4(c["x"], c["wq"], c["scale"], c["zp"], group=case["g"])
    check(run_dev(c, case["M"], case["N"], case["K"], case["g"]), ref)


def test_prefill_2048_tokens_against_fp32_matmul(route):
    """BASELINE config 2 at M=2048: the fp32 reference is the oracle's dequantised weight times x in fp32 (torch).
    The handle's own choice at this size (the bf16 copy of the weight) is held to its wider bound, the fused kernel
    to the plain one."""
    M = 2048
    c = synth.a16_w4(seed=2, M=M)
    W = torch.from_numpy(oracle.a16_dequant_w4(c["wq"], c["scale"], c["zp"], group=64)).cuda()
    x = torch.from_numpy(oracle.bf16_bits_to_f32(c["x"])).cuda()
    torch.backends.cuda.matmul.allow_tf32 = False
    ref = (x @ W.T).cpu().numpy()
    check_rounded_weight(run_handle(c, M, 11008, 4096, 64), ref)
    route(2)
    check_f32(run_handle(c, M, 11008, 4096, 64), ref)


def test_prefill_ragged_with_bias(route):
    M, K, N, g = 37, 320, 200, 64
    c = synth.a16_w4(seed=5, M=M, K=K, N=N, group=g)
    bias = np.random.default_rng(2).standard_normal(N).astype(np.float32)
    ref = oracle.a16matmul_w4(c["x"], c["wq"], c["scale"], c["zp"], bias, group=g)
    check(run_handle(c, M, N, K, g, bias), ref)
    route(3)
    check_rounded_weight(run_handle(c, M, N, K, g, bias), oracle.bf16_bits_to_f32(ref))


# ------------------------------------------------------------------ w4f16
def check_f16(y_bits, ref_bits):
    """The same plain bound on IEEE half outputs."""
    y = np.asarray(y_bits, dtype=np.uint16).view(np.float16).astype(np.float64)
    r = np.asarray(ref_bits, dtype=np.uint16).view(np.float16).astype(np.float64)
    rms = np.sqrt(np.mean(r * r))
    bad = np.abs(y - r) > 1e-2 * np.maximum(np.abs(r), 1e-2 * rms)
    assert not bad.any(), (int(bad.sum()), float(np.abs(y - r).max()), float(rms))


@pytest.mark.parametrize("case", [dict(M=1, K=4096, N=11008, g=64), dict(M=2, K=4096, N=1000, g=64), dict(M=1, K=96, N=7, g=32),
                                  dict(M=5, K=1024, N=300, g=128), dict(M=16, K=4096, N=2048, g=64),
                                  dict(M=100, K=512, N=384, g=64), dict(M=300, K=2048, N=1000, g=256)])
def test_w4f16_device_face(case):
    """out_dtype = F16 (A16MatMul.cpp:240-246 rounds with F16()): f16 activations and scales, f16 output rounded to
    nearest even; one or two tokens on the CUDA cores, everything else through kind::f16 on f16 operands."""
    M, K, N, g = case["M"], case["K"], case["N"], case["g"]
    c = synth.a16_w4(seed=11, M=M, K=K, N=N, group=g, f16=True)
    bias = np.random.default_rng(2).standard_normal(N).astype(np.float32)
    ref = oracle.a16matmul_w4(c["x"], c["wq"], c["scale"], c["zp"], bias, group=g, f16=True)
    x, wq, sc, zp, b = dev(c["x"]), dev(c["wq"]), dev(c["scale"]), dev(c["zp"]), dev(bias)
    y = torch.empty((M, N), dtype=torch.uint16, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    L.check(L.lib().b200q_a16_w4_dev_dt(ptr(x), ptr(wq), ptr(sc), ptr(zp), ptr(b), ptr(y), M, N, K, g, L.DT_F16, ptr(st), None))
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    check_f16(y.cpu().numpy(), ref)
    # handle API
    h = C.c_void_p()
    L.check(L.lib().b200q_a16_dev_create_dt(ptr(wq), ptr(sc), ptr(zp), ptr(b), N, K, g, L.DT_F16, C.byref(h)))
    y2 = torch.empty_like(y)
    L.check(L.lib().b200q_a16_dev_run(h, ptr(x), ptr(y2), M, None))
    L.check(L.lib().b200q_a16_dev_status(h, None))
    L.lib().b200q_a16_dev_destroy(C.byref(h))
    assert torch.equal(y, y2)


def test_w4f16_operator_face_and_exact_rounding():
    """Through host float buffers; and on a case whose fp32 sums are exact (integer activations, power-of-two scales) the
    f16 output must be the reference's F16() rounding bit for bit."""
    M, K, N, g = 3, 256, 64, 64
    rng = np.random.default_rng(5)
    q = rng.integers(0, 16, size=(N, K), dtype=np.uint8)
    wq = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
    scale = np.full(N * K // g, 2.0 ** -9, np.float32) * rng.choice([1.0, 2.0, 4.0], N * K // g).astype(np.float32)
    zp = rng.integers(0, 16, size=N * K // g, dtype=np.uint8)
    x = rng.integers(-3, 4, size=(M, K)).astype(np.float32)         # every product and partial sum is exact in fp32
    ref = oracle.a16matmul_w4(x.astype(np.float16).view(np.uint16), wq, scale.astype(np.float16).view(np.uint16), zp, group=g, f16=True)
    op = A16MatMulOp(M=M, K=K, N=N, q_group_size=g, out_dtype=L.DT_F16)
    out = np.zeros((M, N), np.float32)
    p = InferenceParameter(inputs=[x, wq.astype(np.float32), scale, zp.astype(np.float32), None], outputs=[out])
    op.inference(p)
    assert np.array_equal(out.astype(np.float16).view(np.uint16), ref)
    assert np.array_equal(out.astype(np.float16).astype(np.float32), out), "output is f16-representable"


# ------------------------------------------------------------------ warpgroup kernel (route 4)
@pytest.mark.parametrize("case", [dict(M=4, K=64, N=128, g=64), dict(M=16, K=256, N=128, g=64), dict(M=2, K=1024, N=300, g=128),
                                  dict(M=9, K=256, N=128, g=32), dict(M=17, K=4096, N=256, g=64), dict(M=32, K=2048, N=512, g=256),
                                  dict(M=1, K=4096, N=11008, g=64), dict(M=16, K=4096, N=11008, g=64),
                                  dict(M=32, K=4096, N=11008, g=64), dict(M=3, K=11008, N=4096, g=64),
                                  dict(M=30, K=11008, N=130, g=128), dict(M=4, K=192, N=100, g=64),
                                  dict(M=12, K=1024, N=700, g=512)])
@pytest.mark.parametrize("f16", [False, True])
def test_warpgroup_kernel(route, case, f16):
    """b200q_a16_set_route(4): up to 32 tokens, weights by TMA, each lane converts its own output channel, the exact
    hi + lo split of (q - zp) * scale in two MMAs, K slices summed in a workspace that every launch leaves zeroed - so
    the second call must give the first one's bits as far as the (unordered) float additions allow: the bound again."""
    route(4)
    M, K, N, g = case["M"], case["K"], case["N"], case["g"]
    c = synth.a16_w4(seed=17, M=M, K=K, N=N, group=g, f16=f16)
    bias = np.random.default_rng(4).standard_normal(N).astype(np.float32)
    ref = oracle.a16matmul_w4(c["x"], c["wq"], c["scale"], c["zp"], bias, group=g, f16=f16)
    x, wq, sc, zp, b = dev(c["x"]), dev(c["wq"]), dev(c["scale"]), dev(c["zp"]), dev(bias)
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(2):
        y = torch.zeros((M, N), dtype=torch.uint16, device="cuda")
        L.check(L.lib().b200q_a16_w4_dev_dt(ptr(x), ptr(wq), ptr(sc), ptr(zp), ptr(b), ptr(y), M, N, K, g,
                                            L.DT_F16 if f16 else L.DT_BF16, ptr(st), None))
        torch.cuda.synchronize()
        assert int(st.item()) == 0
        (check_f16 if f16 else check)(y.cpu().numpy(), ref)


def test_warpgroup_kernel_refuses_more_than_32_tokens(route):
    route(4)
    c = synth.a16_w4(seed=1, M=33, K=256, N=128, group=64)
    x, wq, sc, zp = dev(c["x"]), dev(c["wq"]), dev(c["scale"]), dev(c["zp"])
    y = torch.zeros((33, 128), dtype=torch.uint16, device="cuda")
    rc = L.lib().b200q_a16_w4_dev(ptr(x), ptr(wq), ptr(sc), ptr(zp), None, ptr(y), 33, 128, 256, 64, None, None)
    assert rc == L.ERR_UNSUPPORTED


# ------------------------------------------------------------------ per-channel w4 and w8bf16 (operator face)
@pytest.mark.parametrize("M", [1, 4, 20, 70])
def test_per_channel_w4(M):
    """q_group_size = 0: one scale and zero point per output channel (A16MatMul.cpp:176-187) = a group of K."""
    K, N = 1024, 200
    c = synth.a16_w4(seed=21, M=M, K=K, N=N, group=K)
    ref = oracle.a16matmul_w4(c["x"], c["wq"], c["scale"], c["zp"], group=K)
    f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32)  # noqa: E731
    op = A16MatMulOp(M=M, K=K, N=N, q_group_size=0)
    out = np.zeros((M, N), np.float32)
    p = InferenceParameter(inputs=[oracle.bf16_bits_to_f32(c["x"]), f32(c["wq"]), oracle.bf16_bits_to_f32(c["scale"]), f32(c["zp"]), None],
                           outputs=[out])
    op.inference(p)
    if M >= 64:
        check_rounded_weight(oracle.f32_to_bf16_bits_fast(out), oracle.bf16_bits_to_f32(ref))   # the handle's bf16-copy route
    else:
        check(oracle.f32_to_bf16_bits_fast(out), ref)


@pytest.mark.parametrize("case", [dict(M=1, K=512, N=96, g=64, signed=False), dict(M=5, K=4096, N=300, g=128, signed=True),
                                  dict(M=130, K=1024, N=257, g=0, signed=False), dict(M=33, K=264, N=40, g=8, signed=True)])
def test_w8bf16_operator_face(case):
    """weight_bits = 8 (A16MatMul.cpp:209-246): the reference rounds the dequantised weight to bf16 and multiplies in fp32;
    here that bf16 matrix is built once per weight version and every M runs the bf16 tensor-core GEMM.  Weights signed or
    unsigned, float-stored like every interpreter buffer.  The plain bound, with a bias."""
    M, K, N, g = case["M"], case["K"], case["N"], case["g"]
    group = g if g else K
    rng = np.random.default_rng(31)
    w = (rng.integers(-128, 128, size=(N, K)) if case["signed"] else rng.integers(0, 256, size=(N, K))).astype(np.float32)
    zp = (rng.integers(-8, 8, size=N * K // group) if case["signed"] else rng.integers(120, 136, size=N * K // group)).astype(np.float32)
    scale = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits_fast((rng.random(N * K // group) * 0.01 + 0.002).astype(np.float32)))
    x = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits_fast(rng.standard_normal((M, K)).astype(np.float32)))
    bias = rng.standard_normal(N).astype(np.float32)
    ref = oracle.a16matmul_w8(oracle.f32_to_bf16_bits_fast(x), w, oracle.f32_to_bf16_bits_fast(scale), zp, bias, group=group)
    op = A16MatMulOp(M=M, K=K, N=N, q_group_size=g, weight_bits=8, with_bias=True)
    out = np.zeros((M, N), np.float32)
    p = InferenceParameter(inputs=[x, w, scale, zp, bias], outputs=[out])
    op.init(p)
    op.inference(p)
    op.inference(p)
    op.deinit(p)
    check(oracle.f32_to_bf16_bits_fast(out), ref)


@pytest.mark.parametrize("case", [dict(M=1, K=512, N=96, g=64, signed=False), dict(M=70, K=1024, N=257, g=0, signed=True)])
def test_w8f16_operator_face(case):
    """weight_bits = 8 in an F16 mode (A16MatMul.cpp:226-246): the dequantised weight and the output are rounded with F16();
    kind::f16 on IEEE half operands."""
    M, K, N, g = case["M"], case["K"], case["N"], case["g"]
    group = g if g else K
    rng = np.random.default_rng(32)
    h16 = lambda a: np.asarray(a, dtype=np.float32).astype(np.float16)  # noqa: E731
    w = (rng.integers(-128, 128, size=(N, K)) if case["signed"] else rng.integers(0, 256, size=(N, K))).astype(np.float32)
    zp = (rng.integers(-8, 8, size=N * K // group) if case["signed"] else rng.integers(120, 136, size=N * K // group)).astype(np.float32)
    scale = h16(rng.random(N * K // group) * 0.01 + 0.002)
    x = h16(rng.standard_normal((M, K)))
    bias = rng.standard_normal(N).astype(np.float32)
    ref = oracle.a16matmul_w8(x.view(np.uint16), w, scale.view(np.uint16), zp, bias, group=group, f16=True)
    op = A16MatMulOp(M=M, K=K, N=N, q_group_size=g, weight_bits=8, with_bias=True, out_dtype=L.DT_F16)
    out = np.zeros((M, N), np.float32)
    p = InferenceParameter(inputs=[x.astype(np.float32), w, scale.astype(np.float32), zp, bias], outputs=[out])
    op.init(p)
    op.inference(p)
    op.deinit(p)
    assert np.array_equal(out.astype(np.float16).astype(np.float32), out)          # the outputs are f16 values
    check_f16(out.astype(np.float16).view(np.uint16), ref)


# ------------------------------------------------------------------ output rounding, bit for bit
@pytest.mark.parametrize("M", [1, 4, 20])
def test_bf16_output_rounding_matches_reference_on_edge_values(M):
    """BF16() (lib/Support/Float16.cpp:603-645 with the denormal rule of :550-601, restated by the oracle and pinned there
    against the reference's own code): every output here is ONE exact product x[m,0] * scale[n] (all other weights equal
    their zero point), chosen around the places where the rule differs from a plain hardware conversion - fp32
    denormals (flushed to zero, or to the smallest normal from fraction 0x7f8000 on), ties, the largest finite value,
    infinity.  One token takes the CUDA-core kernel, four the mma.sync kernel, twenty the tcgen05 kernel."""
    K, g = 64, 64
    bf = lambda v: oracle.f32_to_bf16_bits_fast(np.asarray(v, dtype=np.float32))  # noqa: E731
    scales = np.array([2.0 ** -20, 2.0 ** -27, 1.9921875 * 2.0 ** -28, 1.9921875 * 2.0 ** -27, 1.5 * 2.0 ** -27, 2.0 ** -26, 1.0, 1.0078125,
                       1.0234375, 3.0, 2.0 ** 27, 1.9921875 * 2.0 ** 27, 2.0 ** 28, 0.0, 1.25 * 2.0 ** -30, 1.75 * 2.0 ** -33], np.float32)
    N = scales.size
    xs = np.array([2.0 ** -100, 1.9921875 * 2.0 ** -100, -1.5 * 2.0 ** -99, 1.0078125, -1.0234375, 1.9921875 * 2.0 ** 99, -(2.0 ** 100), 1.4921875 * 2.0 ** -101,
                   1.0, 257.0 / 256.0 * 0 + 1.5, 2.0 ** -96, -(2.0 ** -104), 1.9921875, 0.0, -(2.0 ** 99), 1.0625, 2.0 ** -98, 1.75 * 2.0 ** -100, 1.1171875 * 2.0 ** -99,
                   -1.3359375 * 2.0 ** -100], np.float32)[:M]
    x = np.zeros((M, K), np.float32)
    x[:, 0] = oracle.bf16_bits_to_f32(bf(xs))
    zp = np.full(N, 7, np.uint8)
    q = np.full((N, K), 7, np.uint8)
    q[:, 0] = 8                                            # (q - zp) = 1 at k = 0, 0 elsewhere
    wq = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
    sb = bf(scales)
    with np.errstate(over="ignore"):
        prod = (x[:, :1] * oracle.bf16_bits_to_f32(sb)[None, :]).astype(np.float32)       # exact or IEEE-rounded once, like the kernels' fp32
    want = np.array([[oracle.lib().orc_f32_to_bf16_bits(float(v)) for v in row] for row in prod], np.uint16)
    want[prod == 0] = 0                                    # an exact zero is summed with the +0 of the other 63 terms
    xd, wd, sd, zd = dev(bf(x)), dev(wq), dev(sb), dev(zp)
    y = torch.zeros((M, N), dtype=torch.uint16, device="cuda")
    L.check(L.lib().b200q_a16_w4_dev(ptr(xd), ptr(wd), ptr(sd), ptr(zd), None, ptr(y), M, N, K, g, None, None))
    torch.cuda.synchronize()
    got = y.cpu().numpy()
    assert np.array_equal(got, want), [(m, n, hex(int(got[m, n])), hex(int(want[m, n])), float(prod[m, n])) for m in range(M) for n in range(N) if got[m, n] != want[m, n]][:8]
