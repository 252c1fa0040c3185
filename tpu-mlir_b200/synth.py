"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

The reference ships no datasets or weights for this path, so every workload is generated: uniform int8
activations, clipped-normal int8 weights, int32 biases, per-channel multipliers in [2^30, 2^31) with
right shifts in [8, 20] (the QDM/TFLite requantisation form), packed uint4 weights with bf16 group
scales, and normal(0,1) float images for calibration.
"""
from __future__ import annotations

import numpy as np


def qdm_params(rng, channels, *, through_float=False):
    """Per-channel multiplier in [2^30, 2^31) and right shift in [8, 20].  ``through_float`` rounds the
    multiplier to what survives a float32 operand buffer (24 significant bits), as tpu.RequantIntAxis and a
    fuse_rq tpu.MatMul see it."""
    mult = rng.integers(2**30, 2**31, size=channels, dtype=np.int64)
    if through_float:
        mult = mult.astype(np.float32).astype(np.int64)
        mult = np.minimum(mult, 2**31 - 128)
    rshift = rng.integers(8, 21, size=channels, dtype=np.int64)
    return mult, rshift


def matmul_int8(seed=0, M=512, K=1024, N=1024, *, through_float=False):
    """Config 0: A s8 [M,K], B s8 [K,N] uniform in [-128,127], bias s32 in [-2^16, 2^16], QDM per channel."""
    rng = np.random.default_rng(seed)
    A = rng.integers(-128, 128, size=(M, K), dtype=np.int8)
    B = rng.integers(-128, 128, size=(K, N), dtype=np.int8)
    bias = rng.integers(-2**16, 2**16 + 1, size=N, dtype=np.int32)
    mult, rshift = qdm_params(rng, N, through_float=through_float)
    return dict(A=A, B=B, bias=bias, mult=mult, rshift=rshift)


def conv2d_int8(seed=1, N=32, C=256, H=56, W=56, OC=256, KH=3, KW=3, *, unsigned_input=False):
    """Config 1: x s8 NCHW uniform, w s8 = clip(round(normal(0,32)), -127, 127), bias s32, QDM per channel."""
    rng = np.random.default_rng(seed)
    if unsigned_input:
        x = rng.integers(0, 256, size=(N, C, H, W), dtype=np.uint8)
    else:
        x = rng.integers(-128, 128, size=(N, C, H, W), dtype=np.int8)
    w = np.clip(np.rint(rng.normal(0, 32, size=(OC, C, KH, KW))), -127, 127).astype(np.int8)
    bias = rng.integers(-2**16, 2**16 + 1, size=OC, dtype=np.int32)
    mult, rshift = qdm_params(rng, OC)
    return dict(x=x, w=w, bias=bias, mult=mult, rshift=rshift)


def f32_to_bf16_bits(x):
    """Round-to-nearest-even bf16 bit patterns of finite normal float32 values."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def a16_w4(seed=2, M=1, K=4096, N=11008, group=64, f16=False):
    """Config 2: packed uint4 weights [N, K/2] (even k in the low nibble), bf16 scales and uint8 zero points per
    group of `group` along K, bf16 normal(0,1) activations [M, K].  ``f16=True``: the same values as IEEE half bit
    patterns (w4f16)."""
    rng = np.random.default_rng(seed)
    q = rng.integers(0, 16, size=(N, K), dtype=np.uint8)
    wq = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
    to_bits = (lambda a: a.astype(np.float16).view(np.uint16)) if f16 else f32_to_bf16_bits
    scale = to_bits(rng.uniform(0.001, 0.02, size=N * K // group).astype(np.float32))
    zp = rng.integers(0, 16, size=N * K // group, dtype=np.uint8)
    x = to_bits(rng.standard_normal((M, K)).astype(np.float32))
    return dict(x=x, wq=wq, scale=scale, zp=zp)


def calibration_images(seed=4, count=2048, shape=(3, 224, 224), start=0):
    """Config 4: sample i is drawn from its own stream so any rank can produce its contiguous range."""
    out = np.empty((count,) + tuple(shape), dtype=np.float32)
    for i in range(count):
        out[i] = np.random.default_rng([seed, start + i]).standard_normal(shape, dtype=np.float32)
    return out
