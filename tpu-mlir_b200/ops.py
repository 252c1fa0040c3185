"""Python mirror of the reference's per-op inference interface for the ops on the hot path.

The reference dispatches ``InferenceInterface::{init, inference, deinit}(InferenceParameter&)`` per op
(include/tpu_mlir/Interfaces/InferenceInterface.td:16-58); ``InferenceParameter`` is
``{inputs: float*[], outputs: float*[], handle}`` (InferenceInterface.h:15-19) and every tensor - integer
ones included - is a float32 host buffer.  The classes here keep that shape: attributes live on the op
object (they come from the MLIR op in the reference), operands travel in an ``InferenceParameter`` of
float32 numpy arrays in operand order, and the work happens in libb200q.so on the GPU.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np

from . import _lib as L


@dataclass
class InferenceParameter:
    """InferenceParameter of the reference (InferenceInterface.h:15-19): host float buffers + op handle."""
    inputs: List[Optional[np.ndarray]] = field(default_factory=list)
    outputs: List[Optional[np.ndarray]] = field(default_factory=list)
    handle: Optional[C.c_void_p] = None


def _f32(a):
    if a is None:
        return None
    if a.dtype != np.float32 or not a.flags.c_contiguous:
        raise TypeError("InferenceParameter buffers must be C-contiguous float32 arrays")
    return a


def _i64_array(values):
    v = np.ascontiguousarray(np.atleast_1d(np.asarray(values, dtype=np.int64)))
    return v, v.ctypes.data_as(C.POINTER(C.c_int64))


class MatMulOp:
    """tpu.MatMul with uniform-quantized operands (lib/Dialect/Tpu/Interfaces/Common/MatMul.cpp:387-733).

    Operands: input, right, bias, multi, buffer (TpuOps.td:4592-4616).  Attribute names follow the op:
    ``right_transpose, do_relu, input_zp, right_zp, quant_mode, multipliers, rshifts, fuse_rq, out_scales``.
    """

    def __init__(self, *, batch=1, M, K, N, with_bias=False, do_relu=False, right_transpose=False,
                 left_transpose=False, output_transpose=False, hdim_is_batch=False, right_batched=False,
                 right_is_weight=True, input_zp=0, right_zp=0, input_dtype=L.DT_I8, right_dtype=L.DT_I8,
                 out_dtype=L.DT_I8, quant_mode=L.QM_MULTIPLIER_SHIFT, is_cv18xx=False, fuse_rq=False, out_zp=0,
                 multipliers: Sequence[int] = (), rshifts: Sequence[int] = (), out_scale=0.0, algo=L.ALGO_AUTO, batch_low=1):
        self._mult, mult_p = _i64_array(multipliers if len(np.atleast_1d(multipliers)) else [1])
        self._rs, rs_p = _i64_array(rshifts if len(np.atleast_1d(rshifts)) else [0])
        n_quant = 0 if (len(np.atleast_1d(multipliers)) == 0 and len(np.atleast_1d(rshifts)) == 0) else \
            max(self._mult.size, self._rs.size)
        if n_quant and self._mult.size != self._rs.size:
            if self._mult.size == 1:
                self._mult, mult_p = _i64_array(np.full(n_quant, self._mult[0]))
            elif self._rs.size == 1:
                self._rs, rs_p = _i64_array(np.full(n_quant, self._rs[0]))
            else:
                raise ValueError("multipliers and rshifts must have the same length")
        self.desc = L.MatMulDesc(batch=batch, M=M, K=K, N=N, with_bias=int(with_bias), do_relu=int(do_relu),
                                 right_transpose=int(right_transpose), left_transpose=int(left_transpose),
                                 output_transpose=int(output_transpose), hdim_is_batch=int(hdim_is_batch),
                                 right_batched=int(right_batched), right_is_weight=int(right_is_weight),
                                 weight_version=0, input_zp=input_zp, right_zp=right_zp, input_dtype=input_dtype,
                                 right_dtype=right_dtype, out_dtype=out_dtype, quant_mode=quant_mode,
                                 is_cv18xx=int(is_cv18xx), fuse_rq=int(fuse_rq), out_zp=out_zp, n_quant=n_quant,
                                 multipliers=mult_p, rshifts=rs_p, out_scale=float(out_scale), algo=algo, batch_low=int(batch_low))

    def invalidate_weights(self):
        """Call after rewriting the weight/bias buffers in place (the interpreter does that in setTensor)."""
        self.desc.weight_version += 1

    def init(self, p: InferenceParameter):
        h = C.c_void_p()
        L.check(L.lib().b200q_matmul_init(C.byref(self.desc), C.byref(h)))
        p.handle = h

    def inference(self, p: InferenceParameter):
        h = p.handle if p.handle is not None else C.c_void_p()
        ins = [_f32(a) for a in p.inputs]
        outs = [_f32(a) for a in p.outputs]
        rc = L.lib().b200q_matmul_inference(C.byref(self.desc), L.float_pp(ins), len(ins), L.float_pp(outs),
                                            len(outs), C.byref(h))
        L.check(rc)

    def deinit(self, p: InferenceParameter):
        if p.handle is not None:
            L.lib().b200q_matmul_deinit(C.byref(p.handle))
            p.handle = None


class Conv2DOp:
    """tpu.Conv2D with a uniform-quantized output (lib/Dialect/Tpu/Interfaces/Common/Conv2D.cpp:19-344).

    Operands: input, filter, bias (TpuOps.td:1557-1560).  ``kernel_shape, strides, dilations, pads
    (top, left, bottom, right as in the op's `pads` attribute), group, do_relu, quant_mode, multiplier,
    rshift`` follow the op's attribute names.
    """

    def __init__(self, *, input_shape, oc, kernel_shape, strides=(1, 1), dilations=(1, 1), pads=(0, 0, 0, 0),
                 group=1, pad_value=0, with_bias=True, do_relu=False, input_dtype=L.DT_I8, out_dtype=L.DT_I8,
                 quant_mode=L.QM_MULTIPLIER_SHIFT, is_cv18xx=False, out_zp=0, multiplier: Sequence[int] = (1,),
                 rshift: Sequence[int] = (0,), algo=L.ALGO_AUTO):
        n, ic, ih, iw = input_shape
        pht, pwl, phb, pwr = pads   # the op stores pads as [top, left, bottom, right] (Conv2D.cpp:44-48)
        self._mult, mult_p = _i64_array(multiplier)
        self._rs, rs_p = _i64_array(rshift)
        if self._mult.size != self._rs.size:
            if self._mult.size == 1:
                self._mult, mult_p = _i64_array(np.full(self._rs.size, self._mult[0]))
            else:
                raise ValueError("multiplier and rshift must have the same length")
        self.desc = L.Conv2DDesc(n=n, ic=ic, ih=ih, iw=iw, oc=oc, kh=kernel_shape[0], kw=kernel_shape[1],
                                 sh=strides[0], sw=strides[1], dh=dilations[0], dw=dilations[1], pht=pht, phb=phb,
                                 pwl=pwl, pwr=pwr, groups=group, pad_value=pad_value, with_bias=int(with_bias),
                                 do_relu=int(do_relu), input_dtype=input_dtype, out_dtype=out_dtype,
                                 quant_mode=quant_mode, is_cv18xx=int(is_cv18xx), out_zp=out_zp,
                                 n_quant=self._rs.size, multipliers=mult_p, rshifts=rs_p, weight_version=0,
                                 algo=algo)
        self.desc._arrays = (self._mult, self._rs)  # the descriptor points into these: they live as long as it does
        self.out_shape = (n, oc,
                          (ih + pht + phb - dilations[0] * (kernel_shape[0] - 1) - 1) // strides[0] + 1,
                          (iw + pwl + pwr - dilations[1] * (kernel_shape[1] - 1) - 1) // strides[1] + 1)

    def invalidate_weights(self):
        """Call after rewriting the filter / bias buffers in place (the interpreter does that in setTensor and
        fake_quant_weight): the next inference uploads and repacks them again."""
        self.desc.weight_version += 1

    def init(self, p: InferenceParameter):
        ins = [_f32(a) for a in p.inputs]
        h = C.c_void_p()
        L.check(L.lib().b200q_conv2d_init(C.byref(self.desc), L.float_pp(ins), len(ins), C.byref(h)))
        p.handle = h

    def inference(self, p: InferenceParameter):
        if p.handle is None:
            raise L.B200QError(L.ERR_INVALID, "Conv2D inference without init (the reference fails the same way)")
        ins = [_f32(a) for a in p.inputs]
        outs = [_f32(a) for a in p.outputs]
        L.check(L.lib().b200q_conv2d_inference(C.byref(self.desc), L.float_pp(ins), len(ins), L.float_pp(outs),
                                               len(outs), C.byref(p.handle)))

    def deinit(self, p: InferenceParameter):
        if p.handle is not None:
            L.lib().b200q_conv2d_deinit(C.byref(p.handle))
            p.handle = None


class TopConvOp:
    """top.Conv in fp32 (lib/Dialect/Top/Interfaces/Conv.cpp:19-231): operands input, filter (OIHW), bias; attributes
    ``kernel_shape, strides, dilations, pads (top, left, bottom, right), group, do_relu, relu_limit``.  The reference
    keeps a oneDNN primitive in ``p.handle``; this operator face is stateless (init / deinit only mark the handle)."""

    def __init__(self, *, input_shape, oc, kernel_shape, strides=(1, 1), dilations=(1, 1), pads=(0, 0, 0, 0), group=1,
                 with_bias=True, do_relu=False, relu_limit=-1.0):
        n, ic, ih, iw = input_shape
        pht, pwl, phb, pwr = pads
        self.desc = L.TopConvDesc(n=n, ic=ic, ih=ih, iw=iw, oc=oc, kh=kernel_shape[0], kw=kernel_shape[1], sh=strides[0],
                                  sw=strides[1], dh=dilations[0], dw=dilations[1], pht=pht, phb=phb, pwl=pwl, pwr=pwr,
                                  groups=group, with_bias=int(with_bias), do_relu=int(do_relu), relu_limit=float(relu_limit))
        self.out_shape = (n, oc, (ih + pht + phb - dilations[0] * (kernel_shape[0] - 1) - 1) // strides[0] + 1,
                          (iw + pwl + pwr - dilations[1] * (kernel_shape[1] - 1) - 1) // strides[1] + 1)

    def init(self, p: InferenceParameter):
        p.handle = True

    def inference(self, p: InferenceParameter):
        if p.handle is None:
            raise L.B200QError(L.ERR_INVALID, "Conv inference without init (the reference fails the same way)")
        ins = [_f32(a) for a in p.inputs]
        outs = [_f32(a) for a in p.outputs]
        L.check(L.lib().b200q_top_conv2d_inference(C.byref(self.desc), L.float_pp(ins), len(ins), L.float_pp(outs), len(outs)))

    def deinit(self, p: InferenceParameter):
        p.handle = None


class A16MatMulOp:
    """tpu.A16MatMul, static 4-bit weights (lib/Dialect/Tpu/Interfaces/Common/A16MatMul.cpp:16-249).

    Operands: input, weight, scale, zp, bias (TpuOps.td:495-500).  Attributes: ``weight_bits, q_group_size,
    w_transpose``.  All buffers are float32 host arrays: activations and scales hold bf16-representable
    values, weight holds the packed bytes [N, K/2] as floats.
    """

    def __init__(self, *, M, K, N, q_group_size=64, weight_bits=4, w_transpose=True, with_bias=False,
                 out_dtype=L.DT_BF16):
        self.desc = L.A16MatMulDesc(M=M, K=K, N=N, weight_bits=weight_bits, q_group_size=q_group_size,
                                    w_transpose=int(w_transpose), with_bias=int(with_bias), out_dtype=out_dtype,
                                    weight_version=0)

    def invalidate_weights(self):
        self.desc.weight_version += 1

    def init(self, p: InferenceParameter):
        h = C.c_void_p()
        L.check(L.lib().b200q_a16matmul_init(C.byref(self.desc), C.byref(h)))
        p.handle = h

    def inference(self, p: InferenceParameter):
        h = p.handle if p.handle is not None else C.c_void_p()
        ins = [_f32(a) for a in p.inputs]
        outs = [_f32(a) for a in p.outputs]
        L.check(L.lib().b200q_a16matmul_inference(C.byref(self.desc), L.float_pp(ins), len(ins), L.float_pp(outs),
                                                  len(outs), C.byref(h)))

    def deinit(self, p: InferenceParameter):
        if p.handle is not None:
            L.lib().b200q_a16matmul_deinit(C.byref(p.handle))
            p.handle = None
