"""ctypes binding of libb200q.so (the C ABI declared in include/b200q.h)."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200q.so")

# enums of include/b200q.h
OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_NO_DEVICE, ERR_TIMEOUT, ERR_NOMEM = 0, -1, -2, -3, -4, -5, -6
QM_TFLITE_LSHIFT, QM_TFLITE, QM_MULTIPLIER_SHIFT, QM_ONLY_SHIFT, QM_QDM, QM_ONLY_SCALE = range(6)
(ROUND_HALF_AWAY_FROM_ZERO, ROUND_HALF_UP, ROUND_HALF_DOWN, ROUND_HALF_TO_EVEN, ROUND_HALF_TO_ODD,
 ROUND_HALF_TOWARDS_ZERO, ROUND_TOWARDS_ZERO, ROUND_AWAY_FROM_ZERO, ROUND_UP, ROUND_DOWN) = range(10)
DT_I8, DT_U8, DT_I16, DT_U16, DT_I32, DT_F32, DT_BF16, DT_F16 = range(8)
RQ_NONE, RQ_MULTIPLIER_SHIFT, RQ_QDM, RQ_MULTIPLIER_SHIFT_F32, RQ_ONLY_SHIFT, RQ_ONLY_SCALE = range(6)
RELU_NONE, RELU_BEFORE_REQUANT, RELU_AFTER_REQUANT = range(3)
ALGO_AUTO, ALGO_TENSOR_CORE, ALGO_CUDA_CORE = 0, 1, 2
LAYOUT_NCHW, LAYOUT_NHWC = 0, 1


class B200QError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"b200q error {code}: {message}")
        self.code = code


class Epilogue(C.Structure):
    _fields_ = [("dialect", C.c_int32), ("round_mode", C.c_int32), ("per_channel", C.c_int32),
                ("out_zp", C.c_int32), ("relu", C.c_int32), ("out_dtype", C.c_int32), ("scale", C.c_float),
                ("bias", C.c_void_p), ("multiplier", C.c_void_p), ("shift", C.c_void_p)]


class MatMulDesc(C.Structure):
    _fields_ = [("batch", C.c_int64), ("M", C.c_int64), ("K", C.c_int64), ("N", C.c_int64),
                ("with_bias", C.c_int32), ("do_relu", C.c_int32), ("right_transpose", C.c_int32),
                ("left_transpose", C.c_int32), ("output_transpose", C.c_int32), ("hdim_is_batch", C.c_int32),
                ("right_batched", C.c_int32), ("right_is_weight", C.c_int32), ("weight_version", C.c_int32),
                ("input_zp", C.c_int32), ("right_zp", C.c_int32),
                ("input_dtype", C.c_int32), ("right_dtype", C.c_int32), ("out_dtype", C.c_int32),
                ("quant_mode", C.c_int32), ("is_cv18xx", C.c_int32), ("fuse_rq", C.c_int32), ("out_zp", C.c_int32),
                ("n_quant", C.c_int32), ("multipliers", C.POINTER(C.c_int64)), ("rshifts", C.POINTER(C.c_int64)),
                ("out_scale", C.c_double), ("algo", C.c_int32), ("batch_low", C.c_int64)]


class FusedAdd(C.Structure):
    """b200q_fused_add: the tpu.Add fused into a convolution's epilogue."""
    _fields_ = [("residual", C.c_void_p), ("residual_dtype", C.c_int32), ("conv_multiplier", C.c_int32),
                ("conv_rshift", C.c_int32), ("residual_multiplier", C.c_int32), ("residual_rshift", C.c_int32),
                ("do_relu", C.c_int32), ("out_dtype", C.c_int32)]


class Conv2DDesc(C.Structure):
    _fields_ = [(k, C.c_int64) for k in ("n", "ic", "ih", "iw", "oc", "kh", "kw", "sh", "sw", "dh", "dw", "pht",
                                         "phb", "pwl", "pwr", "groups")] + \
               [("pad_value", C.c_int32), ("with_bias", C.c_int32), ("do_relu", C.c_int32),
                ("input_dtype", C.c_int32), ("out_dtype", C.c_int32), ("quant_mode", C.c_int32),
                ("is_cv18xx", C.c_int32), ("out_zp", C.c_int32), ("n_quant", C.c_int32),
                ("multipliers", C.POINTER(C.c_int64)), ("rshifts", C.POINTER(C.c_int64)),
                ("weight_version", C.c_int32), ("algo", C.c_int32)]


class TopConvDesc(C.Structure):
    _fields_ = [(k, C.c_int64) for k in ("n", "ic", "ih", "iw", "oc", "kh", "kw", "sh", "sw", "dh", "dw", "pht",
                                         "phb", "pwl", "pwr", "groups")] + \
               [("with_bias", C.c_int32), ("do_relu", C.c_int32), ("relu_limit", C.c_float)]


class RemapDesc(C.Structure):
    _fields_ = [(k, C.c_int64 * 6) for k in ("dims", "src_stride", "mul", "div", "mod", "off", "extent", "dst_stride")] + \
               [("dst_offset", C.c_int64)]


(TOP_ADD_CONST, TOP_SUB_CONST, TOP_RSUB_CONST, TOP_MUL_CONST, TOP_MAX_CONST, TOP_MIN_CONST, TOP_MUL, TOP_SUB, TOP_RSUB, TOP_DIV,
 TOP_RDIV, TOP_SIGMOID, TOP_LOG_SIGMOID, TOP_SILU, TOP_GELU, TOP_FLOOR) = range(16)


class RequantDesc(C.Structure):
    _fields_ = [("outer", C.c_int64), ("channels", C.c_int64), ("inner", C.c_int64), ("per_axis", C.c_int32),
                ("quant_mode", C.c_int32), ("round_mode", C.c_int32), ("fuse_rq_axis", C.c_int32), ("in_zp", C.c_int32),
                ("out_dtype", C.c_int32), ("multiplier", C.c_int64), ("rshift", C.c_int64), ("out_zp", C.c_int32), ("quant_words", C.c_int32)]


class A16MatMulDesc(C.Structure):
    _fields_ = [("M", C.c_int64), ("K", C.c_int64), ("N", C.c_int64), ("weight_bits", C.c_int32),
                ("q_group_size", C.c_int32), ("w_transpose", C.c_int32), ("with_bias", C.c_int32),
                ("out_dtype", C.c_int32), ("weight_version", C.c_int32)]


_FLOATPP = C.POINTER(C.POINTER(C.c_float))
_VPP = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); every function include/b200q.h declares
SIGNATURES = {
    "b200q_version": (C.c_char_p, []),
    "b200q_last_error": (C.c_char_p, []),
    "b200q_device_count": (C.c_int, []),
    "b200q_matmul_init": (C.c_int, [C.POINTER(MatMulDesc), _VPP]),
    "b200q_matmul_inference": (C.c_int, [C.POINTER(MatMulDesc), _FLOATPP, C.c_int, _FLOATPP, C.c_int, _VPP]),
    "b200q_matmul_deinit": (None, [_VPP]),
    "b200q_gemm_i8_dev": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64,
                                    C.POINTER(Epilogue), C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "b200q_gemm_i8_zp_dev": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int32,
                                       C.POINTER(Epilogue), C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "b200q_conv2d_init": (C.c_int, [C.POINTER(Conv2DDesc), _FLOATPP, C.c_int, _VPP]),
    "b200q_conv2d_inference": (C.c_int, [C.POINTER(Conv2DDesc), _FLOATPP, C.c_int, _FLOATPP, C.c_int, _VPP]),
    "b200q_conv2d_deinit": (None, [_VPP]),
    "b200q_conv2d_dev_create": (C.c_int, [C.POINTER(Conv2DDesc), C.c_void_p, C.c_void_p, _VPP]),
    "b200q_conv2d_dev_run": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200q_conv2d_dev_run_layout": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]),
    "b200q_conv2d_dev_run_add": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.POINTER(FusedAdd), C.c_void_p]),
    "b200q_conv2d_dev_route": (C.c_int, [C.c_void_p]),
    "b200q_conv2d_dev_status": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200q_conv2d_dev_destroy": (None, [_VPP]),
    "b200q_requant_int_axis_inference": (C.c_int, [C.POINTER(RequantDesc), _FLOATPP, C.c_int, _FLOATPP, C.c_int]),
    "b200q_requant_int_axis_dev": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p,
                                             C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                             C.c_void_p]),
    "b200q_add_i8_dev": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int64] + [C.c_int32] * 6 +
                         [C.c_void_p, C.c_void_p]),
    "b200q_constop_i8_dev": (C.c_int, [C.c_int32, C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_double, C.c_int32, C.c_int32, C.c_int32,
                                       C.c_float, C.c_int32, C.c_void_p, C.c_void_p]),
    "b200q_sub_i8_dev": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int64] + [C.c_int32] * 6 +
                         [C.c_void_p, C.c_void_p]),
    "b200q_pool2d_i8_dev": (C.c_int, [C.c_void_p, C.c_int32, C.c_int64] + [C.c_int32] * 15 + [C.c_void_p, C.c_void_p]),
    "b200q_lut_dev": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "b200q_mulshift_i8_dev": (C.c_int, [C.c_void_p, C.c_int32, C.c_int64] + [C.c_int32] * 5 + [C.c_void_p, C.c_void_p]),
    "b200q_mul_i8_dev": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int64] + [C.c_int32] * 4 +
                         [C.c_void_p, C.c_void_p]),
    "b200q_pool2d_i8_nhwc_dev": (C.c_int, [C.c_void_p, C.c_int32, C.c_int64] + [C.c_int32] * 16 + [C.c_void_p, C.c_void_p]),
    "b200q_cast_f32_to_q8_dev": (C.c_int, [C.c_void_p, C.c_int64, C.c_double, C.c_int32, C.c_int32, C.c_int32,
                                           C.c_void_p, C.c_void_p]),
    "b200q_cast_q8_to_f32_dev": (C.c_int, [C.c_void_p, C.c_int32, C.c_int64, C.c_double, C.c_int32, C.c_void_p,
                                           C.c_void_p]),
    "b200q_a16matmul_init": (C.c_int, [C.POINTER(A16MatMulDesc), _VPP]),
    "b200q_a16matmul_inference": (C.c_int, [C.POINTER(A16MatMulDesc), _FLOATPP, C.c_int, _FLOATPP, C.c_int, _VPP]),
    "b200q_a16matmul_deinit": (None, [_VPP]),
    "b200q_a16_w4_dev": (C.c_int, [C.c_void_p] * 6 + [C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_void_p,
                                   C.c_void_p]),
    "b200q_a16_set_route": (None, [C.c_int32]),
    "b200q_requant_fp_dev": (C.c_int, [C.c_void_p, C.c_int32, C.c_int64, C.c_double, C.c_double, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                       C.c_void_p, C.c_void_p]),
    "b200q_prelu_dev": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "b200q_addconst_i8_dev": (C.c_int, [C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_double, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                        C.c_void_p, C.c_void_p]),
    "b200q_top_conv2d_inference": (C.c_int, [C.POINTER(TopConvDesc), _FLOATPP, C.c_int, _FLOATPP, C.c_int]),
    "b200q_top_conv2d_dev_create": (C.c_int, [C.POINTER(TopConvDesc), C.c_void_p, C.c_void_p, _VPP]),
    "b200q_top_conv2d_dev_run": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "b200q_top_conv2d_dev_output_shape": (None, [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "b200q_top_conv2d_dev_destroy": (None, [_VPP]),
    "b200q_top_matmul_f32_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                           C.c_int32, C.c_float, C.c_void_p]),
    "b200q_top_pool2d_f32_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64] + [C.c_int32] * 13 + [C.c_float, C.c_void_p]),
    "b200q_top_add_f32_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_float, C.c_void_p]),
    "b200q_top_relu_f32_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_float, C.c_void_p]),
    "b200q_interp_f32_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64] + [C.c_int32] * 7 + [C.c_void_p]),
    "b200q_grid_sampler_f32_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p] + [C.c_int32] * 9 + [C.c_void_p]),
    "b200q_arg_f32_dev": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "b200q_top_cast_f32_dev": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "b200q_gather_dev": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "b200q_gather_elements_dev": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.POINTER(C.c_int64),
                                            C.POINTER(C.c_int64), C.c_int32, C.c_void_p]),
    "b200q_active_f32_dev": (C.c_int, [C.c_int32, C.c_void_p, C.c_double, C.c_double, C.c_void_p, C.c_int64, C.c_void_p]),
    "b200q_top_eltwise_f32_dev": (C.c_int, [C.c_int32, C.c_void_p, C.c_void_p, C.c_double, C.c_void_p, C.c_int64, C.c_int32, C.c_float, C.c_void_p]),
    "b200q_top_scale_f32_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int64, C.c_int32, C.c_float, C.c_void_p]),
    "b200q_top_reduce_f32_dev": (C.c_int, [C.c_int32, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int64, C.c_void_p]),
    "b200q_top_softmax_f32_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int64, C.c_int32, C.c_void_p]),
    "b200q_top_layernorm_f32_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_void_p]),
    "b200q_remap_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.POINTER(RemapDesc), C.c_void_p, C.c_void_p]),
    "b200q_top_fake_quant_f32_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_double, C.c_void_p]),
    "b200q_top_distance_f32_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "b200q_a16_w4_dev_dt": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                      C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "b200q_a16_dev_create_dt": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_int32,
                                          C.POINTER(C.c_void_p)]),
    "b200q_debug_set_wait_fault": (None, [C.c_int32, C.c_int64]),
    "b200q_probe_tensor_peak": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_double), C.POINTER(C.c_double), C.c_void_p]),
    "b200q_a16_dev_create": (C.c_int, [C.c_void_p] * 4 + [C.c_int64, C.c_int64, C.c_int32, _VPP]),
    "b200q_a16_dev_run": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "b200q_a16_dev_status": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200q_a16_dev_destroy": (None, [_VPP]),
    "b200q_calib_create": (C.c_int, [_VPP]),
    "b200q_calib_destroy": (None, [_VPP]),
    "b200q_calib_minmax": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "b200q_calib_minmax_noalloc": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "b200q_calib_histogram": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.POINTER(C.c_float),
                                        C.POINTER(C.c_int32), C.c_void_p, C.c_int64, C.c_void_p]),
    "b200q_calib_set_histogram_layout": (None, [C.c_int32]),
    "b200q_calib_find_thresholds": (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(C.c_void_p), C.POINTER(C.c_int64),
                                              C.POINTER(C.c_float), C.c_int64, C.POINTER(C.c_float),
                                              C.POINTER(C.c_float), C.c_void_p]),
    "kl_diversity_hist": (C.c_float, [C.POINTER(C.c_int), C.c_float, C.c_longlong, C.c_longlong]),
    "kl_diversity": (C.c_float, [C.POINTER(C.c_float), C.c_longlong, C.c_longlong]),
    "b200q_conv2d_dev_set_profiling": (C.c_int, [C.c_void_p, C.c_int]),
    "b200q_conv2d_dev_profile": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_double),
                                           C.POINTER(C.c_double)]),
}


def build(force: bool = False) -> str:
    """Compile libb200q.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
    csrc = os.path.join(_HERE, "csrc")
    if force:
        subprocess.run(["make", "-C", csrc, "clean"], check=True, capture_output=True)
    r = subprocess.run(["make", "-C", csrc, "-j8", "all"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building libb200q.so failed:\n" + r.stdout[-4000:] + r.stderr[-4000:])
    return LIB_PATH


_lib = None


def lib():
    """The loaded library.  Raises if it has not been built: there is no fallback implementation."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200QError(ERR_NO_DEVICE, f"{LIB_PATH} is missing: build it with __graft_entry__.build() "
                                            "or `make -C tpu-mlir_b200/csrc`")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc: int):
    if rc != OK:
        raise B200QError(rc, lib().b200q_last_error().decode("utf-8", "replace"))


def float_pp(arrays):
    """HOST float buffers -> float*[] (None -> NULL), the InferenceParameter inputs/outputs vectors."""
    arr = (C.POINTER(C.c_float) * len(arrays))()
    for i, a in enumerate(arrays):
        if a is not None:
            arr[i] = a.ctypes.data_as(C.POINTER(C.c_float))
    arr._buffers = list(arrays)     # the pointer table keeps its buffers alive
    return arr
