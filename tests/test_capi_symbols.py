"""CPU checks of the C-ABI boundary: the library builds, loads, and exports every function include/b200q.h
declares, and the ctypes signature table names exactly that set.  No compute call is made here."""
import ctypes as C
import os
import re

import pytest

import tpu_mlir_b200._lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "b200q.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b((?:b200q_|kl_)\w+)\s*\(", text)
    return sorted(set(names))


@pytest.fixture(scope="module")
def built():
    return L.build()


def test_header_declares_functions():
    names = declared_functions()
    assert "b200q_conv2d_inference" in names and "b200q_gemm_i8_dev" in names


def test_library_exports_every_declared_symbol(built):
    lib = C.CDLL(built)
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in include/b200q.h but not exported"


def test_signature_table_matches_header(built):
    assert sorted(L.SIGNATURES) == declared_functions()


def test_version_and_error_strings(built):
    lib = L.lib()
    assert lib.b200q_version().startswith(b"b200q")
    assert isinstance(lib.b200q_last_error(), bytes)
    assert lib.b200q_device_count() >= 0


def test_invalid_descriptor_is_reported_not_aborted(built):
    lib = L.lib()
    d = L.MatMulDesc(batch=1, M=4, K=0, N=4, input_dtype=L.DT_I8, right_dtype=L.DT_I8)
    h = C.c_void_p()
    rc = lib.b200q_matmul_init(C.byref(d), C.byref(h))
    assert rc == L.ERR_INVALID and b"shape" in lib.b200q_last_error()
    d = L.MatMulDesc(batch=1, M=4, K=16, N=4, hdim_is_batch=1, input_dtype=L.DT_I8, right_dtype=L.DT_I8)      # no batched right operand
    assert lib.b200q_matmul_init(C.byref(d), C.byref(h)) == L.ERR_INVALID
    d = L.MatMulDesc(batch=1, M=4, K=16, N=4, hdim_is_batch=1, right_batched=1, is_cv18xx=1, input_dtype=L.DT_I8, right_dtype=L.DT_I8)
    assert lib.b200q_matmul_init(C.byref(d), C.byref(h)) == L.ERR_UNSUPPORTED
    assert lib.b200q_conv2d_inference(None, None, 0, None, 0, C.byref(h)) == L.ERR_INVALID
