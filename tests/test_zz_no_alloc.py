"""The allocation-free min/max entry point against the regular one.

Some hosts of this library may not call cudaMalloc once they are running (their device memory is planned up
front, or an allocation's implicit device synchronisation is not acceptable), so b200q_calib_minmax_noalloc
keeps its scratch in a fixed device array inside the library.  The array is shared by all calls and keeps the
previous call's contents, which is why this test calls twice in a row with different shapes: the second call
must not be disturbed by what the first one left behind.  The file sorts last on purpose, so that a run that
stops at the first failure has already run every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

import tpu_mlir_b200._lib as L

pytestmark = pytest.mark.gpu


def both(x, samples):
    lib = L.lib()
    n = x.numel() // samples
    ctx = C.c_void_p()
    L.check(lib.b200q_calib_create(C.byref(ctx)))
    want = torch.empty((samples, 2), dtype=torch.float32, device="cuda")
    got = torch.full((samples, 2), float("nan"), dtype=torch.float32, device="cuda")
    L.check(lib.b200q_calib_minmax(ctx, C.c_void_p(x.data_ptr()), n, samples, C.c_void_p(want.data_ptr()), None))
    L.check(lib.b200q_calib_minmax_noalloc(C.c_void_p(x.data_ptr()), n, samples, C.c_void_p(got.data_ptr()), None))
    torch.cuda.synchronize()
    lib.b200q_calib_destroy(C.byref(ctx))
    return got.cpu().numpy(), want.cpu().numpy()


def test_noalloc_minmax_matches_regular_entry_point_twice_in_a_row():
    rng = np.random.default_rng(12)
    # first call: few samples, many blocks per sample; second call: many samples, so the partial/ticket use differs
    for shape in [(3, 802816), (700, 4099), (1, 5), (1024, 64)]:
        x = torch.from_numpy((rng.standard_normal(shape) * rng.uniform(0.1, 9)).astype(np.float32)).cuda()
        got, want = both(x, shape[0])
        assert np.array_equal(got, want), shape                      # min / max are exact: no tolerance
        assert np.array_equal(got[:, 0], x.min(dim=1).values.cpu().numpy())
        assert np.array_equal(got[:, 1], x.max(dim=1).values.cpu().numpy())


def test_noalloc_minmax_rejects_more_samples_than_the_fixed_scratch_holds():
    x = torch.zeros((1025, 8), dtype=torch.float32, device="cuda")
    out = torch.empty((1025, 2), dtype=torch.float32, device="cuda")
    rc = L.lib().b200q_calib_minmax_noalloc(C.c_void_p(x.data_ptr()), 8, 1025, C.c_void_p(out.data_ptr()), None)
    assert rc == L.ERR_UNSUPPORTED and b"1024" in L.lib().b200q_last_error()
