"""Helpers for the GPU tests: torch owns device memory, the kernels are reached through the C ABI."""
import ctypes as C

import numpy as np
import torch

import tpu_mlir_b200._lib as L

NP_OF_DT = {L.DT_I8: np.int8, L.DT_U8: np.uint8, L.DT_I16: np.int16, L.DT_U16: np.uint16, L.DT_I32: np.int32}
TORCH_OF_NP = {np.dtype(np.int8): torch.int8, np.dtype(np.uint8): torch.uint8, np.dtype(np.int16): torch.int16,
               np.dtype(np.uint16): torch.uint16, np.dtype(np.int32): torch.int32, np.dtype(np.float32): torch.float32,
               np.dtype(np.int64): torch.int64}


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def dt_of(a):
    return L.DT_U8 if a.dtype == np.uint8 else L.DT_I8


def empty_dev(shape, dt):
    return torch.empty(shape, dtype=TORCH_OF_NP[np.dtype(NP_OF_DT[dt])], device="cuda")


class Guarded:
    """A device buffer of `shape` with 4 KB of canary bytes on both sides: `view` is what the kernel gets, `check()`
    fails if anything outside the view changed (a store past a ragged edge)."""
    PAD = 4096

    def __init__(self, shape, torch_dtype, fill=None):
        n = int(np.prod(shape)) * torch.empty(0, dtype=torch_dtype).element_size()
        self.raw = torch.full((n + 2 * self.PAD,), 0xA5, dtype=torch.uint8, device="cuda")
        self.view = self.raw[self.PAD:self.PAD + n].view(torch_dtype).reshape(shape)
        if fill is not None:
            self.view.fill_(fill)
        self.n = n

    def check(self):
        torch.cuda.synchronize()
        assert bool((self.raw[:self.PAD] == 0xA5).all()), "bytes before the output buffer were overwritten"
        assert bool((self.raw[self.PAD + self.n:] == 0xA5).all()), "bytes after the output buffer were overwritten"


def make_epilogue(*, dialect, round_mode, mult=None, shift=None, bias=None, per_channel=True, out_zp=0,
                  relu=L.RELU_NONE, out_dtype=L.DT_I8, scale=0.0):
    """Returns (Epilogue, keepalive list of device tensors)."""
    keep = []

    def up(v):
        if v is None:
            return None
        t = dev(np.asarray(v, dtype=np.int32))
        keep.append(t)
        return t.data_ptr()

    e = L.Epilogue(dialect=dialect, round_mode=round_mode, per_channel=int(per_channel), out_zp=out_zp, relu=relu,
                   out_dtype=out_dtype, scale=scale, bias=up(bias), multiplier=up(mult), shift=up(shift))
    return e, keep
