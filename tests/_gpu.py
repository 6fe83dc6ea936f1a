"""Helpers for the -m gpu parity tests (device buffers via torch; all compute through the C ABI)."""
import os
from contextlib import contextmanager

import numpy as np
import torch


def dev():
    return torch.device("cuda:0")


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev())


@contextmanager
def options(**kv):
    """Temporarily set launcher options (bm_set_option) for the duration of the block."""
    from bare_metal_b200 import _lib
    old = {k: _lib.get_option(k) for k in kv}
    for k, v in kv.items():
        _lib.set_option(k, v)
    try:
        yield
    finally:
        for k, v in old.items():
            _lib.set_option(k, v)


def forced_bn(bn):
    """Pin the tile width (launcher testing hook) for the duration of the block."""
    return options(force_bn=0 if bn is None else bn)


def ulp_diff_f16(a_bits: np.ndarray, b_bits: np.ndarray) -> int:
    """Largest distance in fp16 units-in-the-last-place between two bit arrays."""
    def key(x):
        x = x.astype(np.int32)
        return np.where(x & 0x8000, -(x & 0x7FFF), x & 0x7FFF)
    return int(np.abs(key(a_bits) - key(b_bits)).max()) if a_bits.size else 0


def assert_clean_status():
    from bare_metal_b200 import igemm
    torch.cuda.synchronize()
    assert igemm.last_device_status() == 0, "a bounded device-side wait gave up"


class RefKernel:
    """One of the reference project's own kernels, compiled unmodified for sm_100a by
    `make -C oracle ref_cubins` into oracle/_ref/cubins/<name>.sm_86.cubin (the file name its benches
    open), loaded and launched through the CUDA driver API with the geometry its bench uses."""

    def __init__(self, name):
        import ctypes as C
        import pytest
        path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "cubins",
                            name + ".sm_86.cubin")
        if not os.path.exists(path):
            pytest.skip("reference kernels have not been compiled (oracle/Makefile target ref_cubins)")
        import torch
        torch.zeros(1, device="cuda")                         # primary context current on this thread
        self.C = C
        self.cu = C.CDLL("libcuda.so.1")
        self.mod, self.fn = C.c_void_p(), C.c_void_p()
        self._ck(self.cu.cuModuleLoad(C.byref(self.mod), path.encode()), "cuModuleLoad")
        self._ck(self.cu.cuModuleGetFunction(C.byref(self.fn), self.mod, name.encode()), "cuModuleGetFunction")

    @staticmethod
    def _ck(rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} failed with CUresult {rc}")

    def launch(self, grid, block, args):
        """args: torch tensors (passed as device pointers), python ints (int) and floats (float)."""
        import torch
        C = self.C
        keep = []
        for a in args:
            if isinstance(a, torch.Tensor):
                keep.append(C.c_void_p(a.data_ptr()))
            elif isinstance(a, float):
                keep.append(C.c_float(a))
            else:
                keep.append(C.c_int(int(a)))
        params = (C.c_void_p * len(keep))(*[C.cast(C.byref(x), C.c_void_p) for x in keep])
        torch.cuda.synchronize()
        self._ck(self.cu.cuLaunchKernel(self.fn, grid[0], grid[1], 1, block[0], block[1], 1, 0, None, params, None),
                 "cuLaunchKernel")
        self._ck(self.cu.cuCtxSynchronize(), "cuCtxSynchronize")
