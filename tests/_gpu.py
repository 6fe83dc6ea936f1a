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
def forced_bn(bn):
    """Pin the tile width (launcher testing hook) for the duration of the block."""
    old = os.environ.get("BM_FORCE_BN")
    if bn is None:
        os.environ.pop("BM_FORCE_BN", None)
    else:
        os.environ["BM_FORCE_BN"] = str(bn)
    try:
        yield
    finally:
        if old is None:
            os.environ.pop("BM_FORCE_BN", None)
        else:
            os.environ["BM_FORCE_BN"] = old


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


@contextmanager
def env(**kv):
    """Temporarily set environment variables read by the launchers' testing hooks."""
    old = {k: os.environ.get(k) for k in kv}
    for k, v in kv.items():
        if v is None:
            os.environ.pop(k, None)
        else:
            os.environ[k] = str(v)
    try:
        yield
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
