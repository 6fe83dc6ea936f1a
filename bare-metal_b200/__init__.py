"""bare-metal_b200 — B200-native (sm_100a) INT8 GEMM hot path behind the bare-metal kernel ABI.

Contents: csrc/ (hand-written tcgen05 / TMA kernels and the C ABI of include/bm_igemm.h),
_build.py (in-tree nvcc build), _lib.py (ctypes binding), igemm.py (host-side mirror of the
reference kernel interface), nsplit.py (column-sharded linear across the GPUs of one box).
"""
from . import _build, _lib, igemm, nsplit  # noqa: F401
from ._build import build  # noqa: F401

__version__ = "0.1"
