"""ctypes binding of libbm_igemm.so — the C ABI declared in include/bm_igemm.h.

There is no fallback: if the library is missing and cannot be built, or a launcher rejects
its arguments, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

from . import _build

_p = C.c_void_p
_i = C.c_int
_f = C.c_float
_i64 = C.c_int64
_sz = C.c_size_t

# name -> (restype, argtypes): every symbol include/bm_igemm.h declares
SIGNATURES = {
    "bm_igemm_i8_i32": (_i, [_p, _p, _p, _i, _i, _i, _i64, _i, _p]),
    "bm_igemm_i8_f32": (_i, [_p, _p, _p, _i, _i, _i, _f, _f, _i64, _i, _p]),
    "bm_igemm_i8_f32_perchannel": (_i, [_p, _p, _p, _i, _i, _i, _p, _p, _i64, _i, _p]),
    "bm_w8a8_f16": (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _i64, _i, _p]),
    "bm_w8a8_f16_gather": (_i, [_p, _p, _p, _i, _p, _p, _i, _i, _i, _i64, _i, _p]),
    "bm_quantize_rows_f16": (_i, [_p, _p, _p, _i, _i, _p]),
    "bm_pack_b_kn_to_nk": (_i, [_p, _p, _i, _i, _p]),
    "bm_prune_2_4_i8": (_i, [_p, _p, _p, _i, _i, _p]),
    "bm_online_quant_workspace_bytes": (_sz, [_i, _i, _i]),
    "bm_online_quant_gemm_f32": (_i, [_p, _p, _p, _i, _i, _i, _i, _p, _sz, _p]),
    "bm_sp_meta_tiled_bytes": (_sz, [_i, _i]),
    "bm_sp_pack_meta": (_i, [_p, _i, _p, _i, _i, _p]),
    "bm_igemm_sparse_f32": (_i, [_p, _p, _p, _p, _i, _i, _i, _f, _f, _p]),
    "bm_igemm_sparse_f32_noalloc": (_i, [_p, _p, _p, _p, _i, _i, _i, _f, _f, _p]),
    "bm_hgemm_sparse_f32": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i64, _p]),
    "bm_igemm_sparse_i32": (_i, [_p, _p, _i, _p, _p, _i, _i, _i, _i64, _i, _p]),
    "bm_w8a8_sparse_i32": (_i, [_p, _p, _p, _p, _i, _i, _i, _i64, _p]),
    "bm_w8a8_sparse_f16": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i64, _p]),
    "bm_sp_packed_weight_bytes": (_sz, [_i, _i]),
    "bm_sp_pack_weights": (_i, [_p, _p, _i, _p, _i, _i, _p]),
    "bm_w8a8_sparse_i32_packed": (_i, [_p, _p, _p, _i, _i, _i, _i64, _p]),
    "bm_w8a8_sparse_f16_packed": (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _i64, _p]),
    "bm_last_device_status": (_i, [C.POINTER(_i)]),
    "bm_selftest_bounded_wait": (_i, [C.c_uint, C.POINTER(_i)]),
    "bm_last_error_string": (C.c_char_p, []),
    "bm_shutdown": (None, []),
    "bm_version": (C.c_char_p, []),
}

BM_B_KN, BM_B_NK = 0, 1
BM_META_REF, BM_META_ROWS, BM_META_TILED, BM_META_REF_F16, BM_META_ROWS_F16 = 0, 1, 2, 3, 4

_lib = None


class BmError(RuntimeError):
    pass


def load():
    global _lib
    if _lib is None:
        path = _build.LIB_PATH
        if not os.path.exists(path):
            path = _build.build()
        lib = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)          # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().bm_last_error_string().decode(errors="replace")
        raise BmError(f"{what} failed with status {rc}: {msg}")
