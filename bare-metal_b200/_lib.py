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
    "bm_w8a8_f16_gather": (_i, [_p, _p, _p, _i, _i, _p, _p, _i, _i, _i, _i64, _i, _p]),
    "bm_gather_slab_f16": (_i, [_p, _i, _i, _i, _i, _i64, _p]),
    "bm_peer_barrier": (_i, [_p, _i, _i, _p]),
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
    "bm_noalloc_last_device_status": (_i, [C.POINTER(_i)]),
    "bm_noalloc_selftest_bounded_wait": (_i, [C.c_uint, C.POINTER(_i)]),
    "bm_last_device_status": (_i, [C.POINTER(_i)]),
    "bm_set_option": (_i, [C.c_char_p, _i]),
    "bm_get_option": (_i, [C.c_char_p, C.POINTER(_i)]),
    "bm_tensor_map_cache_stats": (_i, [C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
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


def set_option(name: str, value: int) -> None:
    check(load().bm_set_option(name.encode(), int(value)), f"bm_set_option({name})")


def get_option(name: str) -> int:
    v = _i(0)
    check(load().bm_get_option(name.encode(), C.byref(v)), f"bm_get_option({name})")
    return v.value


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().bm_last_error_string().decode(errors="replace")
        raise BmError(f"{what} failed with status {rc}: {msg}")
