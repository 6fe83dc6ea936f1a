"""No-GPU checks of the drop-in boundary: the library builds, loads, exports every symbol
include/bm_igemm.h declares, and rejects bad arguments before touching the device."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import bare_metal_b200 as bm
from bare_metal_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "bm_igemm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bm_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    path = bm.build()
    assert os.path.exists(path)
    lib = C.CDLL(path)
    names = declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in bm_igemm.h but not exported"
    # the Python binding covers exactly the declared set
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_pure_host_helpers():
    L = _lib.load()
    assert L.bm_version() == b"0.1"
    # tiled metadata: ceil(R/128) * ceil(K/256) blocks of 4 KiB
    assert L.bm_sp_meta_tiled_bytes(4096, 4096) == 32 * 16 * 4096
    assert L.bm_sp_meta_tiled_bytes(130, 288) == 2 * 2 * 4096
    assert L.bm_sp_meta_tiled_bytes(0, 64) == 0


def test_launchers_reject_bad_arguments_without_a_device():
    L = _lib.load()
    buf = np.zeros(4096 + 64, np.uint8)
    base = buf.ctypes.data
    a16 = (base + 15) & ~15
    # NULL operands
    assert L.bm_igemm_i8_i32(None, None, None, 128, 128, 128, 128, _lib.BM_B_KN, None) == -1
    # non-positive shape
    assert L.bm_igemm_i8_i32(a16, a16, a16, 0, 128, 128, 128, _lib.BM_B_KN, None) == -2
    # K not a multiple of 16
    assert L.bm_igemm_i8_i32(a16, a16, a16, 128, 128, 40, 128, _lib.BM_B_KN, None) == -2
    # [K x N] layout needs N % 16 == 0
    assert L.bm_igemm_i8_i32(a16, a16, a16, 128, 100, 64, 100, _lib.BM_B_KN, None) == -2
    # unknown layout tag
    assert L.bm_igemm_i8_i32(a16, a16, a16, 128, 128, 64, 128, 7, None) == -4
    # misaligned operand
    assert L.bm_igemm_i8_i32(a16 + 1, a16, a16, 128, 128, 64, 128, _lib.BM_B_NK, None) == -3
    # pitch smaller than the row
    assert L.bm_igemm_i8_i32(a16, a16, a16, 128, 128, 64, 64, _lib.BM_B_NK, None) == -2
    assert b"pitch" in L.bm_last_error_string()
    # per-channel without parameters, w8a8 without scales
    assert L.bm_igemm_i8_f32_perchannel(a16, a16, a16, 128, 128, 64, None, None, 128, _lib.BM_B_NK, None) == -1
    assert L.bm_w8a8_f16(a16, a16, a16, None, None, 128, 128, 64, 128, _lib.BM_B_NK, None) == -1
    # sparse: K % 32, M % 16 for the reference format
    assert L.bm_igemm_sparse_f32(a16, a16, a16, a16, 128, 128, 48, 1.0, 1.0, None) == -2
    assert L.bm_igemm_sparse_f32(a16, a16, a16, a16, 120, 128, 64, 1.0, 1.0, None) == -2
    assert L.bm_igemm_sparse_f32(a16, a16, a16, None, 128, 128, 64, 1.0, 1.0, None) == -1
    assert L.bm_sp_pack_meta(a16, 9, a16, 128, 64, None) == -4
    assert L.bm_pack_b_kn_to_nk(None, a16, 64, 64, None) == -1


def test_host_mirror_refuses_cpu_tensors():
    import torch
    from bare_metal_b200 import igemm
    a = torch.zeros((128, 64), dtype=torch.int8)
    c = torch.zeros((128, 128), dtype=torch.float32)
    with pytest.raises(igemm.BmError):
        igemm.igemm_wmma(a, a, c, 128, 128, 64, 1.0, 1.0)


def test_launcher_options_are_set_and_read_without_a_device():
    """Options replace per-launch environment reads: known names round-trip, unknown names are refused, the
    defaults are the documented ones, and a variable in the environment seeds its option once, at first use."""
    import subprocess
    import sys
    L = _lib.load()
    for name, default in (("force_bn", 0), ("dense_pair", 1), ("sparse_pair", 1), ("row_balanced", 1),
                          ("tma_store", 1), ("dense_group_m", -1), ("sparse_col_first", -1), ("tail_narrow", 1),
                          ("pdl", 1), ("gather_gbs", 680), ("decode_tile_rows", 0)):
        if ("BM_" + name.upper()) not in os.environ:
            assert _lib.get_option(name) == default, name
    _lib.set_option("force_bn", 128)
    assert _lib.get_option("force_bn") == 128
    _lib.set_option("force_bn", 0)
    v = C.c_int(0)
    assert L.bm_set_option(b"no_such_option", 1) == -4 and L.bm_get_option(b"no_such_option", C.byref(v)) == -4
    assert L.bm_set_option(None, 1) == -1
    code = ("import sys; sys.path.insert(0, %r); from bare_metal_b200 import _lib; "
            "print(_lib.get_option('gather_gbs'), _lib.get_option('force_bn'))" % ROOT)
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120,
                         env=dict(os.environ, BM_GATHER_GBS="555", BM_FORCE_BN="64"))
    assert out.returncode == 0 and out.stdout.split() == ["555", "64"], out.stderr[-1000:]


def test_gather_and_barrier_entry_points_reject_bad_arguments_without_a_device():
    L = _lib.load()
    buf = np.zeros(256, np.uint8)
    a16 = (buf.ctypes.data + 15) & ~15
    ptrs = (C.c_void_p * 2)(a16, a16)
    assert L.bm_w8a8_f16_gather(a16, a16, None, 2, 0, a16, a16, 128, 128, 64, 256, _lib.BM_B_NK, None) == -1
    assert L.bm_w8a8_f16_gather(a16, a16, ptrs, 2, 5, a16, a16, 128, 128, 64, 256, _lib.BM_B_NK, None) == -2
    assert L.bm_gather_slab_f16(None, 2, 0, 8, 16, 32, None) == -1
    assert L.bm_gather_slab_f16(ptrs, 2, 3, 8, 16, 32, None) == -2            # self index outside the list
    assert L.bm_gather_slab_f16(ptrs, 2, 0, 8, 12, 32, None) == -3            # slab width not a multiple of 8
    assert L.bm_gather_slab_f16(ptrs, 2, 0, 8, 64, 32, None) == -2            # pitch smaller than the slab
    assert L.bm_peer_barrier(None, 2, 0, None) == -1
    assert L.bm_peer_barrier(ptrs, 2, 2, None) == -2
    assert L.bm_peer_barrier(ptrs, 9, 0, None) == -1
