"""bm_igemm_sparse_f32_noalloc — the sparse GEMM for callers that may not allocate device memory
(fixed-footprint serving loops, processes whose memory pool owns the whole device).

The entry point keeps its re-tiled metadata in a fixed 2 MiB array inside the library, shared by
every call, so the checks here are: same bits as the allocating entry point, on two calls in a row
whose shapes differ (the second call finds the first call's metadata still in the array), the exact
capacity boundary, a clear refusal beyond it, and the entry point's own error channel.  This file sorts last on purpose: a run that stops at the first
failure has already executed every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from bare_metal_b200 import _lib

pytestmark = pytest.mark.gpu


def _inputs(M, N, K, seed):
    dense = oracle.gen_sparse_2_4_ref(M, K, seed)
    comp, meta = oracle.compress_2_4_ref(dense)
    B = oracle.gen_int8((K, N), seed, 77)
    return dense, comp, meta, B


def _run(fn, comp, meta, B, M, N, K, sa, sb, dev):
    T = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    comp_d, meta_d, B_d = T(comp), T(meta.view(np.int32)), T(B)
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev)
    rc = fn(comp_d.data_ptr(), B_d.data_ptr(), out.data_ptr(), meta_d.data_ptr(), M, N, K,
            C.c_float(sa), C.c_float(sb), None)
    assert rc == 0, _lib.load().bm_last_error_string()
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_no_alloc_entry_matches_the_allocating_one_twice_in_a_row():
    L = _lib.load()
    dev = torch.device("cuda:0")
    s = float(np.float32(1.0) / np.float32(127.0))
    # two different shapes back to back: the second starts with the first one's metadata in the array
    for (M, N, K, seed) in ((512, 384, 1024, 42), (272, 144, 544, 7)):
        dense, comp, meta, B = _inputs(M, N, K, seed)
        want = _run(L.bm_igemm_sparse_f32, comp, meta, B, M, N, K, s, s, dev)
        got = _run(L.bm_igemm_sparse_f32_noalloc, comp, meta, B, M, N, K, s, s, dev)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))       # bit-exact, as everywhere for fp32
        # and both agree with the CPU oracle
        ref = oracle.dequant_per_tensor(oracle.igemm(dense, B, threads=0), np.float32(s), np.float32(s))
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    # no launch gave up: the entry point's own status word (read without allocating) is clear
    code = C.c_int(-1)
    assert L.bm_noalloc_last_device_status(C.byref(code)) == 0 and code.value == 0


def test_no_alloc_entry_at_the_edge_of_its_capacity():
    """M = K = 4096 needs exactly the 2 MiB the fixed array holds (32 x 16 blocks of 4 KiB): accepted, the
    last byte of the array is used, same bits as the allocating entry point and as the CPU oracle.  One more
    128-row block (M = 4224) is refused before anything is launched."""
    L = _lib.load()
    dev = torch.device("cuda:0")
    s = float(np.float32(1.0) / np.float32(127.0))
    M, N, K = 4096, 128, 4096
    dense, comp, meta, B = _inputs(M, N, K, 11)
    want = _run(L.bm_igemm_sparse_f32, comp, meta, B, M, N, K, s, s, dev)
    got = _run(L.bm_igemm_sparse_f32_noalloc, comp, meta, B, M, N, K, s, s, dev)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    ref = oracle.dequant_per_tensor(oracle.igemm(dense, B, threads=0), np.float32(s), np.float32(s))
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    dummy = torch.zeros(64, dtype=torch.int8, device=dev)
    p = dummy.data_ptr()
    rc = L.bm_igemm_sparse_f32_noalloc(p, p, p, p, 4224, 128, 4096, C.c_float(1.0), C.c_float(1.0), None)
    assert rc == -6 and b"2 MiB" in L.bm_last_error_string()


def test_no_alloc_status_word_reports_a_wait_that_gave_up():
    """The error channel of the no-alloc launches: a bounded wait that runs out (a barrier nothing signals,
    2 ms limit — no fault, no hang) is recorded in the entry point's own status word; the reader returns it
    once and clears it, bm_last_device_status sees the same word, and the next GEMM is still correct."""
    L = _lib.load()
    dev = torch.device("cuda:0")
    outcome, code = C.c_int(0), C.c_int(-1)
    assert L.bm_noalloc_selftest_bounded_wait(2000, C.byref(outcome)) == 0 and outcome.value == 2
    assert L.bm_noalloc_last_device_status(C.byref(code)) == 0 and code.value == 5
    assert L.bm_noalloc_last_device_status(C.byref(code)) == 0 and code.value == 0       # cleared by the read
    assert L.bm_noalloc_selftest_bounded_wait(2000, C.byref(outcome)) == 0 and outcome.value == 2
    assert L.bm_last_device_status(C.byref(code)) == 0 and code.value == 5               # the general reader folds it in
    assert L.bm_noalloc_last_device_status(C.byref(code)) == 0 and code.value == 0
    s = float(np.float32(1.0) / np.float32(127.0))
    dense, comp, meta, B = _inputs(256, 128, 512, 3)
    got = _run(L.bm_igemm_sparse_f32_noalloc, comp, meta, B, 256, 128, 512, s, s, dev)
    ref = oracle.dequant_per_tensor(oracle.igemm(dense, B, threads=0), np.float32(s), np.float32(s))
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


def test_no_alloc_entry_rejects_what_does_not_fit():
    L = _lib.load()
    dev = torch.device("cuda:0")
    dummy = torch.zeros(64, dtype=torch.int8, device=dev)
    p = dummy.data_ptr()
    # 8192 x 8192 needs 8 MiB of tiled metadata: refused before anything is launched
    rc = L.bm_igemm_sparse_f32_noalloc(p, p, p, p, 8192, 128, 8192, C.c_float(1.0), C.c_float(1.0), None)
    assert rc == -6
    assert b"2 MiB" in L.bm_last_error_string()
    # argument errors are reported before the capacity check
    assert L.bm_igemm_sparse_f32_noalloc(p, p, p, None, 4096, 128, 4096, C.c_float(1.0), C.c_float(1.0), None) == -1
