"""CPU checker for the INT8 GEMM hot path — TEST INFRASTRUCTURE ONLY.

numpy-facing wrappers over ``liborc.so`` (the C restatement in
``igemm_oracle.c``) and, where it has been built, ``_ref/libbm_ref.so`` (the
reference project's own headers compiled in place by ``oracle/Makefile``).

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this package.  The shipped library never does: it has no CPU path.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import threading

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORC_PATH = os.path.join(_HERE, "liborc.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libbm_ref.so")

_p = C.c_void_p
_i = C.c_int
_f = C.c_float
_u = C.c_uint
_sz = C.c_size_t
_u64 = C.c_uint64


def reference_root():
    """Checkout of the reference project: $BM_REFERENCE_ROOT, else a directory `reference` beside this
    repository; None when there is none (the prebuilt files under oracle/_ref are then used as they are)."""
    env = os.environ.get("BM_REFERENCE_ROOT")
    if env:
        return env if os.path.isdir(env) else None
    beside = os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return beside if os.path.isdir(os.path.join(beside, "kernels", "gemm", "igemm")) else None


def build(force: bool = False) -> None:
    """Compile the checker (and the in-place reference build when the reference
    checkout is present).  Building the checker is not using it."""
    stale = force or not os.path.exists(_ORC_PATH) or (
        os.path.getmtime(_ORC_PATH) < os.path.getmtime(os.path.join(_HERE, "igemm_oracle.c")))
    if stale:
        subprocess.run(["make", "-C", _HERE, "liborc.so"], check=True, capture_output=True)
    ref_root = reference_root()
    if ref_root is None:
        return
    if os.path.isdir(ref_root) and (force or not os.path.exists(_REF_PATH)):
        subprocess.run(["make", "-C", _HERE, "ref", f"REF_ROOT={ref_root}"], check=True,
                       capture_output=True)
    if os.path.isdir(ref_root) and (force or not os.path.exists(os.path.join(_HERE, "_ref", "bench"))):
        subprocess.run(["make", "-C", _HERE, "ref_bench", f"REF_ROOT={ref_root}"], check=True,
                       capture_output=True)
    cubins = os.path.join(_HERE, "_ref", "cubins")
    have_all = os.path.isdir(cubins) and os.path.exists(os.path.join(cubins, "igemm_online_quant_bf_128x256.sm_86.cubin"))
    if os.path.isdir(ref_root) and (force or not have_all):
        # the reference's own kernels for sm_100a: GPU-side checker and "recompiled reference" baseline
        subprocess.run(["make", "-C", _HERE, "ref_cubins", f"REF_ROOT={ref_root}"], check=True,
                       capture_output=True)


_orc = None
_ref = None


def _sig(fn, restype, *argtypes):
    fn.restype = restype
    fn.argtypes = list(argtypes)
    return fn


def lib():
    global _orc
    if _orc is None:
        build()
        L = C.CDLL(_ORC_PATH)
        _sig(L.orc_fill_random, None, _p, _i, _u)
        _sig(L.orc_compute_scale, _f, _p, _i)
        _sig(L.orc_quantize_symmetric, None, _p, _p, _i, _f)
        _sig(L.orc_gen_per_channel_params, None, _p, _p, _i, _f, _f, _u)
        _sig(L.orc_sgemm, None, _i, _i, _i, _f, _p, _i, _p, _i, _f, _p, _i)
        _sig(L.orc_igemm_rows, None, _p, _p, _p, _i, _i, _i, _i, _i)
        _sig(L.orc_igemm, None, _p, _p, _p, _i, _i, _i)
        _sig(L.orc_igemm_parallel, _i, _p, _p, _p, _i, _i, _i, _i, _i, _i)
        _sig(L.orc_igemm_mnk, None, _p, _p, _p, _i, _i, _i)
        _sig(L.orc_igemm_nt_rows, _i, _p, _p, _p, _i, _i, _i, _i, _i, _i)
        _sig(L.orc_dequant_per_tensor, None, _p, _p, _sz, _f, _f)
        _sig(L.orc_dequant_per_channel, None, _p, _p, _i, _i, _p, _p)
        _sig(L.orc_f32_to_f16, C.c_uint16, _f)
        _sig(L.orc_dequant_w8a8_f16, None, _p, _p, _i, _i, _p, _p)
        _sig(L.orc_check_fp32, _i, _p, _p, _i, _f, _f, _p, _p, _p)
        _sig(L.orc_sparse_meta_count, _sz, _i, _i)
        _sig(L.orc_gen_sparse_2_4_ref, None, _p, _i, _i, _u)
        _sig(L.orc_compress_2_4_ref, None, _p, _i, _i, _p, _p)
        _sig(L.orc_decompress_2_4_ref, None, _p, _p, _i, _i, _p)
        _sig(L.orc_decompress_rows, None, _p, _p, _i, _i, _p)
        _sig(L.orc_meta_ref_to_rows, None, _p, _i, _i, _p)
        _sig(L.orc_prune_2_4_rows, None, _p, _i, _i, _p, _p)
        _sig(L.orc_online_quant_gemm, None, _p, _p, _p, _i, _i, _i, _i)
        _sig(L.orc_h_sparse_meta_count, _sz, _i, _i)
        _sig(L.orc_h_gen_sparse_2_4, None, _p, _i, _i, _u)
        _sig(L.orc_h_compress_2_4, None, _p, _i, _i, _p, _p)
        _sig(L.orc_h_cpu_sparse_gemm, None, _p, _p, _p, _i, _i, _i)
        _sig(L.orc_h_decompress_2_4, None, _p, _p, _i, _i, _p)
        _sig(L.orc_gen_int8_uniform, None, _p, _sz, _u64, _u64)
        _sig(L.orc_gen_f32_uniform, None, _p, _sz, _f, _f, _u64, _u64)
        _sig(L.orc_gen_sparse_rows, None, _p, _p, _i, _i, _u64, _u64)
        _sig(L.orc_transpose_i8, None, _p, _p, _i, _i)
        _sig(L.orc_num_threads, _i)
        _orc = L
    return _orc


def have_ref() -> bool:
    return os.path.exists(_REF_PATH)


def ref():
    """The reference project's own CPU functions (None-safe: raises if absent)."""
    global _ref
    if _ref is None:
        if not have_ref():
            build()
        if not have_ref():
            raise FileNotFoundError("oracle/_ref/libbm_ref.so has not been built")
        L = C.CDLL(_REF_PATH)
        _sig(L.ref_fill_random, None, _p, _i, _u)
        _sig(L.ref_cpu_sgemm, None, _i, _i, _i, _f, _p, _i, _p, _i, _f, _p, _i)
        _sig(L.ref_check_fp32, _i, _p, _p, _i, _f, _f, _p, _p, _p)
        _sig(L.ref_sparse_meta_count_int8, _sz, _i, _i)
        _sig(L.ref_gen_random_sparse_2_4_int8, None, _p, _i, _i, _u)
        _sig(L.ref_compress_2_4_int8, None, _p, _i, _i, _p, _p)
        _sig(L.ref_cpu_sparse_gemm_int8, None, _p, _p, _p, _i, _i, _i)
        _ref = L
    return _ref


_ref_f16 = None


def ref_f16():
    """The reference's FP16 2:4 host utilities (kernels/gemm/hgemm_sparse/sparse_meta.h), compiled in place."""
    global _ref_f16
    if _ref_f16 is None:
        path = os.path.join(_HERE, "_ref", "libbm_ref_f16.so")
        if not os.path.exists(path):
            build(force=True)
        if not os.path.exists(path):
            raise FileNotFoundError("oracle/_ref/libbm_ref_f16.so has not been built")
        L = C.CDLL(path)
        _sig(L.ref_h_sparse_meta_count, _sz, _i, _i)
        _sig(L.ref_h_gen_sparse_2_4, None, _p, _i, _i, _u)
        _sig(L.ref_h_compress_2_4, None, _p, _i, _i, _p, _p)
        _sig(L.ref_h_cpu_sparse_gemm, None, _p, _p, _p, _i, _i, _i)
        _ref_f16 = L
    return _ref_f16


def have_ref_f16() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "libbm_ref_f16.so"))


def _ptr(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return a.ctypes.data_as(_p)


# --------------------------------------------------------------------------
# restated reference functions
# --------------------------------------------------------------------------
def fill_random(n: int, seed: int = 42) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().orc_fill_random(_ptr(out), n, seed)
    return out


def compute_scale(x: np.ndarray) -> float:
    x = np.ascontiguousarray(x, np.float32)
    return float(lib().orc_compute_scale(_ptr(x), x.size))


def quantize_symmetric(x: np.ndarray, scale: float) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.int8)
    lib().orc_quantize_symmetric(_ptr(x), _ptr(out), x.size, scale)
    return out


def gen_per_channel_params(N: int, scale_a: float, scale_b: float, seed: int = 123):
    scale = np.empty(N, np.float32)
    zp = np.empty(N, np.int32)
    lib().orc_gen_per_channel_params(_ptr(scale), _ptr(zp), N, scale_a, scale_b, seed)
    return scale, zp


def sgemm(A: np.ndarray, B: np.ndarray) -> np.ndarray:
    M, K = A.shape
    N = B.shape[1]
    A = np.ascontiguousarray(A, np.float32)
    B = np.ascontiguousarray(B, np.float32)
    out = np.zeros((M, N), np.float32)
    lib().orc_sgemm(M, N, K, 1.0, _ptr(A), K, _ptr(B), N, 0.0, _ptr(out), N)
    return out


def igemm(A: np.ndarray, B: np.ndarray, threads: int = 1, rows: tuple[int, int] | None = None) -> np.ndarray:
    """int32 C = A[M,K] @ B[K,N]; `rows` limits the computed row range (other rows stay 0)."""
    M, K = A.shape
    N = B.shape[1]
    A = np.ascontiguousarray(A, np.int8)
    B = np.ascontiguousarray(B, np.int8)
    out = np.zeros((M, N), np.int32)
    r0, r1 = rows if rows is not None else (0, M)
    if threads == 1:
        lib().orc_igemm_rows(_ptr(A), _ptr(B), _ptr(out), M, N, K, r0, r1)
    else:
        lib().orc_igemm_parallel(_ptr(A), _ptr(B), _ptr(out), M, N, K, r0, r1, threads)
    return out


def igemm_mnk(A: np.ndarray, B: np.ndarray) -> np.ndarray:
    M, K = A.shape
    N = B.shape[1]
    A = np.ascontiguousarray(A, np.int8)
    B = np.ascontiguousarray(B, np.int8)
    out = np.zeros((M, N), np.int32)
    lib().orc_igemm_mnk(_ptr(A), _ptr(B), _ptr(out), M, N, K)
    return out


def igemm_nt(A: np.ndarray, W: np.ndarray, threads: int = 0, rows: tuple[int, int] | None = None) -> np.ndarray:
    """int32 C = A[M,K] @ W[N,K]^T (weights K-major)."""
    M, K = A.shape
    N = W.shape[0]
    A = np.ascontiguousarray(A, np.int8)
    W = np.ascontiguousarray(W, np.int8)
    out = np.zeros((M, N), np.int32)
    r0, r1 = rows if rows is not None else (0, M)
    lib().orc_igemm_nt_rows(_ptr(A), _ptr(W), _ptr(out), M, N, K, r0, r1, threads)
    return out


def dequant_per_tensor(acc: np.ndarray, scale_a: float, scale_b: float) -> np.ndarray:
    acc = np.ascontiguousarray(acc, np.int32)
    out = np.empty(acc.shape, np.float32)
    lib().orc_dequant_per_tensor(_ptr(acc), _ptr(out), acc.size, scale_a, scale_b)
    return out


def dequant_per_channel(acc: np.ndarray, scale: np.ndarray, zp: np.ndarray) -> np.ndarray:
    acc = np.ascontiguousarray(acc, np.int32)
    M, N = acc.shape
    scale = np.ascontiguousarray(scale, np.float32)
    zp = np.ascontiguousarray(zp, np.int32)
    out = np.empty((M, N), np.float32)
    lib().orc_dequant_per_channel(_ptr(acc), _ptr(out), M, N, _ptr(scale), _ptr(zp))
    return out


def dequant_w8a8_f16(acc: np.ndarray, sa: np.ndarray, sw: np.ndarray) -> np.ndarray:
    """fp16 bits (as float16 array) of half_rn(float(acc) * (sa[m]*sw[n]))."""
    acc = np.ascontiguousarray(acc, np.int32)
    M, N = acc.shape
    sa = np.ascontiguousarray(sa, np.float32)
    sw = np.ascontiguousarray(sw, np.float32)
    out = np.empty((M, N), np.uint16)
    lib().orc_dequant_w8a8_f16(_ptr(acc), _ptr(out), M, N, _ptr(sa), _ptr(sw))
    return out.view(np.float16)


def check_fp32(gpu: np.ndarray, refv: np.ndarray, abs_tol: float = 1e-3, rel_tol: float = 1e-3):
    gpu = np.ascontiguousarray(gpu, np.float32).ravel()
    refv = np.ascontiguousarray(refv, np.float32).ravel()
    ma, mr, fe = _f(), _f(), _i()
    n = lib().orc_check_fp32(_ptr(gpu), _ptr(refv), gpu.size, abs_tol, rel_tol,
                             C.byref(ma), C.byref(mr), C.byref(fe))
    return {"num_errors": n, "max_abs": ma.value, "max_rel": mr.value, "first_error": fe.value}


def sparse_meta_count(M: int, K: int) -> int:
    return int(lib().orc_sparse_meta_count(M, K))


def gen_sparse_2_4_ref(M: int, K: int, seed: int) -> np.ndarray:
    out = np.empty((M, K), np.int8)
    lib().orc_gen_sparse_2_4_ref(_ptr(out), M, K, seed)
    return out


def compress_2_4_ref(A_dense: np.ndarray):
    A_dense = np.ascontiguousarray(A_dense, np.int8)
    M, K = A_dense.shape
    comp = np.empty((M, K // 2), np.int8)
    meta = np.empty(sparse_meta_count(M, K), np.uint32)
    lib().orc_compress_2_4_ref(_ptr(A_dense), M, K, _ptr(comp), _ptr(meta))
    return comp, meta


def decompress_2_4_ref(comp: np.ndarray, meta: np.ndarray, M: int, K: int) -> np.ndarray:
    comp = np.ascontiguousarray(comp, np.int8)
    meta = np.ascontiguousarray(meta, np.uint32)
    out = np.empty((M, K), np.int8)
    lib().orc_decompress_2_4_ref(_ptr(comp), _ptr(meta), M, K, _ptr(out))
    return out


def decompress_rows(comp: np.ndarray, nib: np.ndarray) -> np.ndarray:
    comp = np.ascontiguousarray(comp, np.int8)
    nib = np.ascontiguousarray(nib, np.uint8)
    R, K2 = comp.shape
    out = np.empty((R, 2 * K2), np.int8)
    lib().orc_decompress_rows(_ptr(comp), _ptr(nib), R, 2 * K2, _ptr(out))
    return out


def online_quant_gemm(A_f16: np.ndarray, B_f16: np.ndarray, col_block: int = 128) -> np.ndarray:
    """igemm_online_quant.cu restated: fp16 A[M,K], B[K,N] -> fp32 C[M,N] (first-tile block scales)."""
    A = np.ascontiguousarray(A_f16, np.float16)
    B = np.ascontiguousarray(B_f16, np.float16)
    M, K = A.shape
    N = B.shape[1]
    C = np.empty((M, N), np.float32)
    lib().orc_online_quant_gemm(_ptr(A), _ptr(B), _ptr(C), M, N, K, col_block)
    return C


# --------------------------------------------------------------------------
# FP16 2:4 utilities (kernels/gemm/hgemm_sparse/sparse_meta.h)
# --------------------------------------------------------------------------
def h_sparse_meta_count(M: int, K: int) -> int:
    return int(lib().orc_h_sparse_meta_count(M, K))


def h_gen_sparse_2_4(M: int, K: int, seed: int) -> np.ndarray:
    out = np.empty((M, K), np.float32)
    lib().orc_h_gen_sparse_2_4(_ptr(out), M, K, seed)
    return out


def h_compress_2_4(A_dense: np.ndarray):
    """fp32 [M,K] with 2:4 zeros -> (A_comp fp16 [M,K/2], meta uint32 [(M/16)(K/16)8])."""
    A = np.ascontiguousarray(A_dense, np.float32)
    M, K = A.shape
    comp = np.empty((M, K // 2), np.float16)
    meta = np.empty(h_sparse_meta_count(M, K), np.uint32)
    lib().orc_h_compress_2_4(_ptr(A), M, K, _ptr(comp), _ptr(meta))
    return comp, meta


def h_cpu_sparse_gemm(A_dense: np.ndarray, B: np.ndarray) -> np.ndarray:
    A = np.ascontiguousarray(A_dense, np.float32)
    B = np.ascontiguousarray(B, np.float32)
    M, K = A.shape
    N = B.shape[1]
    out = np.empty((M, N), np.float32)
    lib().orc_h_cpu_sparse_gemm(_ptr(A), _ptr(B), _ptr(out), M, N, K)
    return out


def h_decompress_2_4(comp: np.ndarray, meta: np.ndarray) -> np.ndarray:
    comp = np.ascontiguousarray(comp, np.float16)
    meta = np.ascontiguousarray(meta, np.uint32)
    M, K2 = comp.shape
    out = np.empty((M, 2 * K2), np.float16)
    lib().orc_h_decompress_2_4(_ptr(comp), _ptr(meta), M, 2 * K2, _ptr(out))
    return out


def prune_2_4_rows(W: np.ndarray):
    """Magnitude pruning to 2:4 along K with compression: (comp[R,K/2] int8, nib[R,K/8] uint8)."""
    W = np.ascontiguousarray(W, np.int8)
    R, K = W.shape
    comp = np.empty((R, K // 2), np.int8)
    nib = np.empty((R, K // 8), np.uint8)
    lib().orc_prune_2_4_rows(_ptr(W), R, K, _ptr(comp), _ptr(nib))
    return comp, nib


def meta_ref_to_rows(meta: np.ndarray, M: int, K: int) -> np.ndarray:
    meta = np.ascontiguousarray(meta, np.uint32)
    out = np.empty((M, K // 8), np.uint8)
    lib().orc_meta_ref_to_rows(_ptr(meta), M, K, _ptr(out))
    return out


# --------------------------------------------------------------------------
# seeded generators of the B200 workloads (new code; streams keyed by name)
# --------------------------------------------------------------------------
def stream_id(config: str, tensor: str) -> int:
    """Stable 63-bit stream key for (config, tensor name) — FNV-1a."""
    h = 0xCBF29CE484222325
    for b in f"{config}/{tensor}".encode():
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h >> 1


def gen_int8(shape, seed: int, stream: int) -> np.ndarray:
    out = np.empty(shape, np.int8)
    lib().orc_gen_int8_uniform(_ptr(out), out.size, seed, stream)
    return out


def gen_scales(n: int, seed: int, stream: int, lo: float = 1e-3, hi: float = 2e-2) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().orc_gen_f32_uniform(_ptr(out), n, np.float32(lo), np.float32(hi) - np.float32(lo), seed, stream)
    return out


def gen_sparse_rows(R: int, K: int, seed: int, stream: int):
    comp = np.empty((R, K // 2), np.int8)
    nib = np.zeros((R, K // 8), np.uint8)
    lib().orc_gen_sparse_rows(_ptr(comp), _ptr(nib), R, K, seed, stream)
    return comp, nib


def num_threads() -> int:
    return int(lib().orc_num_threads())


# --------------------------------------------------------------------------
# the reference's own functions (built in place), for pinning and baselines
# --------------------------------------------------------------------------
def ref_fill_random(n: int, seed: int = 42) -> np.ndarray:
    out = np.empty(n, np.float32)
    ref().ref_fill_random(_ptr(out), n, seed)
    return out


def ref_cpu_sgemm(A: np.ndarray, B: np.ndarray) -> np.ndarray:
    M, K = A.shape
    N = B.shape[1]
    A = np.ascontiguousarray(A, np.float32)
    B = np.ascontiguousarray(B, np.float32)
    out = np.zeros((M, N), np.float32)
    ref().ref_cpu_sgemm(M, N, K, 1.0, _ptr(A), K, _ptr(B), N, 0.0, _ptr(out), N)
    return out


def ref_check_fp32(gpu, refv, abs_tol=1e-3, rel_tol=1e-3):
    gpu = np.ascontiguousarray(gpu, np.float32).ravel()
    refv = np.ascontiguousarray(refv, np.float32).ravel()
    ma, mr, fe = _f(), _f(), _i()
    n = ref().ref_check_fp32(_ptr(gpu), _ptr(refv), gpu.size, abs_tol, rel_tol,
                             C.byref(ma), C.byref(mr), C.byref(fe))
    return {"num_errors": n, "max_abs": ma.value, "max_rel": mr.value, "first_error": fe.value}


def ref_gen_random_sparse_2_4_int8(M: int, K: int, seed: int) -> np.ndarray:
    out = np.empty((M, K), np.int8)
    ref().ref_gen_random_sparse_2_4_int8(_ptr(out), M, K, seed)
    return out


def ref_compress_2_4_int8(A_dense: np.ndarray):
    A_dense = np.ascontiguousarray(A_dense, np.int8)
    M, K = A_dense.shape
    comp = np.empty((M, K // 2), np.int8)
    meta = np.empty(int(ref().ref_sparse_meta_count_int8(M, K)), np.uint32)
    ref().ref_compress_2_4_int8(_ptr(A_dense), M, K, _ptr(comp), _ptr(meta))
    return comp, meta


def ref_cpu_sparse_gemm_int8(A: np.ndarray, B: np.ndarray, threads: int = 1) -> np.ndarray:
    """The reference's verification GEMM.  threads > 1 calls the same function
    on contiguous row slabs from several host threads (ctypes drops the GIL)."""
    M, K = A.shape
    N = B.shape[1]
    A = np.ascontiguousarray(A, np.int8)
    B = np.ascontiguousarray(B, np.int8)
    out = np.empty((M, N), np.int32)
    L = ref()
    if threads <= 1 or M < threads:
        L.ref_cpu_sparse_gemm_int8(_ptr(A), _ptr(B), _ptr(out), M, N, K)
        return out
    bounds = [M * t // threads for t in range(threads + 1)]

    def work(t):
        b, e = bounds[t], bounds[t + 1]
        if e > b:
            L.ref_cpu_sparse_gemm_int8(_ptr(A[b:e]), _ptr(B), _ptr(out[b:e]), e - b, N, K)

    ts = [threading.Thread(target=work, args=(t,)) for t in range(threads)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    return out
