"""Regenerates tests/golden/reference_vectors.npz from the reference project's
OWN CPU code (kernels/_common/check.h and kernels/gemm/igemm/sparse_meta_int8.h
compiled in place into oracle/_ref/libbm_ref.so by oracle/Makefile).

Run where the reference checkout is present:
    python tests/golden/make_golden.py
The .npz it writes is committed; the tests that read it run anywhere.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402


def main() -> None:
    oracle.build()
    out = {}
    # LCG fill (check.h:98-106) at the two seeds the dense bench uses (bench.cu:268-269)
    out["fill_seed42"] = oracle.ref_fill_random(96, 42)
    out["fill_seed99"] = oracle.ref_fill_random(96, 99)
    # fp32 reference GEMM (check.h:76-93)
    a = oracle.ref_fill_random(24 * 40, 42).reshape(24, 40)
    b = oracle.ref_fill_random(40 * 16, 99).reshape(40, 16)
    out["sgemm_c"] = oracle.ref_cpu_sgemm(a, b)
    # 2:4 generator + compressor (sparse_meta_int8.h:65-178), seed 42 as bench_sparse.cu:52
    for (M, K) in ((32, 64), (48, 128)):
        dense = oracle.ref_gen_random_sparse_2_4_int8(M, K, 42)
        comp, meta = oracle.ref_compress_2_4_int8(dense)
        out[f"sp_dense_{M}x{K}"] = dense
        out[f"sp_comp_{M}x{K}"] = comp
        out[f"sp_meta_{M}x{K}"] = meta
        # dense right-hand side from our own counter generator (the bench draws it with
        # libc rand() inline in main(), bench_sparse.cu:55-60, which is not in a header)
        N = 24
        bmat = oracle.gen_int8((K, N), 7, oracle.stream_id("golden", f"B{M}x{K}"))
        out[f"sp_b_{M}x{K}"] = bmat
        out[f"sp_c_{M}x{K}"] = oracle.ref_cpu_sparse_gemm_int8(dense, bmat)
    # comparator (check.h:25-58): AND logic — wrong only if abs AND rel both exceed
    ref = np.array([1.0, 10.0, 0.0, 100.0, 1e-9, -5.0], np.float32)
    gpu = np.array([1.4, 10.6, 0.3, 100.4, 0.7, -5.6], np.float32)
    r = oracle.ref_check_fp32(gpu, ref, 0.5, 0.1)
    out["check_gpu"] = gpu
    out["check_ref"] = ref
    out["check_result"] = np.array([r["num_errors"], r["first_error"]], np.int32)
    out["check_max"] = np.array([r["max_abs"], r["max_rel"]], np.float32)
    path = os.path.join(ROOT, "tests", "golden", "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
