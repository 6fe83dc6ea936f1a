"""FP16 2:4 sparse GEMM (kernels/gemm/hgemm_sparse) on tcgen05.mma.sp.kind::f16 against the CPU
restatement of the reference's host utilities and against the reference's own kernel on the GPU."""
import numpy as np
import pytest
import torch

import oracle
from bare_metal_b200 import igemm as ig
from _gpu import RefKernel, T, assert_clean_status, dev, forced_bn

pytestmark = pytest.mark.gpu


def exact_reference(A16, B16):
    """float64 product of the fp16-rounded operands (the products are exact in fp32; only the order of the
    fp32 additions differs between implementations)."""
    return A16.astype(np.float64) @ B16.astype(np.float64)


def sum_bound(A16, B16, K):
    return 2.0 ** -23 * np.sqrt(K) * 4 * (np.abs(A16.astype(np.float64)) @ np.abs(B16.astype(np.float64))) + 1e-30


def run(comp, B16, meta, M, N, K, bn=None, fmt=None):
    C = torch.full((M, N), -5.0, dtype=torch.float32, device=dev())
    with forced_bn(bn):
        if fmt is None:
            ig.hgemm_sparse_tiled(T(comp), T(B16), C, T(meta.view(np.int32)), M, N, K)
        else:
            ig.hgemm_sparse_tiled(T(comp), T(B16), C, T(meta), M, N, K, fmt)
    assert_clean_status()
    return C.cpu().numpy()


@pytest.mark.parametrize("M,N,K,bn", [(128, 128, 128, 128), (256, 256, 256, 128), (16, 16, 16, None), (144, 272, 80, None),
                                      (512, 512, 1040, 256), (384, 640, 2048, 256),
                                      (256, 224, 128, 224), (400, 1008, 1040, 224), (144, 272, 80, 224)])   # 224: CTA pairs
def test_arbitrary_patterns_bench_section_2(M, N, K, bn):
    """bench.cu:163-197 of hgemm_sparse: generator seed 999, compress_2_4_arbitrary, fp32 CPU reference on
    the unrounded data, tolerance 0.1 / 0.1 — plus the tight bound against the exact product of the
    fp16-rounded operands."""
    A = oracle.h_gen_sparse_2_4(M, K, 999)
    comp, meta = oracle.h_compress_2_4(A)
    B = oracle.fill_random(K * N, 137).reshape(K, N)
    B16 = B.astype(np.float16)
    got = run(comp, B16, meta, M, N, K, bn)
    res = oracle.check_fp32(got, oracle.h_cpu_sparse_gemm(A, B), 0.1, 0.1)
    assert res["num_errors"] == 0, res
    A16 = oracle.h_decompress_2_4(comp, meta)
    assert (np.abs(got - exact_reference(A16, B16)) <= sum_bound(A16, B16, K)).all()


def test_fixed_pattern_bench_section_1_and_known_answer():
    """bench.cu:113-160: positions {0,1} everywhere, metadata 0x44444444 (the naive kernel's case);
    tests/hgemm_sparse/test_mma_sp.cu:82-93: all ones x all ones at K = 16 gives 8."""
    M = N = K = 256
    A = oracle.fill_random(M * K, 42).reshape(M, K)
    B = oracle.fill_random(K * N, 137).reshape(K, N)
    comp = np.ascontiguousarray(A.reshape(M, K // 4, 4)[:, :, :2].reshape(M, K // 2)).astype(np.float16)
    C = torch.zeros((M, N), dtype=torch.float32, device=dev())
    ig.hgemm_sparse_naive(T(comp), T(B.astype(np.float16)), C, M, N, K)
    assert_clean_status()
    masked = A.copy().reshape(M, K // 4, 4)
    masked[:, :, 2:] = 0
    res = oracle.check_fp32(C.cpu().numpy(), oracle.h_cpu_sparse_gemm(masked.reshape(M, K), B), 0.1, 0.1)
    assert res["num_errors"] == 0, res
    ones = torch.ones((16, 8), dtype=torch.float16, device=dev())
    C1 = torch.zeros((16, 16), dtype=torch.float32, device=dev())
    ig.hgemm_sparse_naive(ones, torch.ones((16, 16), dtype=torch.float16, device=dev()), C1, 16, 16, 16)
    assert bool((C1 == 8.0).all())


def test_row_format_metadata_and_independent_rows():
    """Per-row metadata (any of the 6 patterns per row and group — more general than the reference's
    shared rows r / r+8) through BM_META_ROWS."""
    M, N, K = 256, 128, 256
    comp8, nib = oracle.gen_sparse_rows(M, K, 3, 1)                     # positions; values replaced below
    rng = np.random.default_rng(0)
    comp = (rng.random((M, K // 2), dtype=np.float32) * 2 - 1).astype(np.float16)
    B16 = (rng.random((K, N), dtype=np.float32) * 2 - 1).astype(np.float16)
    got = run(comp, B16, nib, M, N, K, fmt=ig.BM_META_ROWS)
    A16 = np.zeros((M, K), np.float16)
    for g in range(K // 4):
        n = np.where(g & 1, nib[:, g // 2] >> 4, nib[:, g // 2] & 0xF)
        A16[np.arange(M), 4 * g + (n & 3)] = comp[:, 2 * g]
        A16[np.arange(M), 4 * g + (n >> 2)] = comp[:, 2 * g + 1]
    assert (np.abs(got - exact_reference(A16, B16)) <= sum_bound(A16, B16, K)).all()


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (2048, 2048, 2048)])
def test_against_the_reference_kernel_on_the_same_buffers(M, N, K):
    A = oracle.h_gen_sparse_2_4(M, K, 999)
    comp, meta = oracle.h_compress_2_4(A)
    g = torch.Generator(device="cuda").manual_seed(11)
    B = (torch.rand((K, N), device=dev(), generator=g) * 2 - 1).half()
    ref = torch.zeros((M, N), dtype=torch.float32, device=dev())
    dA, dM = T(comp), T(meta.view(np.int32))
    RefKernel("hgemm_sparse_tiled").launch(((N + 127) // 128, (M + 127) // 128), (512, 1), [dA, B, ref, dM, M, N, K])
    ours = torch.full((M, N), -1.0, dtype=torch.float32, device=dev())
    ig.hgemm_sparse_tiled(dA, B, ours, dM, M, N, K)
    assert_clean_status()
    diff = float((ours - ref).abs().max())
    assert diff <= 2.0 ** -23 * np.sqrt(K) * 8 * float(ref.abs().max()) + 1e-6, diff


def test_rejects_bad_shapes():
    a = torch.zeros((16, 8), dtype=torch.float16, device=dev())
    b = torch.zeros((16, 16), dtype=torch.float16, device=dev())
    c = torch.zeros((16, 16), dtype=torch.float32, device=dev())
    m = torch.zeros(8, dtype=torch.int32, device=dev())
    with pytest.raises(ig.BmError):
        ig.hgemm_sparse_tiled(a, b, c, m, 16, 16, 24)          # K % 16
    with pytest.raises(ig.BmError):
        ig.hgemm_sparse_tiled(a, b, c, m, 16, 24, 16)          # N % 16
    with pytest.raises(ig.BmError):
        ig.hgemm_sparse_tiled(a, b, c, m, 8, 16, 16)           # M % 16 for the reference metadata
