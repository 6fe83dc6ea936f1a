"""FP16-in GEMM with the reference's per-tile int8 quantisation (igemm_online_quant.cu) on the GPU
against the CPU restatement, through the C ABI."""
import numpy as np
import pytest
import torch

import oracle
from bare_metal_b200 import igemm as ig
from _gpu import T, assert_clean_status, dev

pytestmark = pytest.mark.gpu


def fp16_inputs(M, N, K, seed, outliers=True):
    rng = np.random.default_rng(seed)
    A = rng.random((M, K), dtype=np.float32) * 2 - 1
    B = rng.random((K, N), dtype=np.float32) * 2 - 1
    if outliers and K > 32:
        A[:, 32:] *= rng.choice(np.array([1.0, 1.0, 1.9], np.float32), size=(M, K - 32))
        B[32:, :] *= rng.choice(np.array([1.0, 3.0], np.float32), size=(K - 32, N))
    return A.astype(np.float16), B.astype(np.float16)


def run(A, B, col_block=128):
    M, K = A.shape
    N = B.shape[1]
    C = torch.full((M, N), -3.0, dtype=torch.float32, device=dev())
    if col_block == 256:
        ig.igemm_online_quant_bf_128x256(T(A), T(B), C, M, N, K)
    else:
        ig.igemm_online_quant(T(A), T(B), C, M, N, K)
    assert_clean_status()
    return C.cpu().numpy()


def bound(A, B, col_block):
    """fp32 summation rounding between one scaling of the exact int32 sum and the reference's one
    fused multiply-add per 32-wide K tile: (K/32 + 2) half-ulps of the sum of magnitudes."""
    M, K = A.shape
    absdot = np.abs(A.astype(np.float32)) @ np.abs(B.astype(np.float32))
    return (K // 32 + 2) * 2.0 ** -24 * absdot * 1.5 + 1e-30


@pytest.mark.parametrize("M,N,K,col_block", [(128, 128, 64, 128), (256, 384, 160, 128), (200, 272, 144, 128),
                                            (1, 16, 16, 128), (512, 512, 512, 256), (300, 528, 1040, 256)])
def test_online_quant_matches_the_restated_reference(M, N, K, col_block):
    A, B = fp16_inputs(M, N, K, M + N + K)
    got = run(A, B, col_block)
    want = oracle.online_quant_gemm(A, B, col_block)
    assert np.isfinite(got).all()
    assert (np.abs(got - want) <= bound(A, B, col_block)).all(), float(np.abs(got - want).max())


def test_single_k_tile_is_bit_exact():
    """With K <= 32 the reference adds one product to zero: no summation order is left to differ."""
    A, B = fp16_inputs(256, 256, 32, 9, outliers=False)
    assert np.array_equal(run(A, B).view(np.uint32), oracle.online_quant_gemm(A, B).view(np.uint32))


def test_reference_bench_acceptance_against_fp32_sgemm():
    """bench.cu:292-295,540: uniform [-1,1) data (the bench's LCG), fp32 SGEMM of the unquantised
    values, check_fp32 with max_abs 0.5 / max_rel 0.1 (AND logic)."""
    M = N = K = 512
    a32 = oracle.fill_random(M * K, 1).reshape(M, K)
    b32 = oracle.fill_random(K * N, 2).reshape(K, N)
    A, B = a32.astype(np.float16), b32.astype(np.float16)
    got = run(A, B)
    ref = oracle.sgemm(a32, b32)
    res = oracle.check_fp32(got, ref, 0.5, 0.1)
    assert res["num_errors"] == 0, res


def test_zero_first_tile_gives_zero_like_the_reference():
    """max over the first K tile is 0 -> tile_scale 0: the block's outputs are 0 whatever follows."""
    A, B = fp16_inputs(256, 128, 96, 4)
    A[128:, :32] = 0
    got = run(A, B)
    assert (got[128:] == 0).all() and np.abs(got[:128]).max() > 0
    want = oracle.online_quant_gemm(A, B)
    assert (np.abs(got - want) <= bound(A, B, 128)).all()


def test_rejects_a_short_workspace_and_bad_shapes():
    A, B = fp16_inputs(128, 128, 64, 1)
    C = torch.empty((128, 128), dtype=torch.float32, device=dev())
    with pytest.raises(ig.BmError):
        ig.igemm_online_quant(T(A), T(B), C, 128, 128, 64, workspace=torch.empty(1024, dtype=torch.uint8, device=dev()))
    with pytest.raises(ig.BmError):
        ig.igemm_online_quant(T(A), T(B), C, 128, 120, 64)          # N % 16
    with pytest.raises(ig.BmError):
        ig.igemm_online_quant(T(A), T(B), C, 128, 128, 64, col_block=64)
