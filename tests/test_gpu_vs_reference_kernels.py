"""Same device buffers through the reference's OWN kernels (compiled unmodified for sm_100a into
oracle/_ref/cubins, launched with the geometry of its benches) and through this library: the fp32
outputs must be the same bits.  Sizes stay inside the domain the reference benches exercise
(multiples of the kernels' tiles), up to the 4096^3 headline size the CPU checker cannot reach."""
import numpy as np
import pytest
import torch

import oracle
from bare_metal_b200 import igemm as ig
from _gpu import RefKernel, T, assert_clean_status, dev

pytestmark = pytest.mark.gpu


def rand_i8(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randint(-127, 128, shape, dtype=torch.int8, device=dev(), generator=g)


@pytest.mark.parametrize("M,N,K", [(512, 512, 512), (1024, 2048, 1024), (4096, 4096, 4096)])
def test_dense_per_tensor_and_per_channel_equal_the_reference_kernels(M, N, K):
    A, B = rand_i8((M, K), 1), rand_i8((K, N), 2)
    sa, sb = 0.0123, 0.0456
    ref = torch.zeros((M, N), dtype=torch.float32, device=dev())
    grid, block = ((N + 63) // 64, (M + 63) // 64), (64, 2)            # bench.cu:360-361,448-450
    RefKernel("igemm_pipelined_cpasync").launch(grid, block, [A, B, ref, M, N, K, sa, sb])
    ours = torch.full((M, N), -1.0, dtype=torch.float32, device=dev())
    ig.igemm_pipelined_cpasync(A, B, ours, M, N, K, sa, sb)
    assert_clean_status()
    assert torch.equal(ours.view(torch.int32), ref.view(torch.int32))

    g = torch.Generator(device="cuda").manual_seed(3)
    scale = torch.rand(N, device=dev(), generator=g) * 1e-3 + 1e-4
    zp = torch.randint(-2, 3, (N,), dtype=torch.int32, device=dev(), generator=g)
    ref.zero_()
    RefKernel("igemm_pipelined_cpasync_perchannel").launch(grid, block, [A, B, ref, M, N, K, scale, zp])
    ours.fill_(-1.0)
    ig.igemm_pipelined_cpasync_perchannel(A, B, ours, M, N, K, scale, zp)
    assert_clean_status()
    assert torch.equal(ours.view(torch.int32), ref.view(torch.int32))


@pytest.mark.parametrize("M,N,K", [(512, 512, 512), (2048, 2048, 2048)])
def test_sparse_equals_the_reference_kernel(M, N, K):
    dense = oracle.gen_sparse_2_4_ref(M, K, 42)                         # bench_sparse.cu:52-64
    comp, meta = oracle.compress_2_4_ref(dense)
    B = rand_i8((K, N), 5)
    s = float(np.float32(1.0) / np.float32(127.0))
    ref = torch.zeros((M, N), dtype=torch.float32, device=dev())
    RefKernel("igemm_sparse_tiled").launch(((N + 127) // 128, (M + 127) // 128), (512, 1),
                                           [T(comp), B, ref, T(meta.view(np.int32)), M, N, K, s, s])
    ours = torch.full((M, N), -1.0, dtype=torch.float32, device=dev())
    ig.igemm_sparse_tiled(T(comp), B, ours, T(meta.view(np.int32)), M, N, K, s, s)
    assert_clean_status()
    assert torch.equal(ours.view(torch.int32), ref.view(torch.int32))


def test_fp16_in_gemm_against_the_reference_kernel_at_4096():
    """The reference adds one fp32 product per 32-wide K tile, this library scales the exact int32 sum
    once: equal up to that summation rounding (bounded by (K/32 + 2) half-ulps of sum |a||b|)."""
    M = N = K = 4096
    g = torch.Generator(device="cuda").manual_seed(7)
    A = (torch.rand((M, K), device=dev(), generator=g) * 2 - 1).half()
    B = (torch.rand((K, N), device=dev(), generator=g) * 2 - 1).half()
    ref = torch.zeros((M, N), dtype=torch.float32, device=dev())
    RefKernel("igemm_online_quant").launch(((N + 127) // 128, (M + 127) // 128), (256, 1), [A, B, ref, M, N, K])
    ours = torch.full((M, N), -1.0, dtype=torch.float32, device=dev())
    ig.igemm_online_quant(A, B, ours, M, N, K)
    assert_clean_status()
    bound = (K // 32 + 2) * 2.0 ** -24 * 1.5 * (A.float().abs() @ B.float().abs())
    assert bool(((ours - ref).abs() <= bound).all())
    assert float((ours - ref).abs().max()) < 1e-2 and float(ref.abs().max()) > 10.0


def test_fp16_in_gemm_with_256_column_blocks_against_the_reference_kernel():
    """igemm_online_quant_bf_128x256 (128 x 256 tiles: one factor per 256 columns of B): the library with
    col_block = 256 against the reference's own kernel, same bound as for the 128-column variants.

    Rows 0 and 1 of every 128-row block are left out.  The reference kernel keeps its cross-warp reduction
    scratch (`reduce_max`, 32 floats) in a union that overlays the first 128 bytes of its fp16 A tile
    (igemm_online_quant_bf_128x256.cu:275-290), and its first-tile quantiser writes that scratch BEFORE it
    converts the tile (:93-96 before :105-121): the first two rows of the first K tile are quantised from the
    block maxima instead of from A.  No bench of the reference launches this kernel, so its output on those
    rows is not a result anything depends on; every other row pins the 256-column arithmetic."""
    M = N = K = 2048
    g = torch.Generator(device="cuda").manual_seed(11)
    A = (torch.rand((M, K), device=dev(), generator=g) * 2 - 1).half()
    B = (torch.rand((K, N), device=dev(), generator=g) * 2 - 1).half()
    ref = torch.zeros((M, N), dtype=torch.float32, device=dev())
    RefKernel("igemm_online_quant_bf_128x256").launch(((N + 255) // 256, (M + 127) // 128), (512, 1), [A, B, ref, M, N, K])
    ours = torch.full((M, N), -1.0, dtype=torch.float32, device=dev())
    ig.igemm_online_quant_bf_128x256(A, B, ours, M, N, K)
    assert_clean_status()
    keep = (torch.arange(M, device=dev()) % 128) >= 2
    bound = (K // 32 + 2) * 2.0 ** -24 * 1.5 * (A.float().abs() @ B.float().abs())
    assert bool(((ours - ref).abs() <= bound)[keep].all())
    assert float((ours - ref)[keep].abs().max()) < 1e-2 and float(ref.abs().max()) > 10.0
    # the block width is part of the result: the 128-column arithmetic gives other numbers
    other = torch.empty_like(ours)
    ig.igemm_online_quant(A, B, other, M, N, K)
    assert not torch.equal(other, ours)
