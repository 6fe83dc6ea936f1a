"""2:4 structured-sparse INT8 GEMM on the GPU against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

import oracle
from bare_metal_b200 import igemm as ig
from _gpu import T, assert_clean_status, dev, forced_bn, ulp_diff_f16

pytestmark = pytest.mark.gpu


def bench_sparse_inputs(M, N, K):
    """bench_sparse.cu:52-64: generator seed 42, reference compressor, scales 1/127."""
    dense = oracle.gen_sparse_2_4_ref(M, K, 42)
    comp, meta = oracle.compress_2_4_ref(dense)
    B = oracle.gen_int8((K, N), 137, 1)
    B[B == 0] = 1                                  # the bench draws non-zero B (bench_sparse.cu:55-60)
    return dense, comp, meta, B


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (512, 512, 512), (128, 16, 32), (144, 272, 1056)])
def test_reference_sparse_kernel_abi(M, N, K):
    """igemm_sparse_tiled's ABI and acceptance test: fp32 out vs exact int32 CPU GEMM * (1/127)^2."""
    dense, comp, meta, B = bench_sparse_inputs(M, N, K)
    s = np.float32(1.0) / np.float32(127.0)
    C = torch.full((M, N), -1.0, dtype=torch.float32, device=dev())
    ig.igemm_sparse_tiled(T(comp), T(B), C, T(meta.view(np.int32)), M, N, K, float(s), float(s))
    assert_clean_status()
    want = oracle.dequant_per_tensor(oracle.igemm(dense, B, threads=0), s, s)
    got = C.cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    r = oracle.check_fp32(got, want, 0.5, 0.1)
    assert r["num_errors"] == 0 and r["max_abs"] == 0.0        # the reference fixture shows max_abs=0


def test_golden_sparse_vectors_from_the_reference_build(golden):
    """Inputs AND outputs produced by the reference's own CPU code (tests/golden)."""
    for (M, K) in ((32, 64), (48, 128)):
        comp, meta = golden[f"sp_comp_{M}x{K}"], golden[f"sp_meta_{M}x{K}"]
        B, want = golden[f"sp_b_{M}x{K}"], golden[f"sp_c_{M}x{K}"]
        N = B.shape[1]
        Bp = np.zeros((K, 32), np.int8)             # pad N 24 -> 32 for the 16-byte pitch rule
        Bp[:, :N] = B
        C = torch.zeros((M, 32), dtype=torch.int32, device=dev())
        ig.igemm_sparse_i32(T(comp), T(meta.view(np.int32)), ig.BM_META_REF, T(Bp), C, M, 32, K, ig.BM_B_KN)
        assert_clean_status()
        assert np.array_equal(C.cpu().numpy()[:, :N], want)


def test_known_answer_all_ones():
    """tests/hgemm_sparse/test_mma_sp.cu pattern: all-ones operands, metadata 0x44444444
    (positions 0,1 in every group) -> every output equals K/2."""
    M, N, K = 128, 128, 512
    comp = np.ones((M, K // 2), np.int8)
    meta = np.full(oracle.sparse_meta_count(M, K), 0x44444444, np.uint32)
    B = np.ones((K, N), np.int8)
    C = torch.zeros((M, N), dtype=torch.int32, device=dev())
    ig.igemm_sparse_i32(T(comp), T(meta.view(np.int32)), ig.BM_META_REF, T(B), C, M, N, K, ig.BM_B_KN)
    assert_clean_status()
    assert (C.cpu().numpy() == K // 2).all()
    # position decode: B[k][:] = k % 4 makes the output the sum of the selected positions
    Bpos = (np.arange(K) % 4).astype(np.int8)[:, None].repeat(N, 1)
    for nibble, s in ((0x4, 0 + 1), (0xE, 2 + 3), (0x9, 1 + 2), (0xC, 0 + 3)):
        word = sum(nibble << (4 * i) for i in range(8))
        meta[:] = word
        ig.igemm_sparse_i32(T(comp), T(meta.view(np.int32)), ig.BM_META_REF, T(Bpos), C, M, N, K, ig.BM_B_KN)
        assert (C.cpu().numpy() == s * (K // 4)).all()


@pytest.mark.parametrize("layout", [ig.BM_B_NK, ig.BM_B_KN])
@pytest.mark.parametrize("M,N,K,bn", [(128, 128, 256, 128), (128, 256, 256, 256), (128, 128, 64, 128),
                                      (256, 256, 512, 128), (128, 64, 256, 64), (272, 400, 1056, None),
                                      (512, 512, 1024, None)])
def test_sparse_left_rows_format(layout, M, N, K, bn):
    """Independent 6-pattern sparsity per row (no r/r+8 sharing), per-row nibble metadata."""
    if layout == ig.BM_B_KN and bn == 64:
        bn = 128
    comp, nib = oracle.gen_sparse_rows(M, K, 0, 11)
    B = oracle.gen_int8((K, N), 0, 12)
    want = oracle.igemm(oracle.decompress_rows(comp, nib), B, threads=0)
    C = torch.full((M, N), -7, dtype=torch.int32, device=dev())
    with forced_bn(bn):
        ig.igemm_sparse_i32(T(comp), T(nib), ig.BM_META_ROWS, T(B) if layout == ig.BM_B_KN else T(B.T),
                            C, M, N, K, layout)
    assert_clean_status()
    assert np.array_equal(C.cpu().numpy(), want)


@pytest.mark.parametrize("M,N,K,bn", [(16, 128, 256, 16), (1, 256, 512, 16), (32, 128, 256, 32), (64, 256, 512, 64),
                                      (128, 256, 512, 128), (256, 384, 1024, 256), (100, 200, 288, None),
                                      (3, 136, 96, None), (64, 1024, 2048, None), (300, 520, 800, None)])
def test_sparse_weights_i32_and_f16(M, N, K, bn):
    """Sparse WEIGHTS W[N,K] (the convention of the sparse-weight workloads): C = X @ W^T, int32 bit-exact, fp16 <= 1 ulp."""
    comp, nib = oracle.gen_sparse_rows(N, K, 0, 21)
    X = oracle.gen_int8((M, K), 0, 22)
    want = oracle.igemm_nt(X, oracle.decompress_rows(comp, nib))
    tiled = ig.sp_pack_meta(T(nib), ig.BM_META_ROWS, N, K)
    guard = torch.full((M + 2, N), 0x5A5A5A5A, dtype=torch.int32, device=dev())
    C = guard[1:M + 1]
    with forced_bn(bn):
        ig.w8a8_sparse_i32(T(X), T(comp), tiled, C, M, N, K)
    assert_clean_status()
    g = guard.cpu().numpy()
    assert np.array_equal(g[1:M + 1], want)
    assert (g[0] == 0x5A5A5A5A).all() and (g[-1] == 0x5A5A5A5A).all()
    sa, sw = oracle.gen_scales(M, 0, 3), oracle.gen_scales(N, 0, 4)
    D = torch.zeros((M, N), dtype=torch.float16, device=dev())
    with forced_bn(bn):
        ig.w8a8_sparse_linear(T(X), T(comp), tiled, D, T(sa), T(sw), M, N, K)
    assert_clean_status()
    assert ulp_diff_f16(D.cpu().numpy().view(np.uint16), oracle.dequant_w8a8_f16(want, sa, sw).view(np.uint16)) <= 1


def test_metadata_repack_formats_agree():
    """Reference uint32 words and per-row nibbles describe the same positions -> same tiled bytes."""
    M, K = 272, 800
    dense = oracle.gen_sparse_2_4_ref(M, K, 42)
    comp, meta = oracle.compress_2_4_ref(dense)
    nib = oracle.meta_ref_to_rows(meta, M, K)
    t_ref = ig.sp_pack_meta(T(meta.view(np.int32)), ig.BM_META_REF, M, K).cpu().numpy()
    t_rows = ig.sp_pack_meta(T(nib), ig.BM_META_ROWS, M, K).cpu().numpy()
    assert np.array_equal(t_ref, t_rows)
    # tiled order: [row block][k block][chunk][row][16 bytes]; padding is the valid pattern 0x44
    kb = (K + 255) // 256
    t = t_rows.reshape((M + 127) // 128, kb, 2, 128, 16)
    rows = t.transpose(0, 3, 1, 2, 4).reshape(-1, kb * 32)
    assert np.array_equal(rows[:M, :K // 8], nib)
    assert (rows[M:] == 0x44).all() and (rows[:M, K // 8:] == 0x44).all()


def test_sparse_repeat_launches_are_bit_identical():
    M, N, K = 64, 2048, 4096
    comp, nib = oracle.gen_sparse_rows(N, K, 1, 21)
    X = T(oracle.gen_int8((M, K), 1, 22))
    compd, tiled = T(comp), ig.sp_pack_meta(T(nib), ig.BM_META_ROWS, N, K)
    first = None
    for i in range(30):
        C = torch.empty((M, N), dtype=torch.int32, device=dev())
        ig.w8a8_sparse_i32(X, compd, tiled, C, M, N, K)
        if first is None:
            first = C.clone()
        else:
            assert torch.equal(C, first), f"launch {i} differs"
    assert_clean_status()


@pytest.mark.parametrize("M,N,K,bn", [(1, 256, 512, 16), (16, 384, 1024, 16), (64, 200, 288, 64), (128, 256, 512, 128),
                                      (300, 520, 800, None), (33, 1024, 2048, None)])
def test_packed_sparse_weights_match_oracle(M, N, K, bn):
    """Packed weight blocks (pre-swizzled values + metadata, 20 KiB per block): same results."""
    comp, nib = oracle.gen_sparse_rows(N, K, 2, 31)
    X = oracle.gen_int8((M, K), 2, 32)
    want = oracle.igemm_nt(X, oracle.decompress_rows(comp, nib))
    packed = ig.sp_pack_weights(T(comp), T(nib), ig.BM_META_ROWS, N, K)
    C = torch.full((M, N), -7, dtype=torch.int32, device=dev())
    with forced_bn(bn):
        ig.w8a8_sparse_i32_packed(T(X), packed, C, M, N, K)
    assert_clean_status()
    assert np.array_equal(C.cpu().numpy(), want)
    sa, sw = oracle.gen_scales(M, 2, 3), oracle.gen_scales(N, 2, 4)
    D = torch.zeros((M, N), dtype=torch.float16, device=dev())
    with forced_bn(bn):
        ig.w8a8_sparse_linear_packed(T(X), packed, D, T(sa), T(sw), M, N, K)
    assert_clean_status()
    assert ulp_diff_f16(D.cpu().numpy().view(np.uint16), oracle.dequant_w8a8_f16(want, sa, sw).view(np.uint16)) <= 1
    # packing from already-tiled metadata gives the same blocks
    tiled = ig.sp_pack_meta(T(nib), ig.BM_META_ROWS, N, K)
    packed2 = ig.sp_pack_weights(T(comp), tiled, ig.BM_META_TILED, N, K)
    assert torch.equal(packed, packed2)


@pytest.mark.parametrize("M,N,K", [(240, 256, 256), (100, 130, 288), (400, 520, 1056), (500, 512, 4096), (1000, 1100, 544)])
def test_sparse_weights_on_cta_pairs(M, N, K):
    """Sparse weights on the CTA-pair kernel (tcgen05.mma.sp.cta_group::2, 256 channels x 240 tokens)."""
    comp, nib = oracle.gen_sparse_rows(N, K, 4, 51)
    X = oracle.gen_int8((M, K), 4, 52)
    want = oracle.igemm_nt(X, oracle.decompress_rows(comp, nib))
    tiled = ig.sp_pack_meta(T(nib), ig.BM_META_ROWS, N, K)
    guard = torch.full((M + 2, N), 0x5A5A5A5A, dtype=torch.int32, device=dev())
    with forced_bn(240):
        ig.w8a8_sparse_i32(T(X), T(comp), tiled, guard[1:M + 1], M, N, K)
    assert_clean_status()
    g = guard.cpu().numpy()
    assert np.array_equal(g[1:M + 1], want)
    assert (g[0] == 0x5A5A5A5A).all() and (g[-1] == 0x5A5A5A5A).all()
    sa, sw = oracle.gen_scales(M, 4, 3), oracle.gen_scales(N, 4, 4)
    D = torch.zeros((M, N), dtype=torch.float16, device=dev())
    with forced_bn(240):
        ig.w8a8_sparse_linear(T(X), T(comp), tiled, D, T(sa), T(sw), M, N, K)
    assert_clean_status()
    assert ulp_diff_f16(D.cpu().numpy().view(np.uint16), oracle.dequant_w8a8_f16(want, sa, sw).view(np.uint16)) <= 1


@pytest.mark.parametrize("M,N,K", [(16, 2000, 512), (1, 28672, 256), (64, 1504, 1024), (5, 4097, 288)])
def test_row_balanced_decode_tiles(M, N, K):
    """Decode shapes on packed weights: rows are dealt to the SMs in multiples of 8 (ragged last
    tiles fetch only their own rows); results must not depend on where the cuts fall."""
    from _gpu import options
    comp, nib = oracle.gen_sparse_rows(N, K, 5, 61)
    X = oracle.gen_int8((M, K), 5, 62)
    want = oracle.igemm_nt(X, oracle.decompress_rows(comp, nib))
    packed = ig.sp_pack_weights(T(comp), T(nib), ig.BM_META_ROWS, N, K)
    sa, sw = oracle.gen_scales(M, 5, 3), oracle.gen_scales(N, 5, 4)
    want16 = oracle.dequant_w8a8_f16(want, sa, sw).view(np.uint16)
    for balanced in (1, 0):
        with options(row_balanced=balanced):
            guard = torch.full((M + 2, N), 0x5A5A5A5A, dtype=torch.int32, device=dev())
            ig.w8a8_sparse_i32_packed(T(X), packed, guard[1:M + 1], M, N, K)
            assert_clean_status()
            g = guard.cpu().numpy()
            assert np.array_equal(g[1:M + 1], want)
            assert (g[0] == 0x5A5A5A5A).all() and (g[-1] == 0x5A5A5A5A).all()
            D = torch.zeros((M, N), dtype=torch.float16, device=dev())
            ig.w8a8_sparse_linear_packed(T(X), packed, D, T(sa), T(sw), M, N, K)
            assert_clean_status()
            assert ulp_diff_f16(D.cpu().numpy().view(np.uint16), want16) <= 1


@pytest.mark.parametrize("R,K", [(16, 32), (300, 1056), (4096, 4096)])
def test_prune_to_2_4_matches_the_oracle_and_feeds_the_sparse_gemm(R, K):
    """Weight tooling: magnitude pruning + compression on the GPU, bit-exact against the CPU restatement,
    then used as the sparse weights of a GEMM whose result equals the dense product of the pruned matrix."""
    W = oracle.gen_int8((R, K), 21, 1)
    comp_want, nib_want = oracle.prune_2_4_rows(W)
    comp, nib = ig.prune_2_4(T(W), R, K)
    assert np.array_equal(comp.cpu().numpy(), comp_want)
    assert np.array_equal(nib.cpu().numpy(), nib_want)
    if R > 1024:
        return
    M = 48
    X = oracle.gen_int8((M, K), 21, 2)
    tiled = ig.sp_pack_meta(nib, ig.BM_META_ROWS, R, K)
    C = torch.empty((M, R), dtype=torch.int32, device=dev())
    ig.w8a8_sparse_i32(T(X), comp, tiled, C, M, R, K)
    assert_clean_status()
    pruned = oracle.decompress_rows(comp_want, nib_want)
    assert np.array_equal(C.cpu().numpy(), oracle.igemm(X, np.ascontiguousarray(pruned.T), threads=0))


@pytest.mark.parametrize("M,N,K", [(256, 224, 256), (512, 448, 512), (144, 272, 1056), (400, 1008, 96), (1024, 2240, 2048)])
def test_reference_orientation_on_cta_pairs(M, N, K):
    """Sparse operand on the left, B[K x N], on CTA pairs (256 x 224 tiles; forced here, chosen by itself
    for large shapes): exact int32 against the CPU GEMM of the decompressed matrix, ragged edges included,
    and the fp32 reference ABI on top of the same integers."""
    dense, comp, meta, B = bench_sparse_inputs(M, N, K)
    want = oracle.igemm(dense, B, threads=0)
    tiled = ig.sp_pack_meta(T(meta.view(np.int32)), ig.BM_META_REF, M, K)
    buf = torch.full((M + 2, N), 0x5A5A5A5A, dtype=torch.int32, device=dev())
    with forced_bn(224):
        ig.igemm_sparse_i32(T(comp), tiled, ig.BM_META_TILED, T(B), buf[1:M + 1], M, N, K, ig.BM_B_KN)
        assert_clean_status()
        g = buf.cpu().numpy()
        assert (g[0] == 0x5A5A5A5A).all() and (g[-1] == 0x5A5A5A5A).all(), "store outside the output"
        assert np.array_equal(g[1:M + 1], want)
        s = np.float32(1.0) / np.float32(127.0)
        C = torch.full((M, N), -1.0, dtype=torch.float32, device=dev())
        ig.igemm_sparse_tiled(T(comp), T(B), C, T(meta.view(np.int32)), M, N, K, float(s), float(s))
        assert_clean_status()
        assert np.array_equal(C.cpu().numpy().view(np.uint32), oracle.dequant_per_tensor(want, s, s).view(np.uint32))


@pytest.mark.parametrize("order", [0, 1])
def test_pair_kernel_tile_orders_give_the_same_integers(order):
    """Sparse weights on CTA pairs with row blocks fastest and with column tiles fastest (the order picked
    for weights larger than L2): exact int32 either way, ragged tiles on both axes."""
    from _gpu import options
    M, N, K = 500, 1100, 512                      # 3 token tiles of 240, 5 channel blocks of 256
    comp, nib = oracle.gen_sparse_rows(N, K, 31, 1)
    X = oracle.gen_int8((M, K), 31, 2)
    tiled = ig.sp_pack_meta(T(nib), ig.BM_META_ROWS, N, K)
    C = torch.full((M, N), -9, dtype=torch.int32, device=dev())
    with options(sparse_col_first=order), forced_bn(240):
        ig.w8a8_sparse_i32(T(X), T(comp), tiled, C, M, N, K)
    assert_clean_status()
    assert np.array_equal(C.cpu().numpy(), oracle.igemm_nt(X, oracle.decompress_rows(comp, nib)))


@pytest.mark.parametrize("M,N,K", [(1, 2400, 1024), (16, 3584, 512), (64, 4744, 768), (33, 9480, 512)])
def test_short_stage_decode_tiles(M, N, K):
    """A CTA that is dealt few rows (the slab of an N-split layer) uses ring stages of 32 or 64 rows and a deeper
    ring; whatever the stage height, chosen or pinned, the integers and the fp16 outputs are the oracle's."""
    from _gpu import options
    comp, nib = oracle.gen_sparse_rows(N, K, 6, 71)
    X = oracle.gen_int8((M, K), 6, 72)
    want = oracle.igemm_nt(X, oracle.decompress_rows(comp, nib))
    packed = ig.sp_pack_weights(T(comp), T(nib), ig.BM_META_ROWS, N, K)
    sa, sw = oracle.gen_scales(M, 6, 3), oracle.gen_scales(N, 6, 4)
    want16 = oracle.dequant_w8a8_f16(want, sa, sw).view(np.uint16)
    for rows in (0, 32, 64, 128):
        with options(decode_tile_rows=rows):
            guard = torch.full((M + 2, N), 0x5A5A5A5A, dtype=torch.int32, device=dev())
            ig.w8a8_sparse_i32_packed(T(X), packed, guard[1:M + 1], M, N, K)
            assert_clean_status()
            g = guard.cpu().numpy()
            assert np.array_equal(g[1:M + 1], want), f"stage rows {rows}"
            assert (g[0] == 0x5A5A5A5A).all() and (g[-1] == 0x5A5A5A5A).all()
            D = torch.zeros((M, N), dtype=torch.float16, device=dev())
            ig.w8a8_sparse_linear_packed(T(X), packed, D, T(sa), T(sw), M, N, K)
            assert_clean_status()
            assert ulp_diff_f16(D.cpu().numpy().view(np.uint16), want16) <= 1, f"stage rows {rows}"
