"""The CPU checker against (1) the committed vectors produced by the reference
project's own code and (2), where it is built, that code itself."""
import numpy as np
import pytest

import oracle


def test_fill_random_matches_reference_vectors(golden):
    assert np.array_equal(oracle.fill_random(96, 42), golden["fill_seed42"])
    assert np.array_equal(oracle.fill_random(96, 99), golden["fill_seed99"])
    v = oracle.fill_random(4096, 42)
    assert v.min() >= -1.0 and v.max() < 1.0


def test_sgemm_matches_reference_vectors(golden):
    a = oracle.fill_random(24 * 40, 42).reshape(24, 40)
    b = oracle.fill_random(40 * 16, 99).reshape(40, 16)
    assert np.array_equal(oracle.sgemm(a, b), golden["sgemm_c"])


@pytest.mark.parametrize("M,K", [(32, 64), (48, 128)])
def test_sparse_format_matches_reference_vectors(golden, M, K):
    dense = oracle.gen_sparse_2_4_ref(M, K, 42)
    assert np.array_equal(dense, golden[f"sp_dense_{M}x{K}"])       # same libc rand() stream
    comp, meta = oracle.compress_2_4_ref(dense)
    assert np.array_equal(comp, golden[f"sp_comp_{M}x{K}"])
    assert np.array_equal(meta, golden[f"sp_meta_{M}x{K}"])
    assert meta.size == oracle.sparse_meta_count(M, K) == (M // 16) * (K // 32) * 8
    # decompression inverts compression
    assert np.array_equal(oracle.decompress_2_4_ref(comp, meta, M, K), dense)
    # exact int32 GEMM
    b = golden[f"sp_b_{M}x{K}"]
    c = golden[f"sp_c_{M}x{K}"]
    assert np.array_equal(oracle.igemm(dense, b), c)
    assert np.array_equal(oracle.igemm(dense, b, threads=3), c)
    assert np.array_equal(oracle.igemm_mnk(dense, b), c)
    assert np.array_equal(oracle.igemm_nt(dense, np.ascontiguousarray(b.T)), c)
    assert np.array_equal(dense.astype(np.int64) @ b.astype(np.int64), c)
    # per-row nibble format carries the same positions
    nib = oracle.meta_ref_to_rows(meta, M, K)
    assert np.array_equal(oracle.decompress_rows(comp, nib), dense)


def test_check_fp32_and_logic(golden):
    r = oracle.check_fp32(golden["check_gpu"], golden["check_ref"], 0.5, 0.1)
    assert [r["num_errors"], r["first_error"]] == list(golden["check_result"])
    assert np.allclose([r["max_abs"], r["max_rel"]], golden["check_max"], rtol=0, atol=0)
    # element 1 (abs 0.6, rel 0.06) passes: both limits must be exceeded to fail
    assert r["num_errors"] == 2


@pytest.mark.skipif(not oracle.have_ref(), reason="reference build absent")
def test_restatement_equals_reference_build_on_fresh_inputs():
    for seed in (1, 42, 1234):
        assert np.array_equal(oracle.fill_random(1000, seed), oracle.ref_fill_random(1000, seed))
        d0 = oracle.gen_sparse_2_4_ref(64, 96, seed)
        d1 = oracle.ref_gen_random_sparse_2_4_int8(64, 96, seed)
        assert np.array_equal(d0, d1)
        c0, m0 = oracle.compress_2_4_ref(d0)
        c1, m1 = oracle.ref_compress_2_4_int8(d1)
        assert np.array_equal(c0, c1) and np.array_equal(m0, m1)
        b = oracle.gen_int8((96, 40), seed, 5)
        ref_c = oracle.ref_cpu_sparse_gemm_int8(d1, b)
        assert np.array_equal(oracle.igemm(d0, b), ref_c)
        assert np.array_equal(oracle.ref_cpu_sparse_gemm_int8(d1, b, threads=4), ref_c)
    # compressor fall-backs on groups with fewer than two non-zeros (sparse_meta_int8.h:160-161)
    d = np.zeros((16, 32), np.int8)
    d[0, 1] = 5
    d[3, 7] = -9
    c0, m0 = oracle.compress_2_4_ref(d)
    c1, m1 = oracle.ref_compress_2_4_int8(d)
    assert np.array_equal(c0, c1) and np.array_equal(m0, m1)
    a = oracle.fill_random(20 * 12, 3).reshape(20, 12)
    bb = oracle.fill_random(12 * 8, 4).reshape(12, 8)
    assert np.array_equal(oracle.sgemm(a, bb), oracle.ref_cpu_sgemm(a, bb))


def test_quantize_symmetric():
    x = oracle.fill_random(4096, 42)
    s = oracle.compute_scale(x)
    assert s == np.float32(np.abs(x).max()) / np.float32(127.0)
    q = oracle.quantize_symmetric(x, s)
    assert q.dtype == np.int8 and q.max() == 127 and q.min() >= -128
    expect = np.clip(np.sign(x * (np.float32(1.0) / np.float32(s))) *
                     np.floor(np.abs(x * (np.float32(1.0) / np.float32(s))) + np.float32(0.5)), -128, 127)
    assert np.array_equal(q, expect.astype(np.int8))
    assert oracle.compute_scale(np.zeros(8, np.float32)) == 1.0


def test_epilogues():
    rng = np.random.default_rng(0)
    acc = rng.integers(-(2 ** 26), 2 ** 26, size=(8, 12), dtype=np.int32)
    sa, sb = np.float32(0.013), np.float32(0.0071)
    got = oracle.dequant_per_tensor(acc, sa, sb)
    assert np.array_equal(got, acc.astype(np.float32) * (sa * sb))
    scale, zp = oracle.gen_per_channel_params(12, sa, sb)
    assert zp.min() >= -2 and zp.max() <= 2
    got = oracle.dequant_per_channel(acc, scale, zp)
    assert np.array_equal(got, (acc.astype(np.float32) - zp.astype(np.float32)[None, :]) * scale[None, :])
    sa_m = oracle.gen_scales(8, 0, 1)
    sw_n = oracle.gen_scales(12, 0, 2)
    assert sa_m.min() >= 1e-3 and sa_m.max() <= 2e-2
    got = oracle.dequant_w8a8_f16(acc, sa_m, sw_n)
    y = acc.astype(np.float32) * (sa_m[:, None] * sw_n[None, :])
    assert np.array_equal(got.view(np.uint16), y.astype(np.float16).view(np.uint16))


def test_f32_to_f16_round_to_nearest_even():
    rng = np.random.default_rng(1)
    bits = rng.integers(0, 2 ** 32, size=20000, dtype=np.uint64).astype(np.uint32)
    special = np.array([0, 0x80000000, 0x33000000, 0x33000001, 0x387FC000, 0x387FE000, 0x477FEFFF,
                        0x477FF000, 0x7F800000, 0xFF800000, 0x38800000, 0x3F801000, 0x3F803000], np.uint32)
    f = np.concatenate([bits, special]).view(np.float32)
    f = f[~np.isnan(f)]
    with np.errstate(over="ignore"):
        want = f.astype(np.float16).view(np.uint16)
    got = np.array([oracle.lib().orc_f32_to_f16(float(x)) for x in f], np.uint16)
    assert np.array_equal(got, want)


def test_seeded_generators():
    s = oracle.stream_id("C2", "A")
    a = oracle.gen_int8((64, 128), 0, s)
    assert np.array_equal(a, oracle.gen_int8((64, 128), 0, s))
    assert a.min() >= -127 and a.max() <= 127 and not np.array_equal(a, oracle.gen_int8((64, 128), 1, s))
    big = oracle.gen_int8((1 << 16,), 0, s).astype(np.int32)
    assert abs(big.mean()) < 1.5 and len(np.unique(big)) == 255
    comp, nib = oracle.gen_sparse_rows(32, 256, 0, oracle.stream_id("C3", "W"))
    assert (comp != 0).all()
    lo, hi = nib & 0xF, nib >> 4
    for n in (lo, hi):
        assert ((n & 3) < (n >> 2)).all()
    assert len(np.unique(lo)) == 6
    dense = oracle.decompress_rows(comp, nib)
    assert ((dense.reshape(32, 64, 4) != 0).sum(axis=2) == 2).all()


def test_prune_reproduces_the_reference_compressor_on_2_4_input():
    """The reference has no pruner; on a matrix its own generator made 2:4 (kept values never 0,
    sparse_meta_int8.h:91-96) pruning by magnitude must give exactly what compress_2_4_int8 gives."""
    M, K = 64, 256
    dense = oracle.gen_sparse_2_4_ref(M, K, 42)
    comp_ref, meta_ref = oracle.compress_2_4_ref(dense)
    comp, nib = oracle.prune_2_4_rows(dense)
    assert np.array_equal(comp, comp_ref)
    assert np.array_equal(nib, oracle.meta_ref_to_rows(meta_ref, M, K))
    assert np.array_equal(oracle.decompress_rows(comp, nib), dense)


def test_prune_keeps_the_two_largest_magnitudes_ties_to_the_lower_position():
    W = np.array([[5, -5, 5, 1,   0, 0, 0, 0,   -128, 127, 3, -127,   1, 2, 3, 4] + [0] * 16], np.int8)
    comp, nib = oracle.prune_2_4_rows(W)
    assert comp[0, :8].tolist() == [5, -5, 0, 0, -128, 127, 3, 4]
    assert nib[0, :2].tolist() == [(1 << 2 | 0) | ((1 << 2 | 0) << 4), (1 << 2 | 0) | ((3 << 2 | 2) << 4)]
    rng = np.random.default_rng(5)
    W = rng.integers(-128, 128, (48, 128), dtype=np.int8)
    comp, nib = oracle.prune_2_4_rows(W)
    kept = oracle.decompress_rows(comp, nib).astype(np.int32).reshape(48, 32, 4)
    full = W.astype(np.int32).reshape(48, 32, 4)
    # the dropped pair never outweighs the kept pair, and exactly two positions survive unless zero
    assert (np.abs(full).sum(-1) - np.abs(kept).sum(-1) <= np.abs(kept).sum(-1)).all()
    top2 = np.sort(np.abs(full), axis=-1)[..., 2:].sum(-1)
    assert np.array_equal(np.abs(kept).sum(-1), top2)


def test_online_quant_restatement_equals_the_reference_kernel_bit_for_bit():
    """tests/golden/online_quant_reference.npz holds outputs of the reference's own
    igemm_online_quant kernel (compiled unmodified for sm_100a, run on a B200 by
    tests/golden/make_online_quant_golden.py).  The C restatement must reproduce every bit,
    including blocks whose first K tile is all zero and values clamped by the re-used factors."""
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "online_quant_reference.npz"))
    for i, (M, N, K) in enumerate(g["shapes"]):
        A, B, C = g[f"A{i}"].view(np.float16), g[f"B{i}"].view(np.float16), g[f"C{i}"]
        assert A.shape == (M, K) and B.shape == (K, N)
        got = oracle.online_quant_gemm(A, B)
        assert np.array_equal(got.view(np.uint32), C.view(np.uint32)), (M, N, K)
    assert any((g[f"C{i}"] == 0).any() for i in range(len(g["shapes"])))      # the zero-first-tile block is in there


def test_online_quant_256_column_blocks_share_one_factor():
    rng = np.random.default_rng(3)
    A = (rng.random((128, 64), dtype=np.float32) * 2 - 1).astype(np.float16)
    B = (rng.random((64, 256), dtype=np.float32) * 2 - 1).astype(np.float16)
    B[:32, 128:] *= np.float16(0.25)                   # right half has a smaller first-tile maximum
    c128, c256 = oracle.online_quant_gemm(A, B, 128), oracle.online_quant_gemm(A, B, 256)
    assert np.array_equal(c128[:, :128], c256[:, :128])            # the left block's maximum rules both
    assert not np.array_equal(c128[:, 128:], c256[:, 128:])


@pytest.mark.skipif(not oracle.have_ref_f16(), reason="reference checkout absent and no prebuilt oracle/_ref")
def test_fp16_sparse_utilities_equal_the_reference_headers():
    """kernels/gemm/hgemm_sparse/sparse_meta.h compiled in place vs the restatement, bit for bit."""
    R = oracle.ref_f16()
    for M, K, N, seed in ((16, 16, 16, 1), (64, 96, 48, 999), (128, 256, 32, 7)):
        assert oracle.h_sparse_meta_count(M, K) == R.ref_h_sparse_meta_count(M, K)
        want = np.empty((M, K), np.float32)
        R.ref_h_gen_sparse_2_4(want.ctypes.data, M, K, seed)
        got = oracle.h_gen_sparse_2_4(M, K, seed)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        comp, meta = oracle.h_compress_2_4(got)
        comp_w = np.empty((M, K // 2), np.float16)
        meta_w = np.empty(oracle.h_sparse_meta_count(M, K), np.uint32)
        R.ref_h_compress_2_4(want.ctypes.data, M, K, comp_w.ctypes.data, meta_w.ctypes.data)
        assert np.array_equal(comp.view(np.uint16), comp_w.view(np.uint16)) and np.array_equal(meta, meta_w)
        B = oracle.fill_random(K * N, 137).reshape(K, N)
        c_w = np.empty((M, N), np.float32)
        R.ref_h_cpu_sparse_gemm(want.ctypes.data, B.ctypes.data, c_w.ctypes.data, M, N, K)
        assert np.array_equal(oracle.h_cpu_sparse_gemm(got, B).view(np.uint32), c_w.view(np.uint32))
        # round trip through the format
        assert np.array_equal(oracle.h_decompress_2_4(comp, meta).view(np.uint16), got.astype(np.float16).view(np.uint16))
