"""Full-size cases (4096^3 dense and 2:4 sparse, the 8192-token layer, the decode shapes): sampled rows against the CPU oracle plus size-independent properties."""
import numpy as np
import pytest
import torch

import oracle
from bare_metal_b200 import igemm as ig
from _gpu import T, assert_clean_status, dev, ulp_diff_f16

pytestmark = pytest.mark.gpu


def sample_rows(M, count, seed):
    rng = np.random.default_rng(seed)
    return np.unique(np.concatenate([[0, M - 1, 127, 128], rng.integers(0, M, count)]))


def test_config2_w8a8_4096_sampled_rows_and_linearity():
    """Dense W8A8 at full size: M=N=K=4096, int8 uniform, sa/sw ~ U[1e-3,2e-2], fp16 out."""
    M = N = K = 4096
    A = oracle.gen_int8((M, K), 0, oracle.stream_id("C2", "A"))
    W = oracle.gen_int8((N, K), 0, oracle.stream_id("C2", "W"))
    sa = oracle.gen_scales(M, 0, oracle.stream_id("C2", "sa"))
    sw = oracle.gen_scales(N, 0, oracle.stream_id("C2", "sw"))
    Ad, Wd = T(A), T(W)
    D = torch.empty((M, N), dtype=torch.float16, device=dev())
    ig.w8a8_linear(Ad, Wd, D, T(sa), T(sw), M, N, K)
    C = torch.empty((M, N), dtype=torch.int32, device=dev())
    ig.igemm_i32(Ad, Wd, C, M, N, K, ig.BM_B_NK)
    assert_clean_status()
    rows = sample_rows(M, 40, 0)
    acc = oracle.igemm_nt(np.ascontiguousarray(A[rows]), W)
    assert np.array_equal(C.cpu().numpy()[rows], acc)
    want = oracle.dequant_w8a8_f16(acc, sa[rows], sw)
    assert ulp_diff_f16(D.cpu().numpy()[rows].view(np.uint16), want.view(np.uint16)) <= 1
    # reference-ABI layout gives the same integers
    C2 = torch.empty_like(C)
    ig.igemm_i32(Ad, Wd.t().contiguous(), C2, M, N, K, ig.BM_B_KN)
    assert torch.equal(C, C2)
    # linearity: (A1 + A2) W = A1 W + A2 W, with halves that cannot overflow int8
    A1 = (A // 2).astype(np.int8)
    A2 = (A - A1).astype(np.int8)
    C1, C3 = torch.empty_like(C), torch.empty_like(C)
    ig.igemm_i32(T(A1), Wd, C1, M, N, K, ig.BM_B_NK)
    ig.igemm_i32(T(A2), Wd, C3, M, N, K, ig.BM_B_NK)
    assert torch.equal(C1 + C3, C)
    # checksum of checksums: column sums of C equal (column sums of A) . W, in int64
    col = C.sum(dim=0, dtype=torch.int64).cpu().numpy()
    assert np.array_equal(col, A.astype(np.int64).sum(axis=0) @ W.astype(np.int64).T)


def test_config3_sparse_4096_equals_dense_product():
    """2:4 sparse weights at M=N=K=4096, int32 out must equal the dense product bit for bit."""
    M = N = K = 4096
    comp, nib = oracle.gen_sparse_rows(N, K, 0, oracle.stream_id("C3", "W"))
    X = oracle.gen_int8((M, K), 0, oracle.stream_id("C3", "A"))
    Wdense = oracle.decompress_rows(comp, nib)
    Xd = T(X)
    tiled = ig.sp_pack_meta(T(nib), ig.BM_META_ROWS, N, K)
    Cs = torch.empty((M, N), dtype=torch.int32, device=dev())
    ig.w8a8_sparse_i32(Xd, T(comp), tiled, Cs, M, N, K)
    Cd = torch.empty((M, N), dtype=torch.int32, device=dev())
    ig.igemm_i32(Xd, T(Wdense), Cd, M, N, K, ig.BM_B_NK)       # dense kernel on the decompressed weights
    assert_clean_status()
    assert torch.equal(Cs, Cd)
    rows = sample_rows(M, 24, 1)
    assert np.array_equal(Cs.cpu().numpy()[rows], oracle.igemm_nt(np.ascontiguousarray(X[rows]), Wdense))


@pytest.mark.parametrize("M", [1, 16, 64])
def test_config5_decode_shapes(M):
    """Decode shapes: K=8192, N=28672 sparse weights, M in {1,16,64}, fp16 out; every row checked."""
    N, K = 28672, 8192
    comp, nib = oracle.gen_sparse_rows(N, K, 0, oracle.stream_id("C5", "W"))
    X = oracle.gen_int8((M, K), 0, oracle.stream_id("C5", f"X{M}"))
    sa = oracle.gen_scales(M, 0, oracle.stream_id("C5", "sa"))
    sw = oracle.gen_scales(N, 0, oracle.stream_id("C5", "sw"))
    tiled = ig.sp_pack_meta(T(nib), ig.BM_META_ROWS, N, K)
    D = torch.empty((M, N), dtype=torch.float16, device=dev())
    ig.w8a8_sparse_linear(T(X), T(comp), tiled, D, T(sa), T(sw), M, N, K)
    assert_clean_status()
    rows = np.arange(M) if M <= 16 else np.array([0, 1, 17, 31, 32, 63])
    cols = slice(0, N) if M <= 16 else slice(0, N, 7)
    Wd = oracle.decompress_rows(comp[cols], nib[cols])
    want = oracle.dequant_w8a8_f16(oracle.igemm_nt(np.ascontiguousarray(X[rows]), Wd), sa[rows], sw[cols])
    got = D.cpu().numpy()[rows][:, cols]
    assert ulp_diff_f16(np.ascontiguousarray(got).view(np.uint16), want.view(np.uint16)) <= 1


def test_config4_layer_chain_shapes_sampled():
    """The transformer-layer chain: 8192 tokens, hidden 4096: QKV, out, gate+up, down projections, fp16 out."""
    M = 8192
    rows = sample_rows(M, 6, 4)
    for name, K, N in (("qkv", 4096, 12288), ("out", 4096, 4096), ("gate_up", 4096, 22016), ("down", 11008, 4096)):
        X = oracle.gen_int8((M, K), 0, oracle.stream_id("C4", name + "X"))
        W = oracle.gen_int8((N, K), 0, oracle.stream_id("C4", name + "W"))
        sa = oracle.gen_scales(M, 0, oracle.stream_id("C4", name + "sa"))
        sw = oracle.gen_scales(N, 0, oracle.stream_id("C4", name + "sw"))
        D = torch.empty((M, N), dtype=torch.float16, device=dev())
        ig.w8a8_linear(T(X), T(W), D, T(sa), T(sw), M, N, K)
        assert_clean_status()
        want = oracle.dequant_w8a8_f16(oracle.igemm_nt(np.ascontiguousarray(X[rows]), W), sa[rows], sw)
        assert ulp_diff_f16(D[torch.from_numpy(rows).to(dev())].cpu().numpy().view(np.uint16), want.view(np.uint16)) <= 1
