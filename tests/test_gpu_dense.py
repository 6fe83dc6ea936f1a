"""Dense INT8 GEMM + epilogues on the GPU against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

import oracle
from bare_metal_b200 import igemm as ig
from _gpu import T, assert_clean_status, dev, forced_bn, ulp_diff_f16

pytestmark = pytest.mark.gpu


def run_i32(A, B_kn, layout, bn=None, guard=False):
    M, K = A.shape
    N = B_kn.shape[1]
    Bd = T(B_kn) if layout == ig.BM_B_KN else T(B_kn.T)
    if guard:
        # canary bands on both sides of the output catch any out-of-range store
        buf = torch.full((M + 2, N), 0x5A5A5A5A, dtype=torch.int32, device=dev())
        C = buf[1:M + 1]
    else:
        C = torch.full((M, N), -7, dtype=torch.int32, device=dev())
    with forced_bn(bn):
        ig.igemm_i32(T(A), Bd, C, M, N, K, layout)
    assert_clean_status()
    if guard:
        g = buf.cpu().numpy()
        assert (g[0] == 0x5A5A5A5A).all() and (g[-1] == 0x5A5A5A5A).all(), "store outside the output"
    return C.cpu().numpy()


def test_config1_dense_1024_bit_exact_both_layouts():
    """The 1024^3 dense case: M=N=K=1024, int8 uniform [-127,127], seed 0, int32 out, bit-exact."""
    A = oracle.gen_int8((1024, 1024), 0, oracle.stream_id("C1", "A"))
    B = oracle.gen_int8((1024, 1024), 0, oracle.stream_id("C1", "B"))
    want = oracle.igemm(A, B, threads=0)
    assert np.array_equal(run_i32(A, B, ig.BM_B_KN), want)      # reference ABI: B[K x N]
    assert np.array_equal(run_i32(A, B, ig.BM_B_NK), want)      # K-major weights


@pytest.mark.parametrize("layout", [ig.BM_B_NK, ig.BM_B_KN])
@pytest.mark.parametrize("M,N,K,bn", [
    (128, 256, 128, 256), (128, 128, 32, 128), (128, 64, 64, 64), (256, 512, 256, 256),
    (384, 640, 512, 128), (1, 16, 16, None), (7, 48, 16, None), (129, 272, 144, None),
    (200, 304, 2064, None), (640, 1040, 528, 256), (130, 80, 4096, 64), (1000, 1008, 1008, None),
])
def test_dense_shapes_bit_exact(layout, M, N, K, bn):
    if layout == ig.BM_B_KN and bn == 64:
        bn = 128
    A = oracle.gen_int8((M, K), 3, 1)
    B = oracle.gen_int8((K, N), 3, 2)
    got = run_i32(A, B, layout, bn, guard=True)
    assert np.array_equal(got, oracle.igemm(A, B, threads=0))


def test_extreme_values_no_overflow_surprises():
    """All -127 x all -127 and -128 x 127 corners: exact int32 at K = 8192."""
    M, N, K = 128, 128, 8192
    for a, b in ((-127, -127), (-128, 127), (127, 127), (-128, -128)):
        A = np.full((M, K), a, np.int8)
        B = np.full((K, N), b, np.int8)
        got = run_i32(A, B, ig.BM_B_NK)
        assert (got == a * b * K).all()


def test_reference_bench_inputs_per_tensor_and_per_channel():
    """The dense bench's own recipe (bench.cu:268-289,459-467): LCG fp32 data seeds 42/99,
    symmetric quantisation, per-tensor and per-channel dequantised fp32 outputs."""
    M = N = K = 256
    a32 = oracle.fill_random(M * K, 42).reshape(M, K)
    b32 = oracle.fill_random(K * N, 99).reshape(K, N)
    sa, sb = oracle.compute_scale(a32), oracle.compute_scale(b32)
    A, B = oracle.quantize_symmetric(a32, sa), oracle.quantize_symmetric(b32, sb)
    acc = oracle.igemm_mnk(A, B)
    C = torch.zeros((M, N), dtype=torch.float32, device=dev())
    ig.igemm_wmma(T(A), T(B), C, M, N, K, sa, sb)
    assert_clean_status()
    got = C.cpu().numpy()
    assert np.array_equal(got.view(np.uint32), oracle.dequant_per_tensor(acc, sa, sb).view(np.uint32))
    # the reference's own acceptance test: fp32 SGEMM of the unquantised data, abs 0.5 AND rel 0.1
    r = oracle.check_fp32(got, oracle.sgemm(a32, b32), 0.5, 0.1)
    assert r["num_errors"] == 0 and r["max_abs"] < 0.5
    # every alias of the per-tensor family is the same entry point
    for fn in (ig.igemm_tiled, ig.igemm_pipelined_cpasync, ig.igemm_8warp_256, ig.igemm_persistent):
        C.zero_()
        fn(T(A), T(B), C, M, N, K, sa, sb)
        assert np.array_equal(C.cpu().numpy(), got)
    scale, zp = oracle.gen_per_channel_params(N, sa, sb, 123)
    ig.igemm_pipelined_cpasync_perchannel(T(A), T(B), C, M, N, K, T(scale), T(zp))
    assert_clean_status()
    want = oracle.dequant_per_channel(acc, scale, zp)
    assert np.array_equal(C.cpu().numpy().view(np.uint32), want.view(np.uint32))
    assert oracle.check_fp32(C.cpu().numpy(), want, 0.5, 0.1)["num_errors"] == 0


@pytest.mark.parametrize("layout", [ig.BM_B_NK, ig.BM_B_KN])
@pytest.mark.parametrize("M,N,K", [(256, 384, 512), (100, 208, 1040), (1, 4096, 4096), (513, 272, 64)])
def test_w8a8_fp16_within_one_ulp(layout, M, N, K):
    """fp16 D = half_rn(float(acc) * (sa[m]*sw[n])): tolerance 1 fp16 ulp of the fp32 oracle."""
    A = oracle.gen_int8((M, K), 0, 1)
    B = oracle.gen_int8((K, N), 0, 2)
    sa = oracle.gen_scales(M, 0, 3)
    sw = oracle.gen_scales(N, 0, 4)
    want = oracle.dequant_w8a8_f16(oracle.igemm(A, B, threads=0), sa, sw)
    D = torch.zeros((M, N), dtype=torch.float16, device=dev())
    ig.w8a8_linear(T(A), T(B) if layout == ig.BM_B_KN else T(B.T), D, T(sa), T(sw), M, N, K, layout)
    assert_clean_status()
    got = D.cpu().numpy()
    assert np.isfinite(got.astype(np.float32)).all()
    assert ulp_diff_f16(got.view(np.uint16), want.view(np.uint16)) <= 1


def test_column_slab_written_in_place_with_wider_pitch():
    """N-split building block: a rank writes its column slab of a wider output (ld > N)."""
    M, N, K, N_total, n0 = 256, 256, 256, 768, 256
    A = oracle.gen_int8((M, K), 5, 1)
    B = oracle.gen_int8((K, N), 5, 2)
    sa, sw = oracle.gen_scales(M, 5, 3), oracle.gen_scales(N, 5, 4)
    full = torch.full((M, N_total), 7.0, dtype=torch.float16, device=dev())
    slab = full[:, n0:n0 + N]
    ig.w8a8_linear(T(A), T(B.T), slab, T(sa), T(sw), M, N, K, ig.BM_B_NK, ldd=N_total)
    assert_clean_status()
    got = full.cpu().numpy()
    want = oracle.dequant_w8a8_f16(oracle.igemm(A, B, threads=0), sa, sw)
    assert np.array_equal(got[:, n0:n0 + N].view(np.uint16), want.view(np.uint16))
    assert (got[:, :n0] == 7.0).all() and (got[:, n0 + N:] == 7.0).all()


def test_unaligned_output_pitch_takes_the_scalar_store_path():
    M, N, K = 130, 48, 64
    A = oracle.gen_int8((M, K), 6, 1)
    B = oracle.gen_int8((K, N), 6, 2)
    wide = torch.zeros((M, N + 3), dtype=torch.int32, device=dev())
    C = wide[:, 1:1 + N]                      # 4-byte aligned only, pitch 51 elements
    ig.igemm_i32(T(A), T(B.T), C, M, N, K, ig.BM_B_NK)
    assert_clean_status()
    got = wide.cpu().numpy()
    assert np.array_equal(got[:, 1:1 + N], oracle.igemm(A, B))
    assert (got[:, 0] == 0).all() and (got[:, 1 + N:] == 0).all()


def test_repeat_launches_are_bit_identical():
    """Race detector for the mbarrier pipeline: 50 launches, identical int32 every time."""
    M, N, K = 512, 768, 2048
    A, W = T(oracle.gen_int8((M, K), 8, 1)), T(oracle.gen_int8((N, K), 8, 2))
    first = None
    for i in range(50):
        C = torch.empty((M, N), dtype=torch.int32, device=dev())
        ig.igemm_i32(A, W, C, M, N, K, ig.BM_B_NK)
        if first is None:
            first = C.clone()
        else:
            assert torch.equal(C, first), f"launch {i} differs"
    assert_clean_status()


def test_pack_b_kn_to_nk():
    K, N = 200, 136
    B = oracle.gen_int8((K, N), 9, 1)
    W = ig.pack_b_kn_to_nk(T(B), K, N)
    assert np.array_equal(W.cpu().numpy(), B.T)


def test_bad_arguments_raise_on_the_gpu_too():
    a = torch.zeros((128, 40), dtype=torch.int8, device=dev())
    c = torch.zeros((128, 128), dtype=torch.int32, device=dev())
    with pytest.raises(ig.BmError, match="multiple of 16"):
        ig.igemm_i32(a, a, c, 128, 128, 40, ig.BM_B_NK)
    with pytest.raises(ig.BmError):
        ig.igemm_i32(a, a, c.float(), 128, 128, 32, ig.BM_B_NK)     # wrong output dtype


@pytest.mark.parametrize("M,N,K", [(2560, 2304, 512), (2500, 2256, 272), (2500, 2250, 144), (2816, 2048, 1024)])
def test_half_height_tiles_in_the_last_wave(M, N, K):
    """More 256x256 tiles than CTA pairs and a last wave at most half full: its tiles are computed as two
    128x256 halves by different pairs (M = 128 pair MMAs, 64 rows per CTA).  Same integers as with the
    half-height tail off, for every epilogue and both weight layouts, ragged edges included; canary rows
    catch stores outside the output."""
    from _gpu import options
    A = oracle.gen_int8((M, K), 12, 1)
    B = oracle.gen_int8((K, N), 12, 2)
    acc = oracle.igemm(A, B, threads=0)
    assert np.array_equal(run_i32(A, B, ig.BM_B_NK, guard=True), acc)
    if N % 16 == 0:
        assert np.array_equal(run_i32(A, B, ig.BM_B_KN, guard=True), acc)
    with options(tail_narrow=0):
        assert np.array_equal(run_i32(A, B, ig.BM_B_NK, guard=True), acc)
    Bd = T(B.T)
    sa, sw = oracle.gen_scales(M, 12, 3), oracle.gen_scales(N, 12, 4)
    D = torch.zeros((M, N), dtype=torch.float16, device=dev())
    ig.w8a8_linear(T(A), Bd, D, T(sa), T(sw), M, N, K, ig.BM_B_NK)
    assert_clean_status()
    want16 = oracle.dequant_w8a8_f16(acc, sa, sw).view(np.uint16)
    assert ulp_diff_f16(D.cpu().numpy().view(np.uint16), want16) <= 1
    F = torch.zeros((M, N), dtype=torch.float32, device=dev())
    ig.igemm_wmma(T(A), Bd, F, M, N, K, 0.01, 0.02, ig.BM_B_NK)
    assert_clean_status()
    assert np.array_equal(F.cpu().numpy().view(np.uint32), oracle.dequant_per_tensor(acc, 0.01, 0.02).view(np.uint32))



@pytest.mark.parametrize("group", [0, 3, 8])
def test_banded_tile_order_gives_the_same_integers(group):
    """Tile order of the pair kernel (plain, or bands of G row tiles — chosen for tall problems): the
    integers do not depend on it; 21 row tiles make the last band short for G = 8."""
    from _gpu import options
    M, N, K = 5300, 1000, 256
    A = oracle.gen_int8((M, K), 13, 1)
    B = oracle.gen_int8((K, N), 13, 2)
    with options(dense_group_m=group), forced_bn(256):
        got = run_i32(A, B, ig.BM_B_NK, guard=True)
    assert np.array_equal(got, oracle.igemm(A, B, threads=0))



def test_bounded_wait_gives_up_with_a_status_and_the_context_survives():
    """Failure detection without a fault: a wait nobody satisfies runs out after 2 ms, the kernel
    returns, the status word names the wait, and the next GEMM on the same context is correct."""
    import ctypes
    import time
    from bare_metal_b200 import _lib
    L = _lib.load()
    outcome = ctypes.c_int(0)
    t0 = time.time()
    assert L.bm_selftest_bounded_wait(2000, ctypes.byref(outcome)) == 0
    assert outcome.value == 2 and time.time() - t0 < 5.0
    assert ig.last_device_status() == 5          # DEV_TIMEOUT_DRAIN, recorded by the give-up path
    assert ig.last_device_status() == 0          # reading clears it
    A = oracle.gen_int8((128, 128), 1, 1)
    B = oracle.gen_int8((128, 128), 1, 2)
    assert np.array_equal(run_i32(A, B, ig.BM_B_NK), oracle.igemm(A, B))


@pytest.mark.parametrize("M,K", [(64, 4096), (300, 1040), (8, 16384), (5, 16)])
def test_per_token_quantisation_matches_the_reference_quantiser(M, K):
    """fp16 -> int8 with one scale per row: compute_scale + quantize_symmetric of the reference's
    bench (bench.cu:28-51) applied row by row, bit-exact; then the quantised rows feed the GEMM."""
    rng = np.random.default_rng(M * 1000 + K)
    x = (rng.standard_normal((M, K)) * rng.uniform(0.01, 30.0, (M, 1))).astype(np.float16)
    x[0, :] = 0                                   # an all-zero row keeps scale 1
    if M > 2:
        x[2, 3] = np.float16(65504.0)             # largest finite half
    q, s = ig.quantize_rows(T(x), M, K)
    assert_clean_status()
    x32 = x.astype(np.float32)
    want_s = np.array([oracle.compute_scale(x32[m]) for m in range(M)], np.float32)
    want_q = np.stack([oracle.quantize_symmetric(x32[m], want_s[m]) for m in range(M)])
    assert np.array_equal(s.cpu().numpy(), want_s)
    assert np.array_equal(q.cpu().numpy(), want_q)
    if K % 16 == 0 and K >= 64:
        N = 128
        W = oracle.gen_int8((N, K), 2, 2)
        sw = oracle.gen_scales(N, 2, 4)
        D = torch.zeros((M, N), dtype=torch.float16, device=dev())
        ig.w8a8_linear(q, T(W), D, s, T(sw), M, N, K)
        want = oracle.dequant_w8a8_f16(oracle.igemm_nt(want_q, W), want_s, sw)
        assert ulp_diff_f16(D.cpu().numpy().view(np.uint16), want.view(np.uint16)) <= 1
