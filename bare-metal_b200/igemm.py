"""Host-side mirror of the reference's kernel interface for the INT8 GEMM path.

Each function keeps the NAME and ARGUMENT ORDER of the reference kernel symbol it stands in
for (kernels/gemm/igemm/*.cu: operand pointers, output pointer, M, N, K, scales) and
forwards, through the C ABI in include/bm_igemm.h, to the sm_100a kernels.  Arguments are
torch CUDA tensors used as device buffers; nothing is computed on the host and nothing
falls back to PyTorch: a missing library or a rejected argument raises.

Reference symbol                              -> function here
  igemm_wmma, igemm_tiled, igemm_register_blocked, igemm_pipelined,
  igemm_pipelined_cpasync(_bk64), igemm_8warp(_256, _256x256, _tribuf)
                                              -> igemm_wmma (aliases below)
  igemm_persistent                            -> igemm_persistent (tile counter ignored)
  igemm_pipelined_cpasync_perchannel          -> igemm_pipelined_cpasync_perchannel
  igemm_sparse_tiled (+ _persistent)          -> igemm_sparse_tiled
plus the entry points the B200 workloads add: igemm_i32, w8a8_linear, sparse weights.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import BM_B_KN, BM_B_NK, BM_META_REF, BM_META_REF_F16, BM_META_ROWS, BM_META_ROWS_F16, BM_META_TILED, BmError  # noqa: F401


def _dev(t: torch.Tensor, dtype, name: str) -> int:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise BmError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise BmError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise BmError(f"{name} must be contiguous")
    return t.data_ptr()


def _out(t: torch.Tensor, dtype, name: str) -> int:
    """Output buffers may be strided views (a column slab of a wider matrix): unit inner stride."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise BmError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise BmError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if t.dim() == 2 and t.stride(1) != 1:
        raise BmError(f"{name} must have unit stride along its rows")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


# --------------------------------------------------------------------------------------
# reference kernel ABI: (A, B, C, M, N, K, scale_a, scale_b) — igemm.cu:52-59
# --------------------------------------------------------------------------------------
def igemm_wmma(A, B, C, M, N, K, scale_a, scale_b, b_layout=BM_B_KN):
    """C[M,N] fp32 = float(A[M,K] @ B[K,N]) * (scale_a * scale_b)."""
    L = _lib.load()
    rc = L.bm_igemm_i8_f32(_dev(A, torch.int8, "A"), _dev(B, torch.int8, "B"), _out(C, torch.float32, "C"),
                           M, N, K, scale_a, scale_b, C.stride(0) if C.dim() == 2 else N, b_layout, _stream())
    _lib.check(rc, "bm_igemm_i8_f32")
    return C


igemm_tiled = igemm_register_blocked = igemm_pipelined = igemm_pipelined_cpasync = igemm_wmma
igemm_pipelined_cpasync_bk64 = igemm_8warp = igemm_8warp_256 = igemm_8warp_256x256 = igemm_8warp_tribuf = igemm_wmma


def igemm_persistent(A, B, C, M, N, K, scale_a, scale_b, tile_counter=None):
    """igemm_persistent.cu:60-69.  The reference's atomic tile counter is accepted and left
    untouched: tile scheduling here is static inside the persistent kernel."""
    return igemm_wmma(A, B, C, M, N, K, scale_a, scale_b)


def igemm_pipelined_cpasync_perchannel(A, B, C, M, N, K, per_channel_scale, per_channel_zero_point,
                                       b_layout=BM_B_KN):
    """C[m,n] = (float(acc) - float(zp[n])) * scale[n] — igemm_pipelined_cpasync_perchannel.cu:48-56."""
    L = _lib.load()
    rc = L.bm_igemm_i8_f32_perchannel(_dev(A, torch.int8, "A"), _dev(B, torch.int8, "B"),
                                      _out(C, torch.float32, "C"), M, N, K,
                                      _dev(per_channel_scale, torch.float32, "scale"),
                                      _dev(per_channel_zero_point, torch.int32, "zero_point"),
                                      C.stride(0) if C.dim() == 2 else N, b_layout, _stream())
    _lib.check(rc, "bm_igemm_i8_f32_perchannel")
    return C


def igemm_sparse_tiled(A_comp, B, C, meta, M, N, K, scale_a, scale_b):
    """C[M,N] fp32 = float(A_2:4[M,K] @ B[K,N]) * (scale_a*scale_b); A compressed [M,K/2] with the
    reference's uint32 metadata — igemm_sparse_tiled.cu:88-96."""
    L = _lib.load()
    meta_ptr = _dev(meta.view(torch.int32) if meta.dtype != torch.int32 else meta, torch.int32, "meta")
    rc = L.bm_igemm_sparse_f32(_dev(A_comp, torch.int8, "A_comp"), _dev(B, torch.int8, "B"),
                               _dev(C, torch.float32, "C"), meta_ptr, M, N, K, scale_a, scale_b, _stream())
    _lib.check(rc, "bm_igemm_sparse_f32")
    return C


def igemm_sparse_tiled_persistent(A_comp, B, C, meta, M, N, K, scale_a, scale_b, tile_counter=None):
    return igemm_sparse_tiled(A_comp, B, C, meta, M, N, K, scale_a, scale_b)


# --------------------------------------------------------------------------------------
# FP16-in kernels: (A_f16, B_f16, C, M, N, K) — igemm_online_quant.cu:144-150
# --------------------------------------------------------------------------------------
_oq_workspace = {}


def igemm_online_quant(A, B, C, M, N, K, col_block=128, workspace=None):
    """C[M,N] fp32 = block-quantised int8 product of fp16 A[M,K] and B[K,N]: one factor per 128-row
    block of A and per `col_block` columns of B, taken from the first 32 of K (the reference's
    QUANTIZE_TILE / QUANTIZE_TILE_FAST).  `workspace` (uint8 CUDA tensor) holds the int8 copies; one
    per device is kept and grown when it is not given."""
    L = _lib.load()
    need = L.bm_online_quant_workspace_bytes(M, N, K)
    if workspace is None:
        key = A.device.index
        workspace = _oq_workspace.get(key)
        if workspace is None or workspace.numel() < need:
            workspace = torch.empty(need, dtype=torch.uint8, device=A.device)
            _oq_workspace[key] = workspace
    rc = L.bm_online_quant_gemm_f32(_dev(A, torch.float16, "A"), _dev(B, torch.float16, "B"),
                                    _dev(C, torch.float32, "C"), M, N, K, col_block,
                                    _dev(workspace, torch.uint8, "workspace"), workspace.numel(), _stream())
    _lib.check(rc, "bm_online_quant_gemm_f32")
    return C


igemm_online_quant_inplace = igemm_online_quant_bankfree = igemm_warp_specialized = igemm_online_quant


def igemm_online_quant_bf_128x256(A, B, C, M, N, K, workspace=None):
    """igemm_online_quant_bf_128x256.cu:258-264: 256-column blocks of B share a factor."""
    return igemm_online_quant(A, B, C, M, N, K, 256, workspace)


# --------------------------------------------------------------------------------------
# FP16 2:4 GEMM: (A_compressed, B, C, metadata, M, N, K) — hgemm_sparse_tiled.cu:122-129
# --------------------------------------------------------------------------------------
def hgemm_sparse_tiled(A_comp, B, C, meta, M, N, K, meta_format=BM_META_REF_F16):
    """C[M,N] fp32 = A_2:4[M,K] @ B[K,N]; A_comp fp16 [M,K/2], B fp16, metadata in the reference's
    uint32 format (kernels/gemm/hgemm_sparse/sparse_meta.h), per-row bytes or the tiled order."""
    L = _lib.load()
    if meta.dtype == torch.uint8:
        meta_ptr = _dev(meta, torch.uint8, "meta")
    else:
        meta_ptr = _dev(meta.view(torch.int32) if meta.dtype != torch.int32 else meta, torch.int32, "meta")
    rc = L.bm_hgemm_sparse_f32(_dev(A_comp, torch.float16, "A_comp"), _dev(B, torch.float16, "B"),
                               _out(C, torch.float32, "C"), meta_ptr, meta_format, M, N, K,
                               C.stride(0) if C.dim() == 2 else N, _stream())
    _lib.check(rc, "bm_hgemm_sparse_f32")
    return C


def hgemm_sparse_naive(A_comp, B, C, M, N, K):
    """hgemm_sparse_naive.cu: the fixed pattern — kept positions {0,1} in every group (metadata 0x4444...)."""
    count = (M // 16) * (K // 16) * 8
    meta = torch.full((count,), 0x44444444, dtype=torch.int32, device=A_comp.device)
    return hgemm_sparse_tiled(A_comp, B, C, meta, M, N, K)


# --------------------------------------------------------------------------------------
# entry points of the B200 workloads
# --------------------------------------------------------------------------------------
def igemm_i32(A, B, C, M, N, K, b_layout=BM_B_KN):
    """Raw int32 accumulators C[M,N] = A[M,K] @ B (B[K,N], or W[N,K] with BM_B_NK)."""
    L = _lib.load()
    rc = L.bm_igemm_i8_i32(_dev(A, torch.int8, "A"), _dev(B, torch.int8, "B"), _out(C, torch.int32, "C"),
                           M, N, K, C.stride(0) if C.dim() == 2 else N, b_layout, _stream())
    _lib.check(rc, "bm_igemm_i8_i32")
    return C


def w8a8_linear(X, W, D, sa, sw, M, N, K, w_layout=BM_B_NK, ldd=None):
    """D[M,N] fp16 = half_rn(float(X @ W^T) * (sa[m] * sw[n])); W is [N,K] (or [K,N] with BM_B_KN)."""
    L = _lib.load()
    if ldd is None:
        ldd = D.stride(0) if D.dim() == 2 else N
    rc = L.bm_w8a8_f16(_dev(X, torch.int8, "X"), _dev(W, torch.int8, "W"), D.data_ptr() if _check_f16(D) else 0,
                       _dev(sa, torch.float32, "sa"), _dev(sw, torch.float32, "sw"), M, N, K, ldd, w_layout, _stream())
    _lib.check(rc, "bm_w8a8_f16")
    return D


def _check_f16(D) -> bool:
    if not D.is_cuda or D.dtype != torch.float16:
        raise BmError("D must be a CUDA float16 tensor")
    return True


def quantize_rows(X_f16, M, K):
    """Per-token dynamic quantisation of fp16 activations: returns (int8 [M,K], fp32 scale [M])."""
    L = _lib.load()
    _check_f16(X_f16)
    if not X_f16.is_contiguous():
        raise BmError("X must be contiguous")
    q = torch.empty((M, K), dtype=torch.int8, device=X_f16.device)
    s = torch.empty(M, dtype=torch.float32, device=X_f16.device)
    _lib.check(L.bm_quantize_rows_f16(X_f16.data_ptr(), q.data_ptr(), s.data_ptr(), M, K, _stream()),
               "bm_quantize_rows_f16")
    return q, s


def pack_b_kn_to_nk(B_kn, K, N):
    L = _lib.load()
    W = torch.empty((N, K), dtype=torch.int8, device=B_kn.device)
    _lib.check(L.bm_pack_b_kn_to_nk(_dev(B_kn, torch.int8, "B"), W.data_ptr(), K, N, _stream()), "bm_pack_b_kn_to_nk")
    return W


def prune_2_4(W, R, K):
    """Magnitude-prune W[R,K] int8 to 2:4 along K; returns (W_comp[R,K/2] int8, meta_rows[R,K/8] uint8)."""
    L = _lib.load()
    comp = torch.empty((R, K // 2), dtype=torch.int8, device=W.device)
    meta = torch.empty((R, K // 8), dtype=torch.uint8, device=W.device)
    rc = L.bm_prune_2_4_i8(_dev(W, torch.int8, "W"), comp.data_ptr(), meta.data_ptr(), R, K, _stream())
    _lib.check(rc, "bm_prune_2_4_i8")
    return comp, meta


def sp_pack_meta(meta, meta_format, R, K):
    """Re-tile 2:4 position metadata (reference uint32 words or per-row nibble bytes) once."""
    L = _lib.load()
    nbytes = L.bm_sp_meta_tiled_bytes(R, K)
    tiled = torch.empty(nbytes, dtype=torch.uint8, device=meta.device)
    if not meta.is_cuda or not meta.is_contiguous():
        raise BmError("meta must be a contiguous CUDA tensor")
    _lib.check(L.bm_sp_pack_meta(meta.data_ptr(), meta_format, tiled.data_ptr(), R, K, _stream()), "bm_sp_pack_meta")
    return tiled


def igemm_sparse_i32(A_comp, meta, meta_format, B, C, M, N, K, b_layout=BM_B_KN):
    L = _lib.load()
    rc = L.bm_igemm_sparse_i32(_dev(A_comp, torch.int8, "A_comp"), meta.data_ptr(), meta_format,
                               _dev(B, torch.int8, "B"), _out(C, torch.int32, "C"), M, N, K,
                               C.stride(0) if C.dim() == 2 else N, b_layout, _stream())
    _lib.check(rc, "bm_igemm_sparse_i32")
    return C


def w8a8_sparse_i32(X, W_comp, W_meta_tiled, C, M, N, K):
    L = _lib.load()
    rc = L.bm_w8a8_sparse_i32(_dev(X, torch.int8, "X"), _dev(W_comp, torch.int8, "W_comp"),
                              _dev(W_meta_tiled, torch.uint8, "W_meta"), _out(C, torch.int32, "C"), M, N, K,
                              C.stride(0) if C.dim() == 2 else N, _stream())
    _lib.check(rc, "bm_w8a8_sparse_i32")
    return C


def w8a8_sparse_linear(X, W_comp, W_meta_tiled, D, sa, sw, M, N, K, ldd=None):
    L = _lib.load()
    _check_f16(D)
    if ldd is None:
        ldd = D.stride(0) if D.dim() == 2 else N
    rc = L.bm_w8a8_sparse_f16(_dev(X, torch.int8, "X"), _dev(W_comp, torch.int8, "W_comp"),
                              _dev(W_meta_tiled, torch.uint8, "W_meta"), D.data_ptr(),
                              _dev(sa, torch.float32, "sa"), _dev(sw, torch.float32, "sw"), M, N, K, ldd, _stream())
    _lib.check(rc, "bm_w8a8_sparse_f16")
    return D


def sp_pack_weights(W_comp, W_meta, meta_format, N, K):
    """One-time repack of 2:4 sparse weights (values + positions) into contiguous 20 KiB blocks."""
    L = _lib.load()
    packed = torch.empty(L.bm_sp_packed_weight_bytes(N, K), dtype=torch.uint8, device=W_comp.device)
    _lib.check(L.bm_sp_pack_weights(_dev(W_comp, torch.int8, "W_comp"), W_meta.data_ptr(), meta_format,
                                    packed.data_ptr(), N, K, _stream()), "bm_sp_pack_weights")
    return packed


def w8a8_sparse_i32_packed(X, W_packed, C, M, N, K):
    L = _lib.load()
    rc = L.bm_w8a8_sparse_i32_packed(_dev(X, torch.int8, "X"), _dev(W_packed, torch.uint8, "W_packed"),
                                     _out(C, torch.int32, "C"), M, N, K, C.stride(0) if C.dim() == 2 else N, _stream())
    _lib.check(rc, "bm_w8a8_sparse_i32_packed")
    return C


def w8a8_sparse_linear_packed(X, W_packed, D, sa, sw, M, N, K, ldd=None):
    L = _lib.load()
    _check_f16(D)
    if ldd is None:
        ldd = D.stride(0) if D.dim() == 2 else N
    rc = L.bm_w8a8_sparse_f16_packed(_dev(X, torch.int8, "X"), _dev(W_packed, torch.uint8, "W_packed"), D.data_ptr(),
                                     _dev(sa, torch.float32, "sa"), _dev(sw, torch.float32, "sw"), M, N, K, ldd,
                                     _stream())
    _lib.check(rc, "bm_w8a8_sparse_f16_packed")
    return D


def last_device_status() -> int:
    """Status word a bounded in-kernel wait sets when it gives up (0 = none); clears it."""
    import ctypes
    code = ctypes.c_int(0)
    _lib.check(_lib.load().bm_last_device_status(ctypes.byref(code)), "bm_last_device_status")
    return code.value
