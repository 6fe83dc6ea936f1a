"""N-split (column-sharded) W8A8 linear across the GPUs of one box.

The reference is single-GPU; this is the B200 form of "large GEMMs are partitioned by weight
columns, only the output is exchanged".  Rank r owns output columns [n0, n0 + n_len) — the rows
n0.. of W[N x K] and the matching slice of the per-channel scales — and the full activations.

Two ways to assemble the output on every rank:
  * "nccl"   local GEMM, then `all_gather_into_tensor`: result laid out [world, M, n_len]
             (rank-major column blocks); the baseline.
  * "fused"  the GEMM epilogue itself stores each finished box of the slab into the row-major
             [M x N] output of EVERY rank through peer-mapped symmetric memory
             (bm_w8a8_f16_gather), followed by a group barrier; no separate gather pass.

One process per GPU (torchrun); `torch.distributed` carries the rendezvous only.
"""
from __future__ import annotations

import ctypes
from typing import Callable, Optional

import torch
import torch.distributed as dist


def shard_columns(n_total: int, world: int, rank: int, align: int = 16) -> tuple[int, int]:
    """Contiguous column slab (first column, length) of rank `rank`: lengths differ by at most
    `align`, every slab starts on a multiple of `align` (16 keeps int8 rows 16-byte aligned)."""
    if n_total <= 0 or world <= 0 or not 0 <= rank < world:
        raise ValueError("bad shard request")
    units = -(-n_total // align)
    u0 = units * rank // world
    u1 = units * (rank + 1) // world
    n0 = min(u0 * align, n_total)
    n1 = min(u1 * align, n_total)
    return n0, n1 - n0


def shard_weights(W_full, sw_full, world: int, rank: int, align: int = 16):
    """Row slab of K-major weights W[N x K] and the matching scales for `rank`."""
    n0, n_len = shard_columns(W_full.shape[0], world, rank, align)
    return W_full[n0:n0 + n_len].contiguous(), sw_full[n0:n0 + n_len].contiguous(), n0, n_len


class ColumnShardedLinear:
    """D[M x N] = half(float(X W^T) * sa[m] * sw[n]) with W's rows (output columns) split over ranks.

    `gemm` is the local slab GEMM, (X, W_slab, D_slab_view, sa, sw_slab, M, n_len, K, ldd) -> None;
    it defaults to the sm_100a kernel behind the C ABI.  (The CPU tests of the sharding and gather
    logic inject a checker-based one; the product never does.)
    """

    def __init__(self, W_slab, sw_slab, n_total: int, n0: int, group=None, mode: str = "nccl",
                 gemm: Optional[Callable] = None):
        if mode not in ("nccl", "fused"):
            raise ValueError("mode must be 'nccl' or 'fused'")
        self.W, self.sw = W_slab, sw_slab
        self.n_total, self.n0, self.n_len = n_total, n0, W_slab.shape[0]
        self.K = W_slab.shape[1]
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.mode = mode
        self._gemm = gemm
        self._sym = {}
        lens = [None] * self.world
        dist.all_gather_object(lens, (self.n0, self.n_len), group=self.group)
        self.slabs = lens
        if sum(l for _, l in lens) != n_total:
            raise ValueError(f"column slabs {lens} do not cover N = {n_total}")
        if mode == "nccl" and len({l for _, l in lens}) != 1:
            raise ValueError("the NCCL all-gather path needs equal slabs; use mode='fused' for ragged splits")

    # ---- local GEMM ------------------------------------------------------------------------
    def _local(self, X, sa, D_view, ldd):
        M = X.shape[0]
        if self._gemm is not None:
            self._gemm(X, self.W, D_view, sa, self.sw, M, self.n_len, self.K, ldd)
            return
        from . import igemm
        igemm.w8a8_linear(X, self.W, D_view, sa, self.sw, M, self.n_len, self.K, igemm.BM_B_NK, ldd=ldd)

    # ---- nccl baseline ---------------------------------------------------------------------
    def forward_nccl(self, X, sa, out=None, local=None):
        """Returns [world, M, n_len] (rank-major column blocks)."""
        M = X.shape[0]
        if local is None:
            local = torch.empty((M, self.n_len), dtype=torch.float16, device=X.device)
        self._local(X, sa, local, self.n_len)
        if out is None:
            out = torch.empty((self.world, M, self.n_len), dtype=torch.float16, device=X.device)
        dist.all_gather_into_tensor(out.view(self.world * M, self.n_len), local, group=self.group)
        return out

    @staticmethod
    def blocks_to_row_major(blocks):
        """[world, M, n_len] -> [M, world * n_len] (one extra pass; the fused path does not need it)."""
        w, M, n = blocks.shape
        return blocks.permute(1, 0, 2).reshape(M, w * n)

    # ---- fused GEMM + gather ---------------------------------------------------------------
    def _symmetric(self, M, device):
        key = (M, str(device))
        if key not in self._sym:
            import torch.distributed._symmetric_memory as symm_mem
            buf = symm_mem.empty((M, self.n_total), dtype=torch.float16, device=device)
            hdl = symm_mem.rendezvous(buf, self.group)
            self._sym[key] = (buf, hdl)
        return self._sym[key]

    def forward_fused(self, X, sa):
        """Returns this rank's row-major [M x N] output, complete once the trailing barrier has run."""
        from . import _lib, igemm
        M = X.shape[0]
        buf, hdl = self._symmetric(M, X.device)
        col_bytes = self.n0 * 2
        ptrs = (ctypes.c_void_p * self.world)(*[int(p) + col_bytes for p in hdl.buffer_ptrs])
        L = _lib.load()
        rc = L.bm_w8a8_f16_gather(X.data_ptr(), self.W.data_ptr(), ptrs, self.world, sa.data_ptr(), self.sw.data_ptr(),
                                  M, self.n_len, self.K, self.n_total, igemm.BM_B_NK,
                                  torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "bm_w8a8_f16_gather")
        hdl.barrier()            # every rank's stores have been issued and completed before anyone reads
        return buf

    def forward(self, X, sa):
        return self.forward_fused(X, sa) if self.mode == "fused" else self.forward_nccl(X, sa)
