"""N-split (column-sharded) W8A8 linear layers across the GPUs of one box.

The reference is single-GPU; this is the B200 form of "large GEMMs are partitioned by weight
columns, only the output is exchanged".  Rank r owns output columns [n0, n0 + n_len) — the rows
n0.. of W[N x K] and the matching slice of the per-channel scales — and the full activations.

Ways to assemble the output on every rank:
  * "nccl"   local GEMM, then `all_gather_into_tensor`: result laid out [world, M, n_len]
             (rank-major column blocks); the baseline, equal slabs only.
  * "fused"  dense layers: the GEMM epilogue itself stores each finished box of the slab into the
             row-major [M x N] output of EVERY rank through peer-mapped symmetric memory
             (bm_w8a8_f16_gather; stores that cross NVLink are paced below the link rate),
             followed by a group barrier; no separate gather pass.  Ragged slabs are fine.
  * "push"   2:4-sparse layers: the sparse GEMM writes the slab into the rank's own [M x N]
             output, a copy kernel (bm_gather_slab_f16) stores it to the peers, then the barrier.

Output buffers of the fused / push paths are symmetric memory, two per (M, device), used in turn.
A rank's call i+2 writes the buffer that call i returned; it is ordered behind the barrier of call
i+1, which every rank enqueues after whatever it enqueued to read result i.  So: consume a result
on the stream it was produced on (or order the other stream before the next call), and do not
keep it across more than one further call of the same layer.

Two steps in flight: `forward_fused(..., lane=0 or 1)` names the pair of output buffers AND the
barrier instance of the call, so independent steps (different micro-batches) may run on two streams,
lane 0 on one and lane 1 on the other — the GEMM of one step then overlaps the NVLink tail and the
barrier of the other.  Calls of one lane must be ordered on one stream; every rank must issue the
same lanes in the same order; the rule above holds per lane (a lane's call i+2 reuses the buffer of
its call i, behind the lane's barrier i+1), so read a result on its lane's stream before that
lane's next call is enqueued, or order the reader before it.

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


def shard_sparse_weights(W_comp, W_meta_rows, sw_full, world: int, rank: int):
    """Row slab of 2:4-compressed weights (values [N x K/2], per-row position bytes [N x K/8]) and
    scales for `rank`.  Slabs are cut on multiples of 128 rows where N allows it (whole tiles of the
    sparse kernel), else on multiples of 16."""
    n_total = W_comp.shape[0]
    align = 128 if n_total % (128 * world) == 0 else 16
    n0, n_len = shard_columns(n_total, world, rank, align)
    sl = slice(n0, n0 + n_len)
    return W_comp[sl].contiguous(), W_meta_rows[sl].contiguous(), sw_full[sl].contiguous(), n0, n_len


class GroupBarrier:
    """Barrier across the ranks of a group for the step after a peer-store gather: one small kernel per rank
    (bm_peer_barrier) that signals the peers through flag words in symmetric memory and waits for theirs, ordered
    on the stream behind the kernels whose stores it publishes.  All layers of a group share one instance; every
    rank must call it the same number of times in the same order — a rank that makes one call more than its peers
    waits for a round that never comes, until the kernel's 1 s limit ends the wait (status code 7), so never let
    a per-rank clock or a per-rank condition decide how many steps a rank runs.  The round number lives on the device, so the
    call may be recorded in a CUDA graph.  `hdl.barrier()` of torch's symmetric memory does the same job at a
    higher cost (measured 9.5 us against 6 us per step on two B200s)."""
    _cache = {}

    def __init__(self, group, device):     # collective: every rank of the group constructs it at the same point
        import torch.distributed._symmetric_memory as symm_mem
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.flags = symm_mem.empty((64,), dtype=torch.int32, device=device)
        self.flags.zero_()
        self.hdl = symm_mem.rendezvous(self.flags, group)
        torch.cuda.synchronize(device)
        self.hdl.barrier()                                   # every rank's flags are zero before the first round
        torch.cuda.synchronize(device)
        self.ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in self.hdl.buffer_ptrs])

    @classmethod
    def of(cls, group, device, lane: int = 0):
        """The group's barrier of `lane`: lanes are independent instances (own flags, own round counter), one per
        stream that runs steps of its own."""
        key = (id(group), str(device), lane)
        if key not in cls._cache:
            cls._cache[key] = cls(group, device)
        return cls._cache[key]

    def __call__(self, stream=None):
        from . import _lib
        rc = _lib.load().bm_peer_barrier(self.ptrs, self.world, self.rank, _stream_handle(stream))
        _lib.check(rc, "bm_peer_barrier")


def _stream_handle(stream):
    """cudaStream_t of `stream` (a torch stream, a raw handle, or None = torch's current stream)."""
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)


class _Sharded:
    """What the dense and the sparse layer share: slab bookkeeping, symmetric output buffers, barrier."""

    def __init__(self, n_total: int, n0: int, n_len: int, group, mode: str, modes: tuple):
        if mode not in modes:
            raise ValueError(f"mode must be one of {modes}")
        self.n_total, self.n0, self.n_len = n_total, n0, n_len
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.mode = mode
        self._sym = {}
        self._turn = {}
        lens = [None] * self.world
        dist.all_gather_object(lens, (self.n0, self.n_len), group=self.group)
        self.slabs = lens
        if sum(l for _, l in lens) != n_total:
            raise ValueError(f"column slabs {lens} do not cover N = {n_total}")
        if mode == "nccl" and len({l for _, l in lens}) != 1:
            raise ValueError("the NCCL all-gather path needs equal slabs; use the peer-store path for ragged splits")

    def _symmetric(self, M, device, lane=None):
        """The symmetric [M x N_total] output to fill next, its handle and the slab pointers.  Every lane owns two
        buffers, used in turn (lane None is lane 0); a lane's pair is allocated at its first use — a collective
        step, like everything else here done by all ranks in the same order."""
        key = (M, str(device), lane or 0)
        if key not in self._sym:
            import torch.distributed._symmetric_memory as symm_mem
            pair = []
            for _ in range(2):
                buf = symm_mem.empty((M, self.n_total), dtype=torch.float16, device=device)
                hdl = symm_mem.rendezvous(buf, self.group)
                pair.append((buf, hdl, self._peer_slab_pointers(hdl)))   # + the slab's first column in every rank's buffer
            self._sym[key] = pair
            self._turn[key] = 0
        turn = self._turn[key]
        self._turn[key] = turn ^ 1
        return self._sym[key][turn]

    def _peer_slab_pointers(self, hdl):
        col_bytes = self.n0 * 2
        return (ctypes.c_void_p * self.world)(*[int(p) + col_bytes for p in hdl.buffer_ptrs])

    @staticmethod
    def blocks_to_row_major(blocks):
        """[world, M, n_len] -> [M, world * n_len] (one extra pass; the peer-store paths do not need it)."""
        w, M, n = blocks.shape
        return blocks.permute(1, 0, 2).reshape(M, w * n)


class ColumnShardedLinear(_Sharded):
    """D[M x N] = half(float(X W^T) * sa[m] * sw[n]) with W's rows (output columns) split over ranks.

    `gemm` is the local slab GEMM, (X, W_slab, D_slab_view, sa, sw_slab, M, n_len, K, ldd) -> None;
    it defaults to the sm_100a kernel behind the C ABI.  (The CPU tests of the sharding and gather
    logic inject a checker-based one; the product never does.)
    """

    def __init__(self, W_slab, sw_slab, n_total: int, n0: int, group=None, mode: str = "nccl",
                 gemm: Optional[Callable] = None):
        super().__init__(n_total, n0, W_slab.shape[0], group, mode, ("nccl", "fused"))
        self.W, self.sw = W_slab, sw_slab
        self.K = W_slab.shape[1]
        self._gemm = gemm

    # ---- local GEMM ------------------------------------------------------------------------
    def _local(self, X, sa, D_view, ldd):
        M = X.shape[0]
        if self._gemm is not None:
            self._gemm(X, self.W, D_view, sa, self.sw, M, self.n_len, self.K, ldd)
            return
        from . import igemm
        igemm.w8a8_linear(X, self.W, D_view, sa, self.sw, M, self.n_len, self.K, igemm.BM_B_NK, ldd=ldd)

    def forward_local(self, X, sa, out=None):
        """The rank's slab alone, [M x n_len] (no exchange): the GEMM-only leg of a scaling measurement."""
        M = X.shape[0]
        if out is None:
            out = torch.empty((M, self.n_len), dtype=torch.float16, device=X.device)
        self._local(X, sa, out, self.n_len)
        return out

    # ---- nccl baseline ---------------------------------------------------------------------
    def forward_nccl(self, X, sa, out=None, local=None):
        """Returns [world, M, n_len] (rank-major column blocks)."""
        M = X.shape[0]
        local = self.forward_local(X, sa, local)
        if out is None:
            out = torch.empty((self.world, M, self.n_len), dtype=torch.float16, device=X.device)
        dist.all_gather_into_tensor(out.view(self.world * M, self.n_len), local, group=self.group)
        return out

    # ---- fused GEMM + gather ---------------------------------------------------------------
    def forward_fused(self, X, sa, barrier: bool = True, lane=None, stream=None):
        """Returns this rank's row-major [M x N] output, complete once the trailing barrier has run
        (see the module text for how long it stays valid).  `lane` (0 / 1) picks the lane's pair of output
        buffers and its barrier instance, for two steps in flight on two streams; `stream` is where the step is enqueued
        (default: torch's current stream)."""
        from . import _lib, igemm
        M = X.shape[0]
        buf, _, slab_ptrs = self._symmetric(M, X.device, lane)
        L = _lib.load()
        rc = L.bm_w8a8_f16_gather(X.data_ptr(), self.W.data_ptr(), slab_ptrs, self.world, self.rank, sa.data_ptr(),
                                  self.sw.data_ptr(), M, self.n_len, self.K, self.n_total, igemm.BM_B_NK,
                                  _stream_handle(stream))
        _lib.check(rc, "bm_w8a8_f16_gather")
        if barrier:     # every rank's stores are complete before anyone reads
            GroupBarrier.of(self.group, X.device, lane or 0)(stream)
        return buf

    def forward(self, X, sa):
        return self.forward_fused(X, sa) if self.mode == "fused" else self.forward_nccl(X, sa)


class ColumnShardedSparseLinear(_Sharded):
    """The same layer with 2:4-sparse weights: rank r holds rows [n0, n0 + n_len) of the compressed
    weights W_comp[N x K/2], their position metadata in the kernel's tiled order (bm_sp_pack_meta of
    the slab) and the scales.  Decode shapes (a few tokens) and prefill shapes both go through
    bm_w8a8_sparse_f16, which picks its kernel by the token count.

    `gemm` as for the dense layer: (X, W_comp_slab, meta_slab, D_slab_view, sa, sw_slab, M, n_len, K, ldd).
    """

    def __init__(self, W_comp_slab, W_meta_tiled_slab, sw_slab, n_total: int, n0: int, group=None,
                 mode: str = "push", gemm: Optional[Callable] = None, W_packed_slab=None):
        super().__init__(n_total, n0, W_comp_slab.shape[0], group, mode, ("nccl", "push"))
        self.W_comp, self.W_meta, self.sw = W_comp_slab, W_meta_tiled_slab, sw_slab
        self.K = W_comp_slab.shape[1] * 2
        self._gemm = gemm
        # optional: the slab in the library's packed block form (igemm.sp_pack_weights).  Decode shapes (<= 64
        # tokens) then stream whole blocks and the slab's rows are dealt to ALL CTA slots in multiples of 8 —
        # what keeps every SM busy when a rank's slab is only a few dozen 128-row tiles.
        self.W_packed = W_packed_slab

    def _local(self, X, sa, D_view, ldd):
        M = X.shape[0]
        if self._gemm is not None:
            self._gemm(X, self.W_comp, self.W_meta, D_view, sa, self.sw, M, self.n_len, self.K, ldd)
            return
        from . import igemm
        if self.W_packed is not None and M <= 64:
            igemm.w8a8_sparse_linear_packed(X, self.W_packed, D_view, sa, self.sw, M, self.n_len, self.K, ldd=ldd)
        else:
            igemm.w8a8_sparse_linear(X, self.W_comp, self.W_meta, D_view, sa, self.sw, M, self.n_len, self.K, ldd=ldd)

    def forward_local(self, X, sa, out=None):
        M = X.shape[0]
        if out is None:
            out = torch.empty((M, self.n_len), dtype=torch.float16, device=X.device)
        self._local(X, sa, out, self.n_len)
        return out

    def forward_nccl(self, X, sa, out=None, local=None):
        M = X.shape[0]
        local = self.forward_local(X, sa, local)
        if out is None:
            out = torch.empty((self.world, M, self.n_len), dtype=torch.float16, device=X.device)
        dist.all_gather_into_tensor(out.view(self.world * M, self.n_len), local, group=self.group)
        return out

    def forward_push(self, X, sa, barrier: bool = True):
        """Local sparse GEMM into the rank's own [M x N] output, peer stores of the slab, barrier."""
        from . import _lib
        M = X.shape[0]
        buf, _, slab_ptrs = self._symmetric(M, X.device)
        self._local(X, sa, buf[:, self.n0:self.n0 + self.n_len], self.n_total)
        rc = _lib.load().bm_gather_slab_f16(slab_ptrs, self.world, self.rank, M, self.n_len, self.n_total,
                                            torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "bm_gather_slab_f16")
        if barrier:
            GroupBarrier.of(self.group, X.device)()
        return buf

    def forward(self, X, sa):
        return self.forward_push(X, sa) if self.mode == "push" else self.forward_nccl(X, sa)


def measure_peer_store_bandwidth(device, group=None, rows: int = 8192, cols_per_rank: int = 4096, timeit=None) -> float:
    """GB/s a rank receives while every rank of the group pushes an fp16 slab of `rows x cols_per_rank` to all the
    others at the same time with the library's copy kernel (bm_gather_slab_f16), pacing switched off: what plain
    peer stores achieve on this box, in this run.  Collective: call it on every rank.  `timeit(fn)` must return
    the milliseconds one call of fn(i) takes, measured on the device across the group."""
    from . import _lib
    group = group if group is not None else dist.group.WORLD
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    if world < 2:
        raise ValueError("needs at least two ranks")
    n_total = cols_per_rank * world
    probe = _Sharded(n_total, rank * cols_per_rank, cols_per_rank, group, "push", ("push",))
    buf, hdl, ptrs = probe._symmetric(rows, device)
    L = _lib.load()
    old = _lib.get_option("gather_gbs")
    _lib.set_option("gather_gbs", 0)
    try:
        def push(i):
            _lib.check(L.bm_gather_slab_f16(ptrs, world, rank, rows, cols_per_rank, n_total,
                                            torch.cuda.current_stream().cuda_stream), "bm_gather_slab_f16")
        ms = timeit(push)
    finally:
        _lib.set_option("gather_gbs", old)
    GroupBarrier.of(group, device)()
    torch.cuda.synchronize(device)
    return 2.0 * rows * cols_per_rank * (world - 1) / (ms * 1e-3) / 1e9
