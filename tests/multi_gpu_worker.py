"""Worker run under torchrun by test_gpu_multi.py (and by hand on 2 / 4 / 8 GPUs): the N-split layers on
real GPUs, every gather path, checked against the CPU oracle on every rank.  Exit code 0 = all checks
passed on this rank.  `--full` adds the full-size shapes of the 8192-token layer (sampled rows)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402
from bare_metal_b200 import igemm as ig  # noqa: E402
from bare_metal_b200 import nsplit  # noqa: E402


def check_dense(dev, rank, world, M, N, K, seed, rows=None, nccl=True):
    """Both gather paths of the dense layer; with `rows`, only those output rows are compared (full-size shapes)."""
    W = oracle.gen_int8((N, K), seed, 2)
    sw = oracle.gen_scales(N, seed, 4)
    Wt, swt = torch.from_numpy(W).to(dev), torch.from_numpy(sw).to(dev)
    W_slab, sw_slab, n0, n_len = nsplit.shard_weights(Wt, swt, world, rank)
    del Wt
    fused = nsplit.ColumnShardedLinear(W_slab, sw_slab, N, n0, mode="fused")
    equal = len({l for _, l in fused.slabs}) == 1
    base = nsplit.ColumnShardedLinear(W_slab, sw_slab, N, n0, mode="nccl") if (nccl and equal) else None
    for it in range(3):                      # different activations every time: a stale or early peer write would show
        X = oracle.gen_int8((M, K), seed + it, 1)
        sa = oracle.gen_scales(M, seed + it, 3)
        sel = np.arange(M) if rows is None else rows
        want = oracle.dequant_w8a8_f16(oracle.igemm_nt(np.ascontiguousarray(X[sel]), W), sa[sel], sw).view(np.uint16)
        Xd, sad = torch.from_numpy(X).to(dev), torch.from_numpy(sa).to(dev)
        full = fused.forward(Xd, sad)
        torch.cuda.synchronize()
        got = full.cpu().numpy().view(np.uint16)[sel]
        assert np.array_equal(got, want), f"rank {rank}: fused gather differs from the oracle ({M}x{N}x{K}, pass {it})"
        if base is not None and it == 0:
            blocks = base.forward(Xd, sad)
            torch.cuda.synchronize()
            got = nsplit.ColumnShardedLinear.blocks_to_row_major(blocks).cpu().numpy().view(np.uint16)[sel]
            assert np.array_equal(got, want), f"rank {rank}: NCCL gather path differs from the oracle ({M}x{N}x{K})"
    assert ig.last_device_status() == 0, "a bounded device-side wait gave up"


def check_dense_two_in_flight(dev, rank, world, M, N, K, seed, steps=6):
    """Independent steps alternating between two streams (lane = output buffer + barrier instance): every step has
    activations of its own, results are read only after all steps were enqueued, two steps back at most."""
    W = oracle.gen_int8((N, K), seed, 2)
    sw = oracle.gen_scales(N, seed, 4)
    W_slab, sw_slab, n0, n_len = nsplit.shard_weights(torch.from_numpy(W).to(dev), torch.from_numpy(sw).to(dev), world, rank)
    layer = nsplit.ColumnShardedLinear(W_slab, sw_slab, N, n0, mode="fused")
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    Xs = [oracle.gen_int8((M, K), seed + 100 + i, 1) for i in range(steps)]
    sas = [oracle.gen_scales(M, seed + 100 + i, 3) for i in range(steps)]
    Xd = [torch.from_numpy(x).to(dev) for x in Xs]
    sad = [torch.from_numpy(a).to(dev) for a in sas]
    torch.cuda.synchronize()
    kept = {}
    for i in range(steps):
        lane = i & 1
        out = layer.forward_fused(Xd[i], sad[i], lane=lane, stream=streams[lane])
        if i >= steps - 2:                   # the last result of each lane is still valid after the loop
            kept[i] = out
        else:                                # earlier ones: copy on the lane's stream before the lane is reused
            with torch.cuda.stream(streams[lane]):
                kept[i] = out.clone()
    torch.cuda.synchronize()
    for i, out in kept.items():
        want = oracle.dequant_w8a8_f16(oracle.igemm_nt(Xs[i], W), sas[i], sw).view(np.uint16)
        assert np.array_equal(out.cpu().numpy().view(np.uint16), want), f"rank {rank}: step {i} of two in flight differs"
    assert ig.last_device_status() == 0, "a bounded device-side wait gave up"


def check_sparse(dev, rank, world, M, N, K, seed, rows=None):
    """2:4-sparse weights, N-split: local sparse GEMM + peer-store gather (and the NCCL path for equal slabs)."""
    comp, nib = oracle.gen_sparse_rows(N, K, seed, 5)
    sw = oracle.gen_scales(N, seed, 4)
    Wdense = oracle.decompress_rows(comp, nib)
    c_slab, m_slab, sw_slab, n0, n_len = nsplit.shard_sparse_weights(
        torch.from_numpy(comp).to(dev), torch.from_numpy(nib).to(dev), torch.from_numpy(sw).to(dev), world, rank)
    tiled = ig.sp_pack_meta(m_slab, ig.BM_META_ROWS, n_len, K)
    packed = ig.sp_pack_weights(c_slab, m_slab, ig.BM_META_ROWS, n_len, K) if M <= 64 else None   # decode: packed blocks
    push = nsplit.ColumnShardedSparseLinear(c_slab, tiled, sw_slab, N, n0, mode="push", W_packed_slab=packed)
    equal = len({l for _, l in push.slabs}) == 1
    for it in range(3):
        X = oracle.gen_int8((M, K), seed + it, 1)
        sa = oracle.gen_scales(M, seed + it, 3)
        sel = np.arange(M) if rows is None else rows
        want = oracle.dequant_w8a8_f16(oracle.igemm_nt(np.ascontiguousarray(X[sel]), Wdense), sa[sel], sw).view(np.uint16)
        Xd, sad = torch.from_numpy(X).to(dev), torch.from_numpy(sa).to(dev)
        full = push.forward(Xd, sad)
        torch.cuda.synchronize()
        got = full.cpu().numpy().view(np.uint16)[sel]
        assert np.array_equal(got, want), f"rank {rank}: sparse push gather differs from the oracle ({M}x{N}x{K}, pass {it})"
        if equal and it == 0:
            blocks = nsplit.ColumnShardedSparseLinear(c_slab, tiled, sw_slab, N, n0, mode="nccl").forward(Xd, sad)
            torch.cuda.synchronize()
            got = nsplit.ColumnShardedLinear.blocks_to_row_major(blocks).cpu().numpy().view(np.uint16)[sel]
            assert np.array_equal(got, want), f"rank {rank}: sparse NCCL gather differs from the oracle ({M}x{N}x{K})"
    assert ig.last_device_status() == 0, "a bounded device-side wait gave up"


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    full = "--full" in sys.argv
    try:
        # equal slabs, multiples of 128; then a tall ragged-M case
        check_dense(dev, rank, world, 512, 1024 * world, 1024, 0)
        check_dense(dev, rank, world, 300, 256 * world, 512, 10)
        # ragged split in the proportions of the gate+up projection (22016 columns over 8 GPUs = 2752 each,
        # not a multiple of 128): 344 columns per rank on average, slabs of 336 / 352
        check_dense(dev, rank, world, 777, 344 * world, 640, 20)
        # enough tiles for several waves of CTA pairs and a partly filled last one
        check_dense(dev, rank, world, 2304, 2560 * world, 256, 30)
        # two independent steps in flight on two streams
        check_dense_two_in_flight(dev, rank, world, 1024, 512 * world, 512, 35)
        # 2:4-sparse layers: decode shapes (1 and 64 tokens; 3584 channels per rank at full size) and a prefill chunk
        check_sparse(dev, rank, world, 1, 448 * world, 1024, 40)
        check_sparse(dev, rank, world, 64, 448 * world, 2048, 50)
        check_sparse(dev, rank, world, 300, 280 * world, 512, 60)
        if full:
            rows = np.array([0, 1, 127, 128, 4095, 4096, 8191])
            # the 8192-token layer's largest projection, split as the workload says (2752 columns per rank at 8)
            check_dense(dev, rank, world, 8192, 22016, 4096, 70, rows=rows, nccl=False)
            check_dense(dev, rank, world, 4096, 4096, 4096, 80, rows=rows[:5], nccl=False)
            check_sparse(dev, rank, world, 64, 28672, 8192, 90, rows=np.array([0, 1, 31, 63]))
        dist.barrier()
        print(f"rank {rank}: ok", flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
