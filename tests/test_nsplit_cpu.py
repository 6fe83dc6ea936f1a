"""Host-side logic of the N-split linear on CPU: shard planner, and the gather path run as two
gloo ranks with the CPU checker standing in for the GEMM kernel."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from bare_metal_b200 import nsplit


def test_shard_columns_cover_and_align():
    for n_total, world in ((4096, 8), (22016, 8), (22016, 4), (12288, 2), (28672, 8), (100, 3), (16, 4)):
        slabs = [nsplit.shard_columns(n_total, world, r) for r in range(world)]
        assert slabs[0][0] == 0
        for (a0, alen), (b0, _) in zip(slabs, slabs[1:]):
            assert a0 + alen == b0 and a0 % 16 == 0
        assert slabs[-1][0] + slabs[-1][1] == n_total
    assert nsplit.shard_columns(22016, 8, 0) == (0, 2752)          # the gate+up slab named in the workload
    with pytest.raises(ValueError):
        nsplit.shard_columns(64, 4, 4)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, N, K = 48, 128, 96
        X = oracle.gen_int8((M, K), 0, 1)
        W = oracle.gen_int8((N, K), 0, 2)
        sa, sw = oracle.gen_scales(M, 0, 3), oracle.gen_scales(N, 0, 4)
        Wt, swt = torch.from_numpy(W), torch.from_numpy(sw)
        W_slab, sw_slab, n0, n_len = nsplit.shard_weights(Wt, swt, world, rank)

        def cpu_gemm(Xt, Ws, D, sat, sws, M_, n_, K_, ldd):
            acc = oracle.igemm_nt(Xt.numpy(), Ws.numpy(), threads=1)
            D.copy_(torch.from_numpy(oracle.dequant_w8a8_f16(acc, sat.numpy(), sws.numpy())))

        layer = nsplit.ColumnShardedLinear(W_slab, sw_slab, N, n0, mode="nccl", gemm=cpu_gemm)
        blocks = layer.forward(torch.from_numpy(X), torch.from_numpy(sa))
        full = nsplit.ColumnShardedLinear.blocks_to_row_major(blocks).numpy()
        want = oracle.dequant_w8a8_f16(oracle.igemm_nt(X, W, threads=1), sa, sw)
        ok = np.array_equal(full.view(np.uint16), want.view(np.uint16)) and layer.slabs == [
            nsplit.shard_columns(N, world, r) for r in range(world)]
        # a ragged split is refused on the all-gather path
        try:
            nsplit.ColumnShardedLinear(Wt[: 64 + 16 * rank].contiguous(), swt[: 64 + 16 * rank].contiguous(),
                                       64 * 2 + 16, 0 if rank == 0 else 64, mode="nccl", gemm=cpu_gemm)
            ragged_refused = False
        except ValueError:
            ragged_refused = True
        # the 2:4-sparse layer shares the sharding logic: slabs cut on 16 rows here, values + per-row positions
        # + scales sliced together, the checker's sparse product standing in for the kernel
        Ns, Ks = 96, 64
        comp, nib = oracle.gen_sparse_rows(Ns, Ks, 0, 5)
        sws = oracle.gen_scales(Ns, 0, 6)
        Xs = oracle.gen_int8((M, Ks), 0, 7)
        c_slab, m_slab, sw_s, n0s, n_lens = nsplit.shard_sparse_weights(torch.from_numpy(comp), torch.from_numpy(nib),
                                                                       torch.from_numpy(sws), world, rank)

        def cpu_sparse_gemm(Xt, Wc, Wm, D, sat, swt_, M_, n_, K_, ldd):
            dense = oracle.decompress_rows(Wc.numpy(), Wm.numpy())
            acc = oracle.igemm_nt(Xt.numpy(), dense, threads=1)
            D.copy_(torch.from_numpy(oracle.dequant_w8a8_f16(acc, sat.numpy(), swt_.numpy())))

        sp = nsplit.ColumnShardedSparseLinear(c_slab, m_slab, sw_s, Ns, n0s, mode="nccl", gemm=cpu_sparse_gemm)
        got = nsplit.ColumnShardedSparseLinear.blocks_to_row_major(sp.forward(torch.from_numpy(Xs), torch.from_numpy(sa))).numpy()
        want_s = oracle.dequant_w8a8_f16(oracle.igemm_nt(Xs, oracle.decompress_rows(comp, nib), threads=1), sa, sws)
        ok = ok and np.array_equal(got.view(np.uint16), want_s.view(np.uint16)) and (n0s, n_lens) == nsplit.shard_columns(Ns, world, rank)
        open(os.path.join(result_dir, f"rank{rank}"), "w").write(f"{int(ok)} {int(ragged_refused)}")
    finally:
        dist.destroy_process_group()


def test_two_rank_gather_equals_full_gemm(tmp_path):
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}").read() == "1 1"
