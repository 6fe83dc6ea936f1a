"""Worker run under torchrun by test_gpu_multi.py: N-split linear on real GPUs, both gather paths,
checked against the CPU oracle on every rank.  Exit code 0 = all checks passed on this rank."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402
from bare_metal_b200 import nsplit  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    try:
        for (M, N, K) in ((512, 1024 * world, 1024), (300, 256 * world, 512)):
            X = oracle.gen_int8((M, K), 0, 1)
            W = oracle.gen_int8((N, K), 0, 2)
            sa, sw = oracle.gen_scales(M, 0, 3), oracle.gen_scales(N, 0, 4)
            want = oracle.dequant_w8a8_f16(oracle.igemm_nt(X, W), sa, sw).view(np.uint16)
            Wt, swt = torch.from_numpy(W).to(dev), torch.from_numpy(sw).to(dev)
            W_slab, sw_slab, n0, n_len = nsplit.shard_weights(Wt, swt, world, rank)
            Xd, sad = torch.from_numpy(X).to(dev), torch.from_numpy(sa).to(dev)
            base = nsplit.ColumnShardedLinear(W_slab, sw_slab, N, n0, mode="nccl")
            blocks = base.forward(Xd, sad)
            torch.cuda.synchronize()
            got = nsplit.ColumnShardedLinear.blocks_to_row_major(blocks).cpu().numpy().view(np.uint16)
            assert np.array_equal(got, want), f"rank {rank}: NCCL gather path differs from the oracle"
            fused = nsplit.ColumnShardedLinear(W_slab, sw_slab, N, n0, mode="fused")
            for _ in range(2):                     # twice: buffers and barrier are reused
                full = fused.forward(Xd, sad)
                torch.cuda.synchronize()
                got = full.cpu().numpy().view(np.uint16)
                assert np.array_equal(got, want), f"rank {rank}: fused gather differs from the oracle"
        dist.barrier()
        print(f"rank {rank}: ok", flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
