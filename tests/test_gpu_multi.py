"""N-split layers on 2 real GPUs (skipped on a single-GPU box): the NCCL all-gather baseline, the gather
fused into the dense GEMM's epilogue (paced peer TMA stores) on equal and ragged slabs, and the 2:4-sparse
layers with their peer-store gather, all against the CPU oracle."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_nsplit_two_gpus():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "multi_gpu_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert r.stdout.count(": ok") == 2


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_linkprobe_runs_clean_on_two_gpus():
    """The peer-store / load-interference probe behind the gather's pacing: runs to the end, its bounded waits
    never give up (status word 0), and paced peer stores leave the operand loads at speed where unpaced ones do not."""
    import re
    import bare_metal_b200 as bm
    exe = bm._build.build_host()[3]
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "done" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
    assert "mix status word: 0" in r.stdout
    loads = {m.group(1).strip(): float(m.group(2)) for m in
             re.finditer(r"MIX (.+?)\s+kernel .*?loads: avg \d+ us -> (\d+) GB/s", r.stdout)}
    assert loads["loads + remote TMA stores paced to 620 GB/s"] > 1.5 * loads["loads + remote TMA stores"]
