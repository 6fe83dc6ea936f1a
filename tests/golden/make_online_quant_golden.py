"""Golden vectors for the FP16-in GEMM: outputs of the REFERENCE kernel itself.

Runs on a machine with a GPU.  `make -C oracle ref_cubins` (on a machine that has the reference
checkout) compiles kernels/gemm/igemm/igemm_online_quant.cu, unmodified, to
oracle/_ref/cubins/igemm_online_quant.sm_86.cubin (the file name the reference bench opens; sm_100a code); this script loads that cubin through the CUDA driver
API, launches `igemm_online_quant` with the geometry the reference bench uses
(bench.cu:529-536: grid ((N+127)/128, (M+127)/128), block 256, no dynamic shared memory) on seeded
inputs and stores inputs and outputs in tests/golden/online_quant_reference.npz.  The CPU tests
compare the restatement in oracle/igemm_oracle.c with these bits.

    python tests/golden/make_online_quant_golden.py [output.npz]
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
CUBIN = os.path.join(ROOT, "oracle", "_ref", "cubins", "igemm_online_quant.sm_86.cubin")

# sizes inside the domain the reference bench exercises: M, N multiples of 128, K of 32
CASES = [(128, 128, 64, 1), (256, 384, 160, 2), (256, 256, 512, 3)]


def inputs(M, N, K, seed):
    """Uniform [-1, 1) like the bench's fill_random, plus larger values in later K tiles so that the
    re-used first-tile factors clamp (QUANTIZE_TILE_FAST) and one all-zero first tile (inv = 1)."""
    rng = np.random.default_rng(seed)
    A = (rng.random((M, K), dtype=np.float32) * 2 - 1)
    B = (rng.random((K, N), dtype=np.float32) * 2 - 1)
    A[:, 32:] *= rng.choice(np.array([1.0, 1.0, 1.0, 1.7], np.float32), size=(M, K - 32))
    B[32:, :] *= rng.choice(np.array([1.0, 1.0, 2.5], np.float32), size=(K - 32, N))
    if M > 128:
        A[128:256, :32] = 0.0
    return A.astype(np.float16), B.astype(np.float16)


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "online_quant_reference.npz")
    cu = C.CDLL("libcuda.so.1")
    torch.cuda.init()
    torch.zeros(1, device="cuda")                                    # primary context current on this thread

    def ck(rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} failed with CUresult {rc}")

    mod, fn = C.c_void_p(), C.c_void_p()
    ck(cu.cuModuleLoad(C.byref(mod), CUBIN.encode()), "cuModuleLoad")
    ck(cu.cuModuleGetFunction(C.byref(fn), mod, b"igemm_online_quant"), "cuModuleGetFunction")
    out = {}
    for idx, (M, N, K, seed) in enumerate(CASES):
        A, B = inputs(M, N, K, seed)
        dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
        dC = torch.zeros((M, N), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        pa, pb, pc = C.c_void_p(dA.data_ptr()), C.c_void_p(dB.data_ptr()), C.c_void_p(dC.data_ptr())
        m, n, k = C.c_int(M), C.c_int(N), C.c_int(K)
        params = (C.c_void_p * 6)(*[C.cast(C.byref(x), C.c_void_p) for x in (pa, pb, pc, m, n, k)])
        ck(cu.cuLaunchKernel(fn, (N + 127) // 128, (M + 127) // 128, 1, 256, 1, 1, 0, None, params, None),
           "cuLaunchKernel")
        ck(cu.cuCtxSynchronize(), "cuCtxSynchronize")
        out[f"A{idx}"] = A.view(np.uint16)
        out[f"B{idx}"] = B.view(np.uint16)
        out[f"C{idx}"] = dC.cpu().numpy()
    out["shapes"] = np.array([c[:3] for c in CASES], np.int32)
    ck(cu.cuModuleUnload(mod), "cuModuleUnload")
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
