"""The reference project's own bench programs, UNMODIFIED (compiled from its sources in place into
oracle/_ref by oracle/Makefile), run on top of libbm_igemm.so through the LD_PRELOAD cubin shim:
their cuModuleLoad / cuModuleGetFunction / cuLaunchKernel calls for the INT8 GEMM kernels are served
by the B200 launchers, and their own correctness checks and stdout contract are what is asserted."""
import os
import subprocess

import pytest

import bare_metal_b200 as bm
from bare_metal_b200 import gate

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")


def run_ref(name, args, tmp_path):
    exe = os.path.join(REF, name)
    if not os.path.exists(exe):
        pytest.skip("reference benches have not been built (oracle/Makefile target ref_bench)")
    env = dict(os.environ, LD_PRELOAD=bm._build.build_shim())
    r = subprocess.run([exe, *map(str, args)], capture_output=True, text=True, timeout=300, env=env, cwd=tmp_path)
    return r.returncode, r.stdout.splitlines(), r.stderr


def test_unmodified_dense_bench(tmp_path):
    rc, out, err = run_ref("bench", [512, 512, 512], tmp_path)
    assert rc == 0, err[-2000:]
    text = "\n".join(out)
    # the bench's own checks (0.5 / 0.1 AND logic against its CPU references) for every served kernel
    for label in ("igemm_wmma", "igemm_tiled", "igemm_cpasync (LDGSTS)", "igemm_perchannel (asym)",
                  "igemm_8warp_256 (128x256)", "igemm_persistent"):
        lines = [ln for ln in out if label in ln and ("PASS" in ln or "FAIL" in ln)]
        assert lines and all("PASS" in ln for ln in lines), (label, lines)
    assert "FAIL" not in text
    # the gate's match string for the dense kernel finds a timing line
    p = gate.parse_throughput(out, match="igemm_cpasync")
    assert p["ms"] is not None and p["throughput"] > 0 and p["unit"] == "TOPS"
    # the FP16-in kernels (per-tile int8 quantisation) are served too: the bench's own check against
    # its fp32 SGEMM (bench.cu:540) and its timing lines
    for label in ("igemm_online_quant (FP16", "igemm_inplace (FP16", "igemm_bankfree (FP16", "igemm_warpspec (FP16"):
        lines = [ln for ln in out if label in ln and ("PASS" in ln or "FAIL" in ln)]
        assert lines and all("PASS" in ln for ln in lines), (label, lines)
    p = gate.parse_throughput(out, match="igemm_online_quant")
    assert p["ms"] is not None and p["throughput"] > 0 and p["unit"] == "GFLOPS"
    # kernels outside the path (fp16 HGEMM cubins) are skipped exactly as when their cubins are absent
    assert not any("hgemm" in ln and " ms" in ln for ln in out)


def test_unmodified_sparse_benches(tmp_path):
    rc, out, err = run_ref("bench_sparse", [1024, 1024, 1024], tmp_path)
    assert rc == 0, err[-2000:]
    assert any("igemm_sparse_tiled (INT8)" in ln and "PASS" in ln and "max_abs=0.00e+00" in ln for ln in out)
    p = gate.parse_throughput(out, match="igemm_sparse_tiled", value_label="dense-equiv GFLOPS")
    assert p["throughput"] > 0
    rc, out, err = run_ref("bench_persistent", [1024, 1024, 1024], tmp_path)
    assert rc == 0, err[-2000:]
    p = gate.parse_throughput(out, match="igemm_sparse_tiled_persistent", value_label="eff GFLOPS")
    assert p["throughput"] > 0


def test_reference_kernels_recompiled_for_sm100a_are_the_baseline_we_beat(tmp_path):
    """The same unmodified bench binary twice at 4096^3: once loading the reference's own kernels
    (compiled for sm_100a into oracle/_ref/cubins), once served by this library through the shim.
    Both pass on a B200; the library has to be at least 10x faster on the gate's dense line."""
    cubins = os.path.join(REF, "cubins")
    exe = os.path.join(REF, "bench")
    if not os.path.isdir(cubins) or not os.path.exists(exe):
        pytest.skip("reference kernels / benches have not been built (oracle/Makefile ref_cubins, ref_bench)")
    r = subprocess.run([exe, "4096", "4096", "4096"], capture_output=True, text=True, timeout=600, cwd=cubins)
    assert r.returncode == 0, r.stderr[-2000:]
    theirs = gate.parse_throughput(r.stdout.splitlines(), match="igemm_cpasync")
    rc, out, err = run_ref("bench", [4096, 4096, 4096], tmp_path)
    assert rc == 0, err[-2000:]
    ours = gate.parse_throughput(out, match="igemm_cpasync")
    assert theirs["throughput"] > 0 and ours["throughput"] > 10 * theirs["throughput"], (theirs, ours)
    their_oq = gate.parse_throughput(r.stdout.splitlines(), match="igemm_online_quant")
    our_oq = gate.parse_throughput(out, match="igemm_online_quant")
    assert our_oq["throughput"] > 10 * their_oq["throughput"], (their_oq, our_oq)


def test_unmodified_fp16_sparse_bench_both_ways(tmp_path):
    """kernels/gemm/hgemm_sparse/bench.cu, unmodified: with the reference's own kernels (compiled for
    sm_100a) and served by this library through the shim.  Its three checks (fixed pattern naive + tiled,
    arbitrary pattern tiled; 0.1 / 0.1) pass both ways; the library is faster on its timing line."""
    exe = os.path.join(REF, "bench_hgemm_sparse")
    cubins = os.path.join(REF, "cubins")
    if not os.path.exists(exe) or not os.path.exists(os.path.join(cubins, "hgemm_sparse_tiled.sm_86.cubin")):
        pytest.skip("reference fp16 sparse bench / kernels have not been built")
    r = subprocess.run([exe, "1024", "1024", "1024"], capture_output=True, text=True, timeout=300, cwd=cubins)
    assert r.returncode == 0, r.stderr[-2000:]
    theirs = r.stdout.splitlines()
    rc, ours, err = run_ref("bench_hgemm_sparse", [1024, 1024, 1024], tmp_path)
    assert rc == 0, err[-2000:]
    for out in (theirs, ours):
        checks = [ln for ln in out if "PASS" in ln or "FAIL" in ln]
        assert sum("PASS" in ln for ln in checks) >= 3 and not any("FAIL" in ln for ln in checks), checks

    def tiled_ms(lines):
        row = [ln.split() for ln in lines if ln.strip().startswith("tiled ")]
        return float(row[-1][1])
    assert tiled_ms(ours) < tiled_ms(theirs), (tiled_ms(ours), tiled_ms(theirs))
