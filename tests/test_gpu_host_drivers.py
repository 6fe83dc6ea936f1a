"""The C++ bench drivers (host code above the C ABI) run as processes and are read through the
restated gate parser, the way the reference's R tooling drives its benches."""
import pytest

import bare_metal_b200 as bm
from bare_metal_b200 import gate

pytestmark = pytest.mark.gpu


def test_dense_driver_correctness_and_stdout_contract():
    bench = bm._build.build_host()[0]
    r = gate.run_bench(bench, [512, 512, 512])
    assert r["returncode"] == 0, r["err"][-2000:]
    text = "\n".join(r["out"])
    assert "igemm_cpasync (LDGSTS)" in text and "FAIL" not in text
    assert sum("PASS" in ln for ln in r["out"]) == 3            # per-tensor, per-channel and FP16-in checks
    oq = gate.parse_throughput(r["out"], match="igemm_online_quant")
    assert oq["throughput"] > 0 and oq["unit"] == "GFLOPS"
    p = gate.parse_throughput(r["out"], match="igemm_cpasync")   # the gate's match string for the dense kernel
    assert p["ms"] is not None and p["throughput"] > 0 and p["unit"] == "TOPS"
    pc = gate.parse_throughput(r["out"], match="igemm_perchannel")
    assert pc["throughput"] > 0
    # odd sizes are rounded up to multiples of 16 exactly as the reference bench does
    r2 = gate.run_bench(bench, [100, 200, 90])
    assert r2["returncode"] == 0 and any("C[112×208]" in ln for ln in r2["out"])


def test_sparse_driver_max_abs_zero_and_stdout_contract():
    bench_sparse = bm._build.build_host()[1]
    r = gate.run_bench(bench_sparse, [1024, 1024, 1024])
    assert r["returncode"] == 0, r["err"][-2000:]
    assert any("igemm_sparse_tiled (INT8)" in ln and "PASS" in ln and "max_abs=0.00e+00" in ln for ln in r["out"])
    p = gate.parse_throughput(r["out"], match="igemm_sparse_tiled", value_label="dense-equiv GFLOPS")
    e = gate.parse_throughput(r["out"], match="igemm_sparse_tiled", value_label="eff GFLOPS")
    assert p["throughput"] > 0 and abs(p["throughput"] / e["throughput"] - 2.0) < 0.01
    # argument rule of the reference bench: K % 32, M/N % 16
    bad = gate.run_bench(bench_sparse, [256, 256, 48])
    assert bad["returncode"] == 1


def test_persistent_driver_line_and_check():
    """Twin of the reference's bench_persistent: its one line in the reference's format (label, ms, eff GFLOPS,
    grid) and — beyond what the reference driver does — the output checked against the exact CPU product."""
    bench_persistent = bm._build.build_host()[2]
    r = gate.run_bench(bench_persistent, [512, 512, 512])
    assert r["returncode"] == 0, r["err"][-2000:]
    assert any("igemm_sparse_tiled_persistent" in ln and "PASS" in ln and "max_abs=0.00e+00" in ln for ln in r["out"])
    p = gate.parse_throughput(r["out"], match="igemm_sparse_tiled_persistent", value_label="eff GFLOPS")
    assert p["ms"] is not None and p["throughput"] > 0
    assert any("(grid=16x1)" in ln for ln in r["out"])            # 4 x 4 tiles of 128 x 128
    assert gate.run_bench(bench_persistent, [256, 256, 48])["returncode"] == 1


def test_gate_runs_the_shipped_b200_baselines(tmp_path):
    """The gate end to end on the GPU: the shipped baselines file (its dense entries; the sparse driver's exact CPU
    product at 4096^3 takes half a minute), the C++ driver, one JSONL row per config.
    Boxes differ, so the verdict is not asserted — only that every config was measured and recorded."""
    import json
    bm._build.build_host()
    rec = str(tmp_path / "gate_runs.jsonl")
    rc = gate.main(["--record", rec, "--tolerance", "0.5", "--kernel", "bare-metal_b200/csrc/igemm_dense_pair.cuh"])
    rows = [json.loads(l) for l in open(rec)]
    cfg = [r for r in rows if r["type"] == "config"]
    assert rc in (0, 1) and len(cfg) == 2 and all(r["measured"] and r["throughput"] > 0 for r in cfg)
    assert rows[-1]["type"] == "run" and rows[-1]["total"] == 2 and rows[-1]["skipped"] == 0
