"""The C++ bench drivers (host code above the C ABI) run as processes and are read through the
restated gate parser, the way the reference's R tooling drives its benches."""
import pytest

import bare_metal_b200 as bm
from bare_metal_b200 import gate

pytestmark = pytest.mark.gpu


def test_dense_driver_correctness_and_stdout_contract():
    bench, _ = bm._build.build_host()
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
    _, bench_sparse = bm._build.build_host()
    r = gate.run_bench(bench_sparse, [1024, 1024, 1024])
    assert r["returncode"] == 0, r["err"][-2000:]
    assert any("igemm_sparse_tiled (INT8)" in ln and "PASS" in ln and "max_abs=0.00e+00" in ln for ln in r["out"])
    p = gate.parse_throughput(r["out"], match="igemm_sparse_tiled", value_label="dense-equiv GFLOPS")
    e = gate.parse_throughput(r["out"], match="igemm_sparse_tiled", value_label="eff GFLOPS")
    assert p["throughput"] > 0 and abs(p["throughput"] / e["throughput"] - 2.0) < 0.01
    # argument rule of the reference bench: K % 32, M/N % 16
    bad = gate.run_bench(bench_sparse, [256, 256, 48])
    assert bad["returncode"] == 1
