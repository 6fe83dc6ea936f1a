"""The Python restatement of the reference's stdout gate, on lines in the reference benches' format
(written here, not copied from the reference fixtures)."""
from bare_metal_b200 import gate

DENSE_OUT = """=== IGEMM Benchmark — INT8 Tensor Cores (sm_100a, tcgen05) ===
Matrix: C[4096×4096] = A[4096×4096] * B[4096×4096]  (INT8 in, INT32 accum, FP32 out)

Quantization: scale_a=0.007874  scale_b=0.007874
CPU reference skipped (matrix too large — use M<=512 for correctness check)

Performance (avg of 50 runs, 5 warmup):
  igemm_cpasync (LDGSTS dbuf)           0.071 ms   1935702.11 TOPS
  igemm_8warp_256 (128x256 cp.async)    0.070 ms   1963412.50 TOPS
  igemm_perchannel (asym dequant)       0.072 ms   1908876.00 TOPS
  INT8 Tensor Core peak                    --        4500000 TOPS  (theoretical)
""".splitlines()

SPARSE_OUT = """=== Sparse INT8 GEMM Benchmark ===
M=2048  N=2048  K=2048

  igemm_sparse_tiled (INT8)      PASS  (max_abs=0.00e+00  max_rel=0.00e+00)
  igemm_sparse_tiled                     0.021 ms    409,123 eff GFLOPS    818246 dense-equiv GFLOPS
""".splitlines()


def test_parse_throughput_dense_and_sparse_lines():
    r = gate.parse_throughput(DENSE_OUT, match="igemm_cpasync")
    assert r["ms"] == 0.071 and r["throughput"] == 1935702.11 and r["unit"] == "TOPS"
    assert gate.parse_throughput(DENSE_OUT, match="igemm_cpasync", pick="last")["line"] == r["line"]
    # the peak line has no "ms" token and is never picked
    assert gate.parse_throughput(DENSE_OUT, match="Tensor Core peak")["throughput"] is None
    # first vs last candidate when no match is given
    assert gate.parse_throughput(DENSE_OUT)["throughput"] == 1935702.11
    assert gate.parse_throughput(DENSE_OUT, pick="last")["throughput"] == 1908876.00
    # value_label picks the right column of a multi-number line (and strips thousands separators)
    s = gate.parse_throughput(SPARSE_OUT, match="igemm_sparse_tiled", value_label="dense-equiv GFLOPS")
    assert s["ms"] == 0.021 and s["throughput"] == 818246 and s["unit"] == "GFLOPS"
    e = gate.parse_throughput(SPARSE_OUT, match="igemm_sparse_tiled", value_label="eff GFLOPS")
    assert e["throughput"] == 409123
    # the PASS line carries no "ms": skipped even though it contains the match
    assert "PASS" not in s["line"]
    # section bracketing
    sec = ["=== A ===", "  k  1.0 ms  10 GFLOPS", "--- B ---", "  k  2.0 ms  20 GFLOPS"]
    assert gate.parse_throughput(sec, match="k", section="B")["throughput"] == 20
    assert gate.parse_throughput(sec, match="k", section="C")["line"] is None


def test_check_regression_buckets():
    base = {"tops": 1000.0}
    cur = lambda v, rc=0: {"returncode": rc, "throughput": v, "unit": "TOPS"}
    assert gate.check_regression(cur(1000), base, 0.1)["msg"].startswith("OK 100.0%")
    assert gate.check_regression(cur(880), base, 0.1)["is_reg"] is True
    assert gate.check_regression(cur(1200), base, 0.1)["msg"].startswith("IMPROVED")
    assert gate.check_regression(cur(1000, rc=1), base, 0.1)["msg"] == "CRASH (exit=1)"
    assert gate.check_regression(cur(0), base, 0.1)["msg"].startswith("NO_DATA")
    sk = gate.check_regression(cur(500), base, 0.1, unfair_reasons=["SwPowerCap"])
    assert sk.get("skipped") and not sk["is_reg"]
    # unit falls back across gflops / tops keys
    assert gate.check_regression({"throughput": 50, "unit": "GFLOPS"}, {"tops": 50}, 0.1)["msg"].startswith("OK")


def test_summarise_verdict_and_throttle_decode():
    assert gate.summarise_verdict(3, 3, 0, 0)["exit"] == 0
    assert gate.summarise_verdict(3, 2, 1, 1)["exit"] == 1
    v = gate.summarise_verdict(3, 0, 0, 3)
    assert v["exit"] == 2 and v["status"] == "INCONCLUSIVE"
    assert gate.decode_throttle(0x0004 | 0x0040) == ["SwPowerCap", "HwThermalSlowdown"]
    assert gate.decode_throttle(0) == []
