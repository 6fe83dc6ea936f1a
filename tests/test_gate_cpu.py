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


# ---- sample validity (bench_measure.R) -----------------------------------------------------------
def _state(clock=1650.0, throttle=(), temp=55.0):
    return {"gpu": {"clock_sm": clock, "clock_mem": 3996.0, "temp_c": temp, "power_w": 700.0, "pstate": "P0",
                    "throttle_hex": "0x0", "throttle": list(throttle), "util_gpu": 99.0, "util_mem": 40.0}}


def test_capture_gpu_state_parses_an_nvidia_smi_line():
    st = gate.capture_gpu_state(query=lambda: "1665, 3996, 48, 611.25, P0, 0x0000000000000004, 100, 37")
    assert st["gpu"]["clock_sm"] == 1665 and st["gpu"]["throttle"] == ["SwPowerCap"] and st["gpu"]["pstate"] == "P0"
    assert gate.capture_gpu_state(query=lambda: None) is None
    assert gate.capture_gpu_state(query=lambda: "1, 2, 3") is None


def test_validate_sample_in_the_reference_order():
    ok = _state()
    assert gate.validate_sample(0, 100.0, ok, ok) == {"ok": True, "reason": None}
    assert gate.validate_sample(3, 100.0, ok, ok)["reason"] == "crash(exit=3)"
    assert gate.validate_sample(0, None, ok, ok)["reason"] == "parse-fail"
    assert gate.validate_sample(0, 100.0, None, ok)["reason"] == "no-gpu-meta"
    capped = _state(throttle=["SwPowerCap"])
    assert gate.validate_sample(0, 100.0, ok, capped)["reason"].startswith("unfair(throttle active during run: SwPowerCap")
    assert gate.validate_sample(0, 100.0, capped, capped, {"allow_throttle": ["GpuIdle", "SwPowerCap"]})["ok"]
    assert gate.validate_sample(0, 100.0, ok, _state(clock=1200), {"min_clock_sm": 1300})["reason"].startswith("unfair(clock_sm=1200")
    # two-sided band of a clock-locked measurement
    assert gate.validate_sample(0, 100.0, ok, _state(clock=1700), clock_band=(1575, 1635))["reason"] == \
        "clock 1700 MHz outside band 1575-1635"
    assert gate.validate_sample(0, 100.0, ok, _state(clock=1605), clock_band=(1575, 1635))["ok"]


def test_collect_valid_samples_and_median():
    seq = iter([None, 90.0, 110.0, None, 100.0, 120.0])
    res = gate.collect_valid_samples(lambda: {"t": next(seq)}, lambda s: {"ok": s["t"] is not None, "reason": "parse-fail"},
                                     n_valid=3, max_attempts=10)
    assert res["complete"] and res["attempts"] == 5 and [s["t"] for s in res["samples"]] == [90.0, 110.0, 100.0]
    assert res["rejected"] == ["parse-fail", "parse-fail"]
    short = gate.collect_valid_samples(lambda: {"t": None}, lambda s: {"ok": False, "reason": "x"}, 2, 3)
    assert not short["complete"] and short["attempts"] == 3
    m = gate.report_median_metrics([90.0, 110.0, 100.0], [1.1, 0.9, 1.0], [1600, 1650, 1620])
    assert m["median_throughput"] == 100.0 and m["median_ms"] == 1.0 and (m["tput_lo"], m["tput_hi"]) == (90.0, 110.0)
    assert (m["clk_lo"], m["clk_hi"], m["n"]) == (1600, 1650, 3)


# ---- the wiring end to end: a fake bench (a shell script printing one bench-shaped line), a baselines file
# in the reference's schema, the gate's main() and the run record it leaves ---------------------------
def _fixture(tmp_path, throughput, baseline=1000, clock_lock=None):
    import json
    import os
    exe = tmp_path / "fake_bench"
    if throughput is not None:
        exe.write_text(f'#!/bin/sh\necho "  fixture 1.000 ms  {throughput} GFLOPS"\n')
        os.chmod(exe, 0o755)
    cfg = {"ms": 1.0, "gflops": baseline}
    if clock_lock is not None:
        cfg["clock_lock"] = clock_lock
    base = {"recorded_date": "fixture", "platform": "fixture", "default_valid_when": {"require_no_throttle": False},
            "kernels": {"kernels/fixture/fake.cu": {"exe": "fake_bench", "1_2": cfg, "3_4": dict(cfg)}}}
    path = tmp_path / "baselines.json"
    path.write_text(json.dumps(base))
    return str(path), str(tmp_path / "rec" / "gate_runs.jsonl")


def _rows(path):
    import json
    return [json.loads(l) for l in open(path)]


def test_gate_main_passes_fails_and_is_inconclusive(tmp_path, capsys):
    b, rec = _fixture(tmp_path, 1000)
    assert gate.main(["--baselines", b, "--record", rec]) == 0
    assert "RESULT: PASSED -- 2 of 2 config(s) measured" in capsys.readouterr().out
    rows = _rows(rec)
    assert [r["type"] for r in rows] == ["config", "config", "run"] and rows[0]["verdict"] == "OK" and rows[0]["measured"]
    assert rows[0]["throughput"] == 1000 and rows[0]["unit"] == "GFLOPS" and rows[2]["status"] == "PASSED"
    # a measured regression fails the run and is recapped above the verdict; the record is appended, never rewritten
    b, _ = _fixture(tmp_path, 850)
    assert gate.main(["--baselines", b, "--record", rec]) == 1
    out = capsys.readouterr().out
    assert "REGRESSION 85.0% of baseline" in out and "Configs behind this verdict" in out
    assert len(_rows(rec)) == 6 and _rows(rec)[-1]["regressions"] == 2
    # median of several samples goes through the same funnel
    b, _ = _fixture(tmp_path, 1200)
    assert gate.main(["--baselines", b, "--record", rec, "--samples", "3", "--kernel", "kernels/fixture/fake.cu"]) == 0
    assert _rows(rec)[-2]["verdict"] == "IMPROVED" and _rows(rec)[-2]["samples"] == 3
    # nothing measured: missing executable, or clock_lock configs without a locked GPU — exit 2, configs still counted
    (tmp_path / "fake_bench").unlink()
    assert gate.main(["--baselines", b, "--record", rec]) == 2
    assert "INCONCLUSIVE -- 0 of 2 config(s) measured (2 skipped)" in capsys.readouterr().out
    b, _ = _fixture(tmp_path, 1000, clock_lock=1605)
    assert gate.main(["--baselines", b, "--record", rec]) == 2
    assert _rows(rec)[-2]["msg"].startswith("SKIPPED (clock_lock 1605 MHz")
    assert gate.main(["--baselines", b, "--record", rec, "--clock-locked", "1710"]) == 2
    assert gate.main(["--baselines", b, "--list"]) == 0 and "[clock_lock 1605 MHz]" in capsys.readouterr().out
    assert gate.main(["--baselines", b, "--kernel", "nope"]) == 1


def test_shipped_b200_baselines_follow_the_schema():
    import json
    with open(gate.DEFAULT_BASELINES) as f:
        base = json.load(f)
    assert "SwPowerCap" in base["default_valid_when"]["allow_throttle"]
    for kernel, entry in base["kernels"].items():
        assert entry["exe"].startswith("../host/bin/")
        for cfg, d in entry.items():
            if cfg == "exe":
                continue
            assert len(cfg.split("_")) == 3 and d["ms"] > 0 and (d.get("tops") or d.get("gflops")) > 0 and d["match"]
            assert "clock_lock" not in d
