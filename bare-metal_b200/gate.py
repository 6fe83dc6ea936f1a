"""Python restatement of the reference's stdout-parsing regression gate, for driving the C++ bench
drivers (bare-metal_b200/host) the way the reference's R tooling drives its benches (R is absent
here).  Behaviour follows the R functions line for line:

  parse_throughput   R/cuasmR/R/bench_run.R:84-140     — pick a kernel's line, extract ms + value
  check_regression   R/cuasmR/R/bench_regression.R:28-77 — CRASH / SKIPPED / NO_DATA / REGRESSION / OK / IMPROVED
  summarise_verdict  scripts/bench/bench_regress.R:290-308 — exit 0 PASSED / 1 FAILED / 2 INCONCLUSIVE
  decode_throttle    R/cuasmR/R/bench_meta.R:41-64     — nvidia-smi throttle bitmask
  capture_gpu_state  R/cuasmR/R/bench_meta.R:204-227   — nvidia-smi snapshot (read-only query)
  classify_meta      R/cuasmR/R/bench_meta.R:245-310   — was the GPU in a fit state to be measured?
  validate_sample / collect_valid_samples / report_median_metrics
                     R/cuasmR/R/bench_measure.R:38-63,91-134 — per-sample verdict, N valid samples, median
  main               scripts/bench/bench_regress.R:399-640 — per-config loop over a baselines file in the
                     reference's schema (data/baselines.json:11-19), one append-only JSONL row per decided
                     config (bench_regress.R:311-380), exit code from summarise_verdict

    python -m bare_metal_b200.gate [--baselines FILE] [--tolerance 0.10] [--kernel KEY] [--list]
                                   [--samples N] [--clock-locked MHZ] [--record FILE]

Clock locking: configs carrying `clock_lock` are measured only when --clock-locked names the same
frequency, and then every sample's observed SM clock must lie inside the band — as in the reference.
This module never sets or resets a clock, power limit or any other GPU setting; it only reads them.
"""
from __future__ import annotations

import json
import os
import re
import subprocess
import sys
import time
from typing import Callable, Optional, Sequence

THROTTLE_BITS = {
    "GpuIdle": 0x0001, "ApplicationsClocksSet": 0x0002, "SwPowerCap": 0x0004, "HwSlowdown": 0x0008,
    "SyncBoost": 0x0010, "SwThermalSlowdown": 0x0020, "HwThermalSlowdown": 0x0040,
    "HwPowerBrakeSlowdown": 0x0080, "DisplayClocksSetting": 0x0100,
}
UNFAIR_THROTTLES = ("ApplicationsClocksSet", "SwPowerCap", "HwSlowdown", "SwThermalSlowdown",
                    "HwThermalSlowdown", "HwPowerBrakeSlowdown")


def decode_throttle(mask: int) -> list[str]:
    return [name for name, bit in THROTTLE_BITS.items() if mask & bit]


def parse_throughput(lines: Sequence[str], match: Optional[str] = None, section: Optional[str] = None,
                     value_label: Optional[str] = None, pick: str = "first") -> dict:
    """Select a kernel's line and extract its timing and throughput.

    Selection order: lines after a `section` header (a line whose trimmed form starts with === or
    ---) up to the next header; lines containing `match`; lines containing "ms"; lines carrying
    `value_label` if given, else a GFLOPS/TOPS token; then the first or last survivor.
    """
    if pick not in ("first", "last"):
        raise ValueError("pick must be 'first' or 'last'")
    na = {"ms": None, "throughput": None, "unit": None, "line": None}
    lines = list(lines)
    if section:
        in_sec, kept = False, []
        for ln in lines:
            if re.match(r"^(===|---)", ln.strip()):
                in_sec = section in ln
                continue
            if in_sec:
                kept.append(ln)
        lines = kept
    cand = [ln for ln in lines if not match or match in ln]
    cand = [ln for ln in cand if "ms" in ln]
    if value_label:
        cand = [ln for ln in cand if value_label in ln]
    else:
        cand = [ln for ln in cand if re.search(r"GFLOPS|TOPS", ln, re.I)]
    if not cand:
        return na
    line = cand[0] if pick == "first" else cand[-1]
    m = re.search(r"([0-9.]+)\s*ms", line)
    ms = float(m.group(1)) if m else None
    if value_label:
        m = re.search(r"([0-9][0-9,.]*)\s*" + re.escape(value_label), line, re.I)
        tp = float(m.group(1).replace(",", "")) if m else None
        u = re.search(r"(GFLOPS|TOPS)\b", value_label, re.I)
        unit = u.group(1).upper() if u else "GFLOPS"
    else:
        m = re.search(r"([0-9][0-9,.]*)\s*(GFLOPS|TOPS)", line, re.I)
        tp, unit = (float(m.group(1).replace(",", "")), m.group(2).upper()) if m else (None, None)
    return {"ms": ms, "throughput": tp, "unit": unit, "line": line}


def check_regression(current: dict, baseline: dict, tolerance: float, unfair_reasons: Sequence[str] = ()) -> dict:
    """current: returncode, throughput, unit; baseline: gflops / tops.  `unfair_reasons` non-empty
    means the GPU state made the sample incomparable (SKIPPED, never REGRESSION)."""
    rc = current.get("returncode")
    if rc is not None and rc != 0:
        return {"is_reg": True, "msg": f"CRASH (exit={rc})"}
    if unfair_reasons:
        return {"is_reg": False, "skipped": True, "msg": "SKIPPED (" + "; ".join(unfair_reasons) + ")"}
    unit = current.get("unit") or "GFLOPS"
    base = baseline.get(unit.lower()) or baseline.get("gflops") or baseline.get("tops") or 0
    cur = current.get("throughput") or 0
    if base == 0 or cur == 0:
        return {"is_reg": True, "msg": f"NO_DATA (baseline={base:g}, current={cur:g})"}
    ratio = cur / base
    detail = f"{ratio * 100:.1f}% of baseline ({cur:.0f} vs {base:.0f} {unit})"
    if ratio < 1.0 - tolerance:
        return {"is_reg": True, "msg": "REGRESSION " + detail}
    if ratio > 1.0 + tolerance:
        return {"is_reg": False, "msg": "IMPROVED " + detail}
    return {"is_reg": False, "msg": "OK " + detail}


def summarise_verdict(total: int, measured: int, regressions: int, skipped: int) -> dict:
    if regressions > 0:
        return {"status": "FAILED", "exit": 1,
                "msg": f"FAILED -- {regressions} regression(s) detected ({measured} of {total} config(s) measured)"}
    if measured < 1:
        return {"status": "INCONCLUSIVE", "exit": 2,
                "msg": f"INCONCLUSIVE -- 0 of {total} config(s) measured ({skipped} skipped); nothing was verified"}
    return {"status": "PASSED", "exit": 0,
            "msg": f"PASSED -- {measured} of {total} config(s) measured, all within tolerance ({skipped} skipped)"}


def run_bench(exe: str, args: Sequence[str], timeout: float = 120.0) -> dict:
    """Run a bench executable as the gate does (process boundary, stdout captured, 120 s limit,
    R/cuasmR/R/bench_run.R:35-48)."""
    try:
        r = subprocess.run([exe, *map(str, args)], capture_output=True, text=True, timeout=timeout)
        return {"returncode": r.returncode, "out": r.stdout.splitlines(), "err": r.stderr}
    except subprocess.TimeoutExpired as e:
        return {"returncode": 124, "out": (e.stdout or "").splitlines() if isinstance(e.stdout, str) else [], "err": "timeout"}


# ----------------------------------------------------------------------------------------------
# GPU state and sample validity
# ----------------------------------------------------------------------------------------------
NVIDIA_SMI_FIELDS = ("clocks.current.sm", "clocks.current.memory", "temperature.gpu", "power.draw", "pstate",
                     "clocks_throttle_reasons.active", "utilization.gpu", "utilization.memory")


def capture_gpu_state(index: int = 0, query: Optional[Callable[[], Optional[str]]] = None) -> Optional[dict]:
    """One nvidia-smi snapshot of GPU `index` (None when no GPU / no nvidia-smi).  `query` lets a test
    supply the CSV line instead of running nvidia-smi."""
    if query is None:
        def query():
            try:
                r = subprocess.run(["nvidia-smi", f"--id={index}", "--query-gpu=" + ",".join(NVIDIA_SMI_FIELDS),
                                    "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=20)
            except (OSError, subprocess.TimeoutExpired):
                return None
            return r.stdout.splitlines()[0] if r.returncode == 0 and r.stdout.strip() else None
    line = query()
    if not line:
        return None
    vals = [v.strip() for v in line.split(",")]
    if len(vals) != len(NVIDIA_SMI_FIELDS):
        return None
    raw = dict(zip(NVIDIA_SMI_FIELDS, vals))

    def num(k):
        try:
            return float(raw[k])
        except ValueError:
            return None
    try:
        mask = int(raw["clocks_throttle_reasons.active"], 16)
    except ValueError:
        mask = 0
    return {"gpu": {"clock_sm": num("clocks.current.sm"), "clock_mem": num("clocks.current.memory"),
                    "temp_c": num("temperature.gpu"), "power_w": num("power.draw"), "pstate": raw["pstate"],
                    "throttle_hex": raw["clocks_throttle_reasons.active"], "throttle": decode_throttle(mask),
                    "util_gpu": num("utilization.gpu"), "util_mem": num("utilization.memory")},
            "iso_time": time.strftime("%Y-%m-%dT%H:%M:%S%z")}


def classify_meta(pre: Optional[dict], post: Optional[dict], valid_when: Optional[dict] = None) -> dict:
    """ok True / False / None (no metadata), with the reasons a sample is not comparable."""
    if pre is None or post is None:
        return {"ok": None, "reasons": ["no GPU metadata captured"], "summary": "meta unavailable"}
    cfg = {"require_no_throttle": True, "allow_throttle": ["GpuIdle"], "min_clock_sm": None, "max_temp_c": None}
    cfg.update({k: v for k, v in (valid_when or {}).items() if k in cfg})
    reasons = []
    if cfg["require_no_throttle"]:
        bad = [t for t in dict.fromkeys(pre["gpu"]["throttle"] + post["gpu"]["throttle"]) if t not in cfg["allow_throttle"]]
        if bad:
            reasons.append("throttle active during run: " + ",".join(bad))
    if cfg["min_clock_sm"] is not None:
        clk = post["gpu"]["clock_sm"]
        if clk is None or clk < cfg["min_clock_sm"]:
            reasons.append(f"clock_sm={'NA' if clk is None else int(clk)} MHz < required {int(cfg['min_clock_sm'])} MHz")
    if cfg["max_temp_c"] is not None and post["gpu"]["temp_c"] is not None and post["gpu"]["temp_c"] > cfg["max_temp_c"]:
        reasons.append(f"temp={int(post['gpu']['temp_c'])}C > max {int(cfg['max_temp_c'])}C")
    g = post["gpu"]
    summary = (f"clk={g['clock_sm']}/{g['clock_mem']} MHz  temp={g['temp_c']}C  power={g['power_w']}W  pstate={g['pstate']}  "
               + ("throttle=[" + ",".join(g["throttle"]) + "]" if g["throttle"] else "throttle=none"))
    return {"ok": not reasons, "reasons": reasons, "summary": summary}


def validate_sample(rc, throughput, pre, post, valid_when: Optional[dict] = None,
                    clock_band: Optional[Sequence[float]] = None) -> dict:
    """Checks in the reference's order: exit status, parsed throughput, GPU state, two-sided clock band."""
    if rc is not None and rc != 0:
        return {"ok": False, "reason": f"crash(exit={int(rc)})"}
    if throughput is None:
        return {"ok": False, "reason": "parse-fail"}
    cls = classify_meta(pre, post, valid_when)
    if cls["ok"] is None:
        return {"ok": False, "reason": "no-gpu-meta"}
    if cls["ok"] is False:
        return {"ok": False, "reason": "unfair(" + ";".join(cls["reasons"]) + ")"}
    if clock_band is not None:
        clk = post["gpu"]["clock_sm"]
        if clk is None or clk < clock_band[0] or clk > clock_band[1]:
            return {"ok": False, "reason": f"clock {'NA' if clk is None else int(clk)} MHz outside band "
                                           f"{int(clock_band[0])}-{int(clock_band[1])}"}
    return {"ok": True, "reason": None}


def collect_valid_samples(sample_fn: Callable[[], dict], validate_fn: Callable[[dict], dict], n_valid: int,
                          max_attempts: int, on_sample: Optional[Callable] = None) -> dict:
    """Loop until `n_valid` samples pass `validate_fn` or `max_attempts` runs were made; valid samples are
    kept whole, reject reasons are listed."""
    samples, rejected, attempt = [], [], 0
    while len(samples) < n_valid and attempt < max_attempts:
        attempt += 1
        s = sample_fn()
        v = validate_fn(s)
        if v["ok"]:
            samples.append(s)
        else:
            rejected.append(v["reason"])
        if on_sample is not None:
            on_sample(attempt, bool(v["ok"]), s, v["reason"])
    return {"samples": samples, "rejected": rejected, "attempts": attempt, "complete": len(samples) >= n_valid}


def _median(xs):
    xs = sorted(x for x in xs if x is not None)
    if not xs:
        return None
    n = len(xs)
    return xs[n // 2] if n % 2 else 0.5 * (xs[n // 2 - 1] + xs[n // 2])


def report_median_metrics(throughput: Sequence[float], ms: Sequence[float], clk: Optional[Sequence[float]] = None) -> dict:
    tp = [t for t in throughput if t is not None]
    ck = [c for c in (clk or []) if c is not None]
    return {"median_throughput": _median(tp), "median_ms": _median(ms), "tput_lo": min(tp) if tp else None,
            "tput_hi": max(tp) if tp else None, "clk_lo": min(ck) if ck else None, "clk_hi": max(ck) if ck else None,
            "n": len(tp)}


# ----------------------------------------------------------------------------------------------
# the gate: baselines file -> runs -> verdicts -> run record
# ----------------------------------------------------------------------------------------------
PKG_DIR = os.path.dirname(os.path.abspath(__file__))
DEFAULT_BASELINES = os.path.join(PKG_DIR, "data", "baselines_b200.json")
RESERVED_KEYS = ("exe",)
CLOCK_LOCK_BAND_MHZ = 30


def run_benchmark(exe: str, args: Sequence[str], baseline_cfg: Optional[dict] = None, gpu_index: int = 0) -> dict:
    """One bench process from its own directory (the reference benches open cubins by relative name), GPU
    state captured before and after, the config's line parsed with its match / section / value_label."""
    exe = os.path.abspath(exe)
    pre = capture_gpu_state(gpu_index)
    cwd = os.getcwd()
    try:
        os.chdir(os.path.dirname(exe))
        r = run_bench(exe, args, timeout=120)
    finally:
        os.chdir(cwd)
    post = capture_gpu_state(gpu_index)
    cfg = baseline_cfg or {}
    parsed = parse_throughput(r["out"], match=cfg.get("match"), section=cfg.get("section"),
                              value_label=cfg.get("value_label"), pick="first")
    if parsed["throughput"] is None:
        parsed = parse_throughput(r["out"], value_label=cfg.get("value_label"), pick="first")
    return {"returncode": r["returncode"], "raw_output": "\n".join(r["out"]), "meta_pre": pre, "meta_post": post,
            "ms": parsed["ms"], "throughput": parsed["throughput"], "unit": parsed["unit"],
            "matched_line": parsed["line"]}


def unfair_reasons(current: dict, valid_when: Optional[dict]) -> list:
    """Why this sample cannot be compared with a baseline (empty = fair).  Without GPU metadata nothing is
    held against the sample, as in the reference's CI runs."""
    cls = classify_meta(current.get("meta_pre"), current.get("meta_post"), valid_when)
    return [] if cls["ok"] in (True, None) else cls["reasons"]


def append_jsonl_row(path: str, row: dict) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "a") as f:
        f.write(json.dumps(row, default=str) + "\n")


def meta_digest(current: Optional[dict]) -> Optional[dict]:
    if not current or not current.get("meta_post"):
        return None
    g = current["meta_post"]["gpu"]
    return {"clock_sm": g["clock_sm"], "clock_mem": g["clock_mem"], "temp_c": g["temp_c"], "power_w": g["power_w"],
            "pstate": g["pstate"], "throttle": list(g["throttle"])}


def measure_median(exe, cfg_args, baseline_cfg, valid_when, n_valid, max_attempts, clock_band=None, warmup=1):
    """Median of `n_valid` valid samples (the reference's locked-measurement loop, usable unlocked too).
    Without a clock band a sample taken where no GPU metadata exists (no nvidia-smi) is judged on its exit
    status and parsed throughput alone; with a band the metadata is required, as in the reference."""
    for _ in range(warmup):
        run_benchmark(exe, cfg_args, baseline_cfg)

    def validate(m):
        if clock_band is None and (m["meta_pre"] is None or m["meta_post"] is None):
            if m["returncode"] not in (None, 0):
                return {"ok": False, "reason": f"crash(exit={int(m['returncode'])})"}
            return {"ok": m["throughput"] is not None, "reason": None if m["throughput"] is not None else "parse-fail"}
        return validate_sample(m["returncode"], m["throughput"], m["meta_pre"], m["meta_post"], valid_when, clock_band)

    res = collect_valid_samples(lambda: run_benchmark(exe, cfg_args, baseline_cfg), validate, n_valid, max_attempts)
    if not res["complete"]:
        return {"status": "insufficient",
                "msg": f"INSUFFICIENT ({len(res['samples'])}/{n_valid} valid in {res['attempts']} tries; rejects: "
                       + ", ".join(res["rejected"][:6]) + ")"}
    tputs = [s["throughput"] for s in res["samples"]]
    med = report_median_metrics(tputs, [s["ms"] for s in res["samples"]],
                                [s["meta_post"]["gpu"]["clock_sm"] if s["meta_post"] else None for s in res["samples"]])
    current = dict(min(res["samples"], key=lambda s: abs(s["throughput"] - med["median_throughput"])))
    current["throughput"], current["ms"] = med["median_throughput"], med["median_ms"]
    return {"status": "ok", "current": current, "spread": med}


def main(argv: Optional[Sequence[str]] = None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="bare_metal_b200.gate", description="performance regression gate")
    ap.add_argument("--baselines", default=DEFAULT_BASELINES)
    ap.add_argument("--tolerance", type=float, default=0.10)
    ap.add_argument("--kernel", default=None, help="check only this key of the baselines file")
    ap.add_argument("--list", action="store_true", dest="list_only")
    ap.add_argument("--samples", type=int, default=1, help="median of this many valid samples per config")
    ap.add_argument("--clock-locked", type=int, default=None,
                    help="the SM clock (MHz) an operator has locked the GPU to; this program never locks it")
    ap.add_argument("--record", default=None, help="append-only JSONL run record (default: results/gate_runs.jsonl "
                                                   "beside the baselines file)")
    args = ap.parse_args(argv)

    if not os.path.exists(args.baselines):
        print(f"ERROR: Baselines file not found: {args.baselines}")
        return 1
    with open(args.baselines) as f:
        baselines = json.load(f)
    base_dir = os.path.dirname(os.path.abspath(args.baselines))
    record_path = args.record or os.path.join(base_dir, "results", "gate_runs.jsonl")

    kernels = baselines.get("kernels", {})
    if args.list_only:
        print(f"Baselines recorded: {baselines.get('recorded_date', 'unknown')}")
        print(f"Platform: {baselines.get('platform', 'unknown')}")
        for kernel, entry in kernels.items():
            print(f"\n{kernel}")
            for cfg in [k for k in entry if k not in RESERVED_KEYS]:
                d = entry[cfg]
                unit = "GFLOPS" if d.get("gflops") is not None else "TOPS"
                lock = f"  [clock_lock {int(d['clock_lock'])} MHz]" if d.get("clock_lock") is not None else ""
                print(f"  {cfg}: {d.get('ms', '?')} ms, {d.get('gflops', d.get('tops', '?'))} {unit}{lock}")
        return 0
    if args.kernel is not None:
        if args.kernel not in kernels:
            print(f"ERROR: Kernel '{args.kernel}' not found in baselines")
            return 1
        kernels = {args.kernel: kernels[args.kernel]}

    print("=" * 70)
    print("  Performance Regression Check")
    print(f"  Tolerance: {args.tolerance * 100:.0f}%")
    print(f"  Baselines: {baselines.get('recorded_date', 'unknown')}")
    print("=" * 70)
    state = capture_gpu_state()
    if state is not None:
        print("  GPU state: " + classify_meta(state, state, {"require_no_throttle": False})["summary"])
        print("=" * 70)

    counts = {"total": 0, "measured": 0, "regressions": 0, "improvements": 0, "skipped": 0}
    failed, written, attempted = [], 0, 0
    run_id = time.strftime("%Y%m%dT%H%M%S", time.gmtime()) + f".{int(time.time() * 1000) % 1000:03d}Z"
    default_vw = baselines.get("default_valid_when", {})

    def record(row):
        nonlocal written, attempted
        attempted += 1
        try:
            append_jsonl_row(record_path, row)
            written += 1
        except OSError as e:                          # recording never changes the verdict
            print(f"WARNING: could not write the run record to {record_path}: {e}", file=sys.stderr)

    def emit(kernel, cfg, msg, verdict=None, current=None, header="", extra=None):
        """The one funnel for a config's outcome: print, count, record."""
        print(f"\n{kernel} [{cfg}]{header}\n  {msg}")
        v = verdict if verdict is not None else {"is_reg": False, "skipped": True, "msg": msg}
        if v.get("skipped"):
            counts["skipped"] += 1
        else:
            counts["measured"] += 1
            if v["is_reg"]:
                counts["regressions"] += 1
                failed.append((kernel, cfg, msg))
            elif "IMPROVED" in v["msg"]:
                counts["improvements"] += 1
        m = re.match(r"^[A-Z_]+", msg)
        row = {"type": "config", "run_id": run_id, "recorded_at": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()),
               "kernel": kernel, "config": cfg, "verdict": m.group(0) if m else None, "msg": msg,
               "measured": not v.get("skipped", False)}
        row.update(extra or {})
        row.update({"throughput": current.get("throughput") if current else None,
                    "unit": current.get("unit") if current else None,
                    "returncode": current.get("returncode") if current else None, "meta": meta_digest(current)})
        record(row)

    for kernel, entry in kernels.items():
        cfg_names = [k for k in entry if k not in RESERVED_KEYS]
        exe = entry.get("exe")
        if exe and not os.path.isabs(exe):
            exe = os.path.join(base_dir, exe)
        if not exe or not os.path.exists(exe):
            for cfg in cfg_names:
                counts["total"] += 1
                emit(kernel, cfg, "SKIPPED -- executable not found (build the host drivers first)", extra={"exe": exe})
            continue
        for cfg in cfg_names:
            counts["total"] += 1
            cfg_args = cfg.split("_")
            bcfg = entry[cfg]
            cl = int(round(float(bcfg["clock_lock"]))) if bcfg.get("clock_lock") is not None else None
            extra = {"baseline_gflops": bcfg.get("gflops"), "baseline_tops": bcfg.get("tops"), "clock_lock": cl,
                     "clock_locked_arg": args.clock_locked}
            vw = bcfg.get("valid_when", default_vw)
            tol = float(bcfg["tolerance"]) if bcfg.get("tolerance") is not None else args.tolerance
            band = None
            if cl is not None:
                if args.clock_locked is None:
                    emit(kernel, cfg, f"SKIPPED (clock_lock {cl} MHz; rerun with --clock-locked {cl} after a host-side lock)",
                         extra=extra)
                    continue
                if args.clock_locked != cl:
                    emit(kernel, cfg, f"SKIPPED (--clock-locked {args.clock_locked} != entry clock_lock {cl})", extra=extra)
                    continue
                band = (cl - CLOCK_LOCK_BAND_MHZ, cl + CLOCK_LOCK_BAND_MHZ)
            n = max(args.samples, 7 if cl is not None else 1)
            if n > 1:
                ml = measure_median(exe, cfg_args, bcfg, vw, n, 3 * n, band)
                if ml["status"] == "insufficient":
                    emit(kernel, cfg, f"SKIPPED ({ml['msg']})", extra=extra)
                    continue
                current = ml["current"]
                verdict = check_regression(current, bcfg, tol)
                emit(kernel, cfg, verdict["msg"], verdict, current, header=f" (median of {n})",
                     extra=dict(extra, tolerance=tol, samples=n, spread=ml["spread"]))
                continue
            current = run_benchmark(exe, cfg_args, bcfg)
            verdict = check_regression(current, bcfg, tol, unfair_reasons(current, vw))
            emit(kernel, cfg, verdict["msg"], verdict, current, extra=dict(extra, tolerance=tol))

    print("\n" + "=" * 70)
    print("  Total: {total} | Measured: {measured} | Regressions: {regressions} | Improvements: {improvements} | "
          "Skipped: {skipped}".format(**counts))
    v = summarise_verdict(counts["total"], counts["measured"], counts["regressions"], counts["skipped"])
    if failed:
        print("\n  Configs behind this verdict:")
        for k, c, m in failed:
            print(f"    {k} [{c}]\n      {m}")
    record({"type": "run", "run_id": run_id, "recorded_at": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()),
            "status": v["status"], "exit": v["exit"], "tolerance": args.tolerance, **counts,
            "config_rows_written": written, "config_rows_attempted": attempted})
    print(f"\n  RESULT: {v['msg']}")
    print(f"  Run record: {record_path} ({written} of {attempted} row(s) written)")
    return v["exit"]


if __name__ == "__main__":
    sys.exit(main())
