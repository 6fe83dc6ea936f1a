"""Python restatement of the reference's stdout-parsing regression gate, for driving the C++ bench
drivers (bare-metal_b200/host) the way the reference's R tooling drives its benches (R is absent
here).  Behaviour follows the R functions line for line:

  parse_throughput   R/cuasmR/R/bench_run.R:84-140     — pick a kernel's line, extract ms + value
  check_regression   R/cuasmR/R/bench_regression.R:28-77 — CRASH / SKIPPED / NO_DATA / REGRESSION / OK / IMPROVED
  summarise_verdict  scripts/bench/bench_regress.R:290-308 — exit 0 PASSED / 1 FAILED / 2 INCONCLUSIVE
  decode_throttle    R/cuasmR/R/bench_meta.R:41-64     — nvidia-smi throttle bitmask
"""
from __future__ import annotations

import re
import subprocess
from typing import Optional, Sequence

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
