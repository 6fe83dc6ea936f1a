#!/usr/bin/env python
"""Benchmark of the B200-native INT8 GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: the dense W8A8 GEMM M=N=K=4096 — int8 operands uniform on [-127,127], per-row activation
scale and per-column weight scale ~ U[1e-3, 2e-2], fp16 output D = half_rn(float(A.W^T) * sa[m]*sw[n]),
int32 accumulate.  A "step" is one such GEMM.  With N > 1 GPUs the SAME problem is split by weight
columns (4096/N per GPU, strong scaling): every rank computes its slab and the GEMM epilogue stores it
into the row-major output of every rank over NVLink (fused all-gather), then a group barrier.

Prints ONE JSON line (rank 0).  `value` is dense-equivalent TOPS with operands resident in HBM; `e2e`
is the same metric through the public API with HOST buffers (H2D of the operands and scales, D2H of the
result, inside the timed region).  `extras` carries the other workloads of the path, each with its own
roofline: 2:4-sparse 4096^3, the decode shapes, the 8192-token layer chain — and with N > 1 their
N-split forms with GEMM-only and gathered scaling efficiency against a single-GPU run of the same
process.  `--impl reference` times the reference project's own CPU verification GEMM
(cpu_sparse_gemm_int8, compiled in place into oracle/_ref) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M = N_TOTAL = K = 4096
METRIC = "INT8 dense-equiv TOPS at 4096^3 (W8A8 dense, fp16 out)"
UNIT = "TOPS"
NOMINAL_INT8_TOPS = 4500.0          # B200 dense INT8 datasheet figure
NOMINAL_HBM_GBS = 8000.0


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock / throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [l.split(", ") for (t, l) in self.lines if t0 - 0.05 <= t <= t1 + 0.15]
        if not rows:
            rows = [l.split(", ") for (_, l) in self.lines]
        clocks, reasons, smax, power = [], set(), None, []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 7:
                continue
            try:
                clocks.append(float(r[0])); smax = float(r[1]); power.append(float(r[2]))
            except ValueError:
                continue
            for n, v in zip(names, r[3:7]):
                if v.strip().lower() == "active":
                    reasons.add(n)
        clocks.sort()
        med = clocks[len(clocks) // 2] if clocks else None
        return {"sm_mhz": med, "sm_max_mhz": smax, "reasons": sorted(reasons), "samples": len(clocks),
                "power_w_max": max(power) if power else None}


class GpuState:
    """Read-only NVML snapshots (SM clock, power, throttle reasons) of one CUDA device, for the per-batch
    validity check.  Nothing is ever set through this handle."""
    REASONS = {0x4: "SwPowerCap", 0x8: "HwSlowdown", 0x20: "SwThermalSlowdown", 0x40: "HwThermalSlowdown",
               0x80: "HwPowerBrakeSlowdown", 0x2: "ApplicationsClocksSet"}

    def __init__(self, torch, device_index: int):
        self.h = None
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode() if not uuid.startswith("GPU-") else uuid.encode())
        except Exception:
            self.h = None

    def snapshot(self):
        if self.h is None:
            return None
        nv = self.nv
        try:
            mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            return {"gpu": {"clock_sm": float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)),
                            "clock_mem": float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_MEM)),
                            "temp_c": float(nv.nvmlDeviceGetTemperature(self.h, nv.NVML_TEMPERATURE_GPU)),
                            "power_w": nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0, "pstate": "P?",
                            "throttle_hex": hex(mask), "throttle": [n for b, n in self.REASONS.items() if mask & b]}}
        except Exception:
            return None


# GPU state a batch must have been measured in: the 1 kW power cap is this part's normal state under a
# tensor-core load, thermal and hardware slowdowns (and a foreign clock lock) make a batch unfair.
VALID_WHEN = {"require_no_throttle": True, "allow_throttle": ["GpuIdle", "SwPowerCap"]}


def measure_batches(torch, run_steps, ms_step_hint: float, state: GpuState, n_valid: int = 7, max_attempts: int = 21,
                    batch_ms: float = 120.0):
    """Median of `n_valid` VALID batches (collect-N-valid of the reference's measurement harness).  A batch is
    long enough (~120 ms of steps) for NVML to report the clocks and power it ran at: the state is read
    once before the batch and once WHILE its last steps are still executing, the batch is timed with CUDA
    events, and a batch taken under a thermal / hardware slowdown is rejected and replaced."""
    from bare_metal_b200 import gate
    steps = max(50, int(batch_ms / max(ms_step_hint, 1e-4)))

    def sample():
        pre = state.snapshot()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run_steps(steps)
        e1.record()
        during = state.snapshot()            # the launches are asynchronous: the GPU is still inside the batch
        torch.cuda.synchronize()
        return {"ms": e0.elapsed_time(e1) / steps, "pre": pre, "post": during}

    def validate(s):
        if s["pre"] is None or s["post"] is None:          # no NVML: nothing to hold against the batch
            return {"ok": True, "reason": None}
        return gate.validate_sample(0, s["ms"], s["pre"], s["post"], VALID_WHEN)

    res = gate.collect_valid_samples(sample, validate, n_valid, max_attempts)
    ms = [s["ms"] for s in res["samples"]]
    clk = [s["post"]["gpu"]["clock_sm"] if s["post"] else None for s in res["samples"]]
    pw = [s["post"]["gpu"]["power_w"] if s["post"] else None for s in res["samples"]]
    thr = [s["post"]["gpu"]["throttle"] if s["post"] else None for s in res["samples"]]
    med = gate.report_median_metrics([1.0 / m for m in ms], ms, clk)
    return {"n_valid": len(ms), "attempts": res["attempts"], "rejected": res["rejected"], "steps_per_batch": steps,
            "median_ms": med["median_ms"], "min_ms": min(ms) if ms else None, "max_ms": max(ms) if ms else None,
            "batch_ms": [round(m, 5) for m in ms], "batch_sm_mhz": clk, "batch_power_w": pw, "batch_throttle": thr}


def reference_arm(args, rank: int, world: int) -> None:
    """The reference's own CPU verification GEMM on the host cores (rank 0 only)."""
    if rank != 0:
        return
    import numpy as np
    import oracle
    kind = "reference" if oracle.have_ref() else "port"
    cores = os.cpu_count() or 1
    A = oracle.gen_int8((M, K), 0, oracle.stream_id("C2", "A"))
    B = oracle.gen_int8((K, N_TOTAL), 0, oracle.stream_id("C2", "Wt"))

    def gemm(rows):
        a = np.ascontiguousarray(A[:rows])
        if kind == "reference":
            return oracle.ref_cpu_sparse_gemm_int8(a, B, threads=cores)
        return oracle.igemm(a, B, threads=cores)

    probe_rows = min(M, 8 * cores)
    t = time.perf_counter(); gemm(probe_rows); per_row = (time.perf_counter() - t) / probe_rows
    rows = int(max(cores, min(M, 0.5 / max(per_row, 1e-9))))      # ~0.5 s per step
    for _ in range(args.warmup):
        gemm(rows)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        gemm(rows)
    dt = (time.perf_counter() - t0) / args.steps
    tops = 2.0 * rows * N_TOTAL * K / dt / 1e12
    sample = f"{rows} of {M} rows of the 4096^3 integer GEMM per step, {cores} host threads on row slabs"
    line = {"impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "s8*s8->s32", "data": "synthetic",
            "config": {"workload": "W8A8 GEMM M=N=K=4096 (integer core on CPU)", "sample": sample},
            "cpu_baseline": {"value": tops, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def cpu_baseline_leg():
    import numpy as np
    import oracle
    kind = "reference" if oracle.have_ref() else "port"
    cores = os.cpu_count() or 1
    A = oracle.gen_int8((M, K), 0, oracle.stream_id("C2", "A"))
    B = oracle.gen_int8((K, N_TOTAL), 0, oracle.stream_id("C2", "Wt"))
    rows = min(M, max(cores * 8, 1024))
    a = np.ascontiguousarray(A[:rows])
    fn = (lambda: oracle.ref_cpu_sparse_gemm_int8(a, B, threads=cores)) if kind == "reference" else \
         (lambda: oracle.igemm(a, B, threads=cores))
    fn()
    reps, t0 = 0, time.perf_counter()
    while reps < 3 or (time.perf_counter() - t0 < 4.0 and reps < 50):
        fn(); reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": 2.0 * rows * N_TOTAL * K / dt / 1e12, "unit": UNIT, "cores": cores, "kind": kind,
            "sample": f"{rows} of {M} rows of the 4096^3 integer GEMM, x{reps}, {cores} host threads on row slabs"}


class Ctx:
    """What every part of the bench needs: modules, device, ranks and the timing helpers."""

    def __init__(self, torch, dist, oracle, ig, devn, rank, world, peaks):
        self.torch, self.dist, self.oracle, self.ig = torch, dist, oracle, ig
        self.devn, self.rank, self.world, self.peaks = devn, rank, world, peaks

    def sync(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        t = self.torch.tensor([v], dtype=self.torch.float64, device=self.devn)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def timeit(self, fn, iters, warm=5, collective=False):
        """ms per call of fn(i): CUDA events on the launching stream; with `collective` the region is
        bracketed by a group barrier and the result is the maximum over the ranks."""
        torch = self.torch
        for i in range(warm):
            fn(i)
        if collective:
            self.sync()
        else:
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        return self.max_over_ranks(ms) if collective else ms


def timeit_graph(cx, fn, per_graph: int = 20, replays: int = 5, collective: bool = False):
    """ms per call of fn(i) when `per_graph` consecutive calls are recorded into ONE CUDA graph and the graph is
    replayed: what a serving loop pays once the per-call host work (Python, argument checks, launch) is out of the
    way — for steps of a few microseconds that host work, not the GPU, sets the eager pace.  Returns None when the
    capture is refused."""
    torch = cx.torch
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(3):
                fn(i)                                    # first-use work (allocations, attributes) stays outside the capture
        torch.cuda.synchronize()
        if collective:
            cx.sync()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(per_graph):
                fn(i)
        if collective:
            cx.sync()
        g.replay()
        torch.cuda.synchronize()
        if collective:
            cx.sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / (replays * per_graph)
        return cx.max_over_ranks(ms) if collective else ms
    except Exception as e:                               # noqa: BLE001 — a refused capture is reported, not fatal
        if cx.rank == 0:
            print(f"graph capture refused: {e}", file=sys.stderr)
        return None


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the sparse / decode / layer-chain side measurements")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N > 1: fused = GEMM epilogue stores to all ranks over NVLink; nccl = GEMM then all-gather")
    ap.add_argument("--lanes", type=int, default=2, choices=[1, 2, 3, 4],
                    help="N > 1, fused gather: steps in flight (L > 1: consecutive steps take turns on L streams)")
    ap.add_argument("--workload", default="dense", choices=["dense", "sparse", "decode", "online_quant", "hgemm_sparse"],
                    help="with --profile: which kernel to run (dense = the headline; sparse = 2:4 at 4096^3; "
                         "decode = the skinny sparse GEMM)")
    ap.add_argument("--decode-m", type=int, default=1, help="with --profile --workload decode: number of tokens (1, 16, 64)")
    ap.add_argument("--profile", action="store_true",
                    help="profiler-friendly run: only warm-up + the timed steps of one kernel")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        reference_arm(args, rank, world)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    import oracle                      # data generators, the parity check of the timed step, the cpu_baseline leg
    import bare_metal_b200 as bm
    from bare_metal_b200 import _lib
    from bare_metal_b200 import igemm as ig

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback exists)")
    torch.cuda.set_device(local_rank)
    devn = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=devn)
    bm.build()
    peaks = load_peaks()
    cx = Ctx(torch, dist, oracle, ig, devn, rank, world, peaks)

    if args.profile and args.workload != "dense":
        profile_side_workload(args, ig, oracle, torch, devn)
        return

    # ---- operands: enough rotating sets that consecutive steps never hit L2 (126 MB) -------------
    from bare_metal_b200 import nsplit
    n0, n_len = nsplit.shard_columns(N_TOTAL, world, rank)
    set_bytes = M * K + n_len * K + 2 * M * (n_len if world == 1 else N_TOTAL)
    n_sets = max(2, -(-3 * 126 * 2 ** 20 // set_bytes))          # > 3x L2 in flight
    sid = oracle.stream_id
    A_h = oracle.gen_int8((M, K), 0, sid("C2", "A"))
    W_full_h = oracle.gen_int8((N_TOTAL, K), 0, sid("C2", "W"))
    sa_h = oracle.gen_scales(M, 0, sid("C2", "sa"))
    sw_full_h = oracle.gen_scales(N_TOTAL, 0, sid("C2", "sw"))
    W_h, sw_h = np.ascontiguousarray(W_full_h[n0:n0 + n_len]), np.ascontiguousarray(sw_full_h[n0:n0 + n_len])
    A_d = [torch.from_numpy(A_h).to(devn) for _ in range(n_sets)]
    W_d = [torch.from_numpy(W_h).to(devn) for _ in range(n_sets)]
    sa_d, sw_d = torch.from_numpy(sa_h).to(devn), torch.from_numpy(sw_h).to(devn)
    D_d = [torch.empty((M, n_len), dtype=torch.float16, device=devn) for _ in range(n_sets)]
    layer = G_blocks = None
    lanes = None
    if world > 1:
        layer = nsplit.ColumnShardedLinear(W_d[0], sw_d, N_TOTAL, n0, mode=args.gather)
        G_blocks = torch.empty((world, M, n_len), dtype=torch.float16, device=devn)
        # two steps in flight: consecutive steps are independent problems (rotating operand sets, the layer's two
        # output buffers), so they alternate between two streams — the GEMM of one step overlaps the NVLink tail
        # and the group barrier of the other, as a server does with independent micro-batches
        if args.gather == "fused" and args.lanes > 1:
            lanes = [torch.cuda.Stream() for _ in range(args.lanes)]

    def step(i: int):
        s = i % n_sets
        if world == 1:
            ig.w8a8_linear(A_d[s], W_d[s], D_d[s], sa_d, sw_d, M, n_len, K)
            return D_d[s]
        layer.W = W_d[s]
        if lanes is not None:
            return layer.forward_fused(A_d[s], sa_d, lane=i % len(lanes), stream=lanes[i % len(lanes)])
        if args.gather == "fused":
            return layer.forward_fused(A_d[s], sa_d)
        return layer.forward_nccl(A_d[s], sa_d, out=G_blocks, local=D_d[s])

    def fork_lanes(ev):
        """The lane streams start behind `ev` (recorded on the current stream)."""
        for ln in lanes or ():
            ln.wait_event(ev)

    def join_lanes():
        """The current stream continues behind everything enqueued on the lane streams."""
        for ln in lanes or ():
            torch.cuda.current_stream().wait_stream(ln)

    def gemm_only(i: int):
        s = i % n_sets
        ig.w8a8_linear(A_d[s], W_d[s], D_d[s], sa_d, sw_d, M, n_len, K)

    # ---- parity of what is being timed (one step against the CPU oracle on sampled rows) -----------
    rows = np.array([0, 1, 127, 128, 2047, 4095])
    want_full = oracle.dequant_w8a8_f16(oracle.igemm_nt(np.ascontiguousarray(A_h[rows]), W_full_h), sa_h[rows], sw_full_h)
    out0 = step(0)
    cx.sync()
    if world == 1 or args.gather == "fused":
        got = out0.cpu().numpy()[rows]            # N > 1: the whole row, i.e. every peer's slab as it arrived here
    else:
        got = nsplit.ColumnShardedLinear.blocks_to_row_major(out0).cpu().numpy()[rows]
    if not np.array_equal(got.view(np.uint16), want_full.view(np.uint16)):
        raise SystemExit("parity check failed: the benchmarked step disagrees with the CPU oracle")

    # ---- timed region: exactly K steps, barrier + synchronize on both sides, max over ranks --------
    for i in range(args.warmup):
        step(i)
    cx.sync()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # the ~0.3 s nvidia-smi needs to come up are spent under the same load, not idle: the timed steps then
    # run at the clocks and power state of a GPU that is doing this work, not of one waking up
    for j in range(0 if args.profile else (2500 if world == 1 else 600)):
        step(j)
        if j % 64 == 63:
            torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    cx.sync()
    t_wall0 = time.time()
    ev0.record()
    fork_lanes(ev0)
    for i in range(args.steps):
        step(i)
    join_lanes()
    ev1.record()
    cx.sync()
    ms_total = ev0.elapsed_time(ev1)
    ms_step = cx.max_over_ranks(ms_total) / args.steps
    # extra untimed load so the clock sampler has samples under load even for a short region.  The number of
    # steps is the same on every rank (derived from the rank-agreed step time, never from a rank's own clock):
    # a step of the N-split layer ends in a group barrier, and a rank that made one call more than its peers
    # would wait in it for a round that never comes.
    n_load = 0 if args.profile else max(64, min(40000, int(1.2 / max(ms_step * 1e-3, 1e-6))))
    for j in range(n_load):
        step(j)
        if j % 64 == 63:
            torch.cuda.synchronize()
    cx.sync()
    t_wall1 = time.time()
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    ops_step = 2.0 * M * N_TOTAL * K
    value = ops_step / (ms_step * 1e-3) / 1e12
    if args.profile:
        if rank == 0:
            print(json.dumps({"profile_run": True, "value": value, "unit": UNIT, "ms_per_step": ms_step}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- median of >= 7 valid batches of the same step (GPU state snapshot around each) ------------
    state = GpuState(torch, local_rank)
    batches = None
    if world == 1:
        batches = measure_batches(torch, lambda n: [step(i) for i in range(n)], ms_step, state)
        batches["median_tops"] = ops_step / (batches["median_ms"] * 1e-3) / 1e12
        batches["min_tops"] = ops_step / (batches["max_ms"] * 1e-3) / 1e12
        batches["max_tops"] = ops_step / (batches["min_ms"] * 1e-3) / 1e12

    # ---- kernel-only duration for the roofline (the GEMM launch alone, same stream) ----------------
    kern_ms = cx.timeit(gemm_only, args.steps, warm=3, collective=world > 1)
    achieved = 2.0 * M * n_len * K / (kern_ms * 1e-3) / 1e12
    int8_peak = 2.0 * peaks["bf16_tflops"]
    roofline = {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TOP/s",
                "frac": achieved / int8_peak,
                "peak_note": f"2 x cuBLAS bf16 burst ({peaks['bf16_tflops']} TFLOP/s, of {peaks['source']}); "
                             f"INT8 runs at twice the bf16 rate on this tensor core",
                "frac_of_nominal_4500": achieved / NOMINAL_INT8_TOPS,
                "kernel": "igemm_dense_pair_kernel<false,EPI_F16_ROWCOL>" if n_len >= 1024 else "igemm_dense_kernel / igemm_dense_pair_kernel (slab GEMM)",
                "kernel_ms": kern_ms, "algorithmic_bytes": M * K + n_len * K + 2 * M * n_len + 4 * (M + n_len),
                "traffic": TRAFFIC_BYTES_NCU if world == 1 else None}

    scaling_detail = None
    if world > 1:
        scaling_detail = sharded_headline_detail(cx, nsplit, _lib, layer, step, gemm_only, A_d, W_d, sa_d, sw_d, D_d, G_blocks,
                                                 W_full_h, sw_full_h, n_len, n_sets, kern_ms, ms_step, args)
        roofline["fused_collective"] = scaling_detail.pop("fused_collective")

    # ---- end to end through the public API with host buffers ---------------------------------------
    e2e = end_to_end(cx, nsplit, args, A_h, W_h, sa_h, sw_h, n0, n_len, rows, want_full, ops_step)

    # ---- side measurements (not the headline) ------------------------------------------------------
    extras = {}
    if not args.no_extras:
        if world == 1:
            extras = side_measurements(cx, ig, oracle, torch, devn, peaks, _lib)
        else:
            extras = sharded_side_measurements(cx, nsplit, _lib)
    if scaling_detail:
        extras["headline_4096_strong_split"] = scaling_detail

    if rank == 0:
        cpu = None if args.no_cpu_baseline else cpu_baseline_leg()
        if world == 1:
            par = "single GPU"
            launches = args.steps
        else:
            par = f"n-split x{world} ({n_len} of {N_TOTAL} weight columns per GPU)" + (
                " + all-gather of the fp16 output fused into the GEMM epilogue (paced peer TMA stores) + group barrier"
                + (f"; {len(lanes)} steps in flight (independent steps take turns on {len(lanes)} streams, each with its own "
                   "output buffers and barrier instance)" if lanes is not None else "")
                if args.gather == "fused" else " + NCCL all-gather of the fp16 output")
            launches = args.steps * (2 if args.gather == "fused" else 1)     # per rank: GEMM+gather kernel, barrier kernel
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "strong" if world > 1 else "weak",
                "vs_baseline": None, "dtype": "s8*s8->s32 (fp32 scale, fp16 out)", "data": "synthetic",
                "config": {"workload": f"W8A8 GEMM M={M} K={K} N={N_TOTAL}, fp16 out (dense 4096^3)",
                           "parallelism": par,
                           "l2": f"{n_sets} rotating operand sets ({n_sets * set_bytes / 2**20:.0f} MiB) exceed the 126 MiB L2",
                           "tile": "CTA pairs (cta_group::2), 256x256x128 per pair, 4-stage TMA ring, 2 TMEM accumulators"},
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches,
                "clocks": clocks, "batches": batches, "extras": extras}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def measure_link(cx, nsplit, _lib):
    """Peer-store bandwidth of THIS run (GB/s a rank receives while every rank pushes a slab to all the others
    at once, unpaced): the denominator of the gather roofline."""
    return nsplit.measure_peer_store_bandwidth(cx.devn, timeit=lambda fn: cx.timeit(fn, 10, warm=2, collective=True))


def sharded_case(cx, nsplit, _lib, name, Mx, Nx, Kx, link_gbs, iters=20, with_nccl=True, single_ms=None):
    """One dense W8A8 GEMM of the 8192-token layer, split by columns over the ranks: single-GPU time of the
    unsplit problem (same process, same run), slab GEMM alone, fused GEMM + gather (+ barrier), NCCL baseline;
    efficiencies = t_single / (N * t) and the fused step against its bound."""
    torch = cx.torch
    world, rank, devn = cx.world, cx.rank, cx.devn
    n0, n_len = nsplit.shard_columns(Nx, world, rank)
    sets = 3 if (Mx * Kx + n_len * Kx) * 3 < 400e6 else 2
    X = [torch.randint(-127, 128, (Mx, Kx), dtype=torch.int8, device=devn) for _ in range(sets)]
    Wf = torch.randint(-127, 128, (Nx, Kx), dtype=torch.int8, device=devn)
    Ws = [Wf[n0:n0 + n_len].contiguous() for _ in range(sets)]
    sa = torch.rand(Mx, device=devn) * 0.019 + 0.001
    swf = torch.rand(Nx, device=devn) * 0.019 + 0.001
    sw = swf[n0:n0 + n_len].contiguous()
    out = {"M": Mx, "N": Nx, "K": Kx, "slab_columns": n_len}
    if single_ms is None:
        Df = torch.empty((Mx, Nx), dtype=torch.float16, device=devn)
        single_ms = cx.timeit(lambda i: cx.ig.w8a8_linear(X[i % sets], Wf, Df, sa, swf, Mx, Nx, Kx), iters, collective=True)
        del Df
    del Wf
    layer = nsplit.ColumnShardedLinear(Ws[0], sw, Nx, n0, mode="fused")
    Dl = torch.empty((Mx, n_len), dtype=torch.float16, device=devn)

    def slab(i):
        layer.W = Ws[i % sets]; layer.forward_local(X[i % sets], sa, Dl)

    def fused(i):
        layer.W = Ws[i % sets]; layer.forward_fused(X[i % sets], sa)

    t_slab = cx.timeit(slab, iters, collective=True)
    t_fused = cx.timeit(fused, iters, collective=True)
    ops = 2.0 * Mx * Nx * Kx
    recv = 2.0 * Mx * (Nx - n_len)
    t_link = recv / (link_gbs * 1e9) * 1e3
    target = max(t_slab, t_link)
    out.update({"single_gpu_ms": single_ms, "single_gpu_tops": ops / single_ms / 1e9,
                "gemm_only_ms": t_slab, "gemm_only_tops": ops / t_slab / 1e9, "gemm_only_efficiency": single_ms / (world * t_slab),
                "gathered_ms": t_fused, "gathered_tops": ops / t_fused / 1e9, "gathered_efficiency": single_ms / (world * t_fused),
                "recv_bytes_per_rank": recv, "link_bound_ms": t_link,
                "bound": "nvlink receive" if t_link > t_slab else "tensor", "frac_of_bound": target / t_fused,
                "achieved_link_gb_per_s": recv / (t_fused * 1e-3) / 1e9})
    if with_nccl and len({l for _, l in layer.slabs}) == 1:
        base = nsplit.ColumnShardedLinear(Ws[0], sw, Nx, n0, mode="nccl")
        G = torch.empty((world, Mx, n_len), dtype=torch.float16, device=devn)

        def nccl(i):
            base.W = Ws[i % sets]; base.forward_nccl(X[i % sets], sa, out=G, local=Dl)
        out["nccl_all_gather_ms"] = cx.timeit(nccl, max(5, iters // 2), collective=True)
        del G
    del X, Ws, layer, Dl
    torch.cuda.empty_cache()
    return out


def sharded_headline_detail(cx, nsplit, _lib, layer, step, gemm_only, A_d, W_d, sa_d, sw_d, D_d, G_blocks, W_full_h, sw_full_h,
                            n_len, n_sets, kern_ms, ms_step, args):
    """The headline problem at N > 1 taken apart: link bandwidth of this run, single-GPU time of the same 4096^3
    in this process, slab GEMM, fused step, NCCL baseline, efficiencies and the fraction of the bound."""
    torch = cx.torch
    link = measure_link(cx, nsplit, _lib)
    Wf = torch.from_numpy(W_full_h).to(cx.devn)
    swf = torch.from_numpy(sw_full_h).to(cx.devn)
    Df = torch.empty((M, N_TOTAL), dtype=torch.float16, device=cx.devn)
    single_ms = cx.timeit(lambda i: cx.ig.w8a8_linear(A_d[i % n_sets], Wf, Df, sa_d, swf, M, N_TOTAL, K), args.steps, collective=True)
    del Wf, Df
    base = nsplit.ColumnShardedLinear(W_d[0], sw_d, N_TOTAL, layer.n0, mode="nccl")

    def nccl(i):
        s = i % n_sets
        base.W = W_d[s]; base.forward_nccl(A_d[s], sa_d, out=G_blocks, local=D_d[s])

    def fused_nobar(i):
        s = i % n_sets
        layer.W = W_d[s]; layer.forward_fused(A_d[s], sa_d, barrier=False)
    def fused_serial(i):
        s = i % n_sets
        layer.W = W_d[s]; layer.forward_fused(A_d[s], sa_d)
    t_nccl = cx.timeit(nccl, max(5, args.steps // 2), collective=True)
    t_kernel = cx.timeit(fused_nobar, args.steps, collective=True)
    cx.sync()
    t_serial = cx.timeit(fused_serial, args.steps, collective=True)      # one step at a time on one stream
    cx.sync()
    recv = 2.0 * M * (N_TOTAL - n_len)
    t_link = recv / (link * 1e9) * 1e3
    target = max(kern_ms, t_link)
    return {"single_gpu_ms": single_ms, "gemm_only_ms": kern_ms, "gemm_only_efficiency": single_ms / (cx.world * kern_ms),
            "gathered_ms": ms_step, "gathered_efficiency": single_ms / (cx.world * ms_step),
            "steps_in_flight": args.lanes if args.gather == "fused" else 1,
            "single_step_latency_ms": t_serial,
            "fused_kernel_without_barrier_ms": t_kernel, "nccl_all_gather_ms": t_nccl,
            "fused_collective": {"bound": "nvlink receive" if t_link > kern_ms else "tensor",
                                 "recv_bytes_per_rank": recv, "link_gb_per_s": link,
                                 "link_note": "peer-store bandwidth measured in this run: all ranks push a slab to all others at once",
                                 "pacing_gb_per_s": _lib.get_option("gather_gbs"),
                                 "target_ms": target, "achieved_ms": ms_step, "frac": target / ms_step,
                                 "achieved_link_gb_per_s": recv / (ms_step * 1e-3) / 1e9, "gemm_only_ms": kern_ms}}


def sharded_side_measurements(cx, nsplit, _lib):
    """N > 1: the largest dense shape, the 8192-token layer chain and the decode shapes, all N-split."""
    torch = cx.torch
    world, rank, devn = cx.world, cx.rank, cx.devn
    out = {}
    link = measure_link(cx, nsplit, _lib)
    out["link_gb_per_s_measured"] = link
    # the 8192-token layer: four projections, each column-sharded with its output gathered on every rank
    chain = {}
    tot = {"single_gpu_ms": 0.0, "gemm_only_ms": 0.0, "gathered_ms": 0.0, "ops": 0.0}
    for name, Kc, Nc in (("qkv", 4096, 12288), ("out", 4096, 4096), ("gate_up", 4096, 22016), ("down", 11008, 4096)):
        r = sharded_case(cx, nsplit, _lib, name, 8192, Nc, Kc, link, iters=10, with_nccl=(name == "gate_up"))
        chain[name] = r
        for k in ("single_gpu_ms", "gemm_only_ms", "gathered_ms"):
            tot[k] += r[k]
        tot["ops"] += 2.0 * 8192 * Nc * Kc
    chain["layer"] = {"single_gpu_ms": tot["single_gpu_ms"], "gemm_only_ms": tot["gemm_only_ms"], "gathered_ms": tot["gathered_ms"],
                      "single_gpu_tops": tot["ops"] / tot["single_gpu_ms"] / 1e9, "gathered_tops": tot["ops"] / tot["gathered_ms"] / 1e9,
                      "gemm_only_efficiency": tot["single_gpu_ms"] / (world * tot["gemm_only_ms"]),
                      "gathered_efficiency": tot["single_gpu_ms"] / (world * tot["gathered_ms"])}
    out["layer_chain_8192_tokens_nsplit"] = chain
    out["largest_shape_gate_up_8192x22016x4096"] = chain["gate_up"]
    # decode shapes, 2:4-sparse weights, 28672 channels split over the ranks
    oracle, ig = cx.oracle, cx.ig
    Nd, Kd = 28672, 8192
    n0 = nsplit.shard_columns(Nd, world, rank, 128 if Nd % (128 * world) == 0 else 16)
    n0, n_len = n0
    comp, nib = oracle.gen_sparse_rows(n_len, Kd, 0, oracle.stream_id("C5", f"W{rank}"))
    sets = max(2, -(-2 * 126 * 2 ** 20 // (n_len * Kd * 5 // 8)))           # the slabs in rotation exceed L2
    sets = min(sets, 16)
    comp_0, nib_0 = torch.from_numpy(comp).to(devn), torch.from_numpy(nib).to(devn)
    til_0 = ig.sp_pack_meta(nib_0, ig.BM_META_ROWS, n_len, Kd)
    pk_d = [ig.sp_pack_weights(comp_0, nib_0, ig.BM_META_ROWS, n_len, Kd) for _ in range(sets)]
    sw = torch.from_numpy(oracle.gen_scales(n_len, 0, oracle.stream_id("C5", f"sw{rank}"))).to(devn)
    layer = nsplit.ColumnShardedSparseLinear(comp_0, til_0, sw, Nd, n0, mode="push", W_packed_slab=pk_d[0])
    dec = {"channels_per_rank": n_len, "l2": f"{sets} weight slabs of {n_len * Kd * 5 // 8 / 2**20:.0f} MiB in rotation",
           "weights": "packed blocks (bm_sp_pack_weights), rows of the slab dealt to all CTA slots in multiples of 8"}
    for Md in (1, 16, 64):
        Xd = torch.from_numpy(oracle.gen_int8((Md, Kd), 0, oracle.stream_id("C5", f"X{Md}"))).to(devn)
        sa = torch.from_numpy(oracle.gen_scales(Md, 0, oracle.stream_id("C5", "sa"))).to(devn)
        Dl = torch.empty((Md, n_len), dtype=torch.float16, device=devn)

        def local(i):
            layer.W_packed = pk_d[i % sets]
            layer.forward_local(Xd, sa, Dl)

        def pushed(i):
            layer.W_packed = pk_d[i % sets]
            layer.forward_push(Xd, sa)
        t_local = cx.timeit(local, 40, collective=True)
        t_push = cx.timeit(pushed, 40, collective=True)
        g_local = timeit_graph(cx, local, collective=True)
        g_push = timeit_graph(cx, pushed, collective=True)
        byts = Nd * Kd / 2 + Nd * Kd / 8 + world * Md * Kd + 2 * Md * Nd + 4 * (world * Md + Nd)
        best_local = min(t for t in (t_local, g_local) if t is not None)
        best_push = min(t for t in (t_push, g_push) if t is not None)
        dec[f"M{Md}"] = {"gemm_only_us": best_local * 1e3, "gathered_us": best_push * 1e3,
                         "eager_us": {"gemm_only": t_local * 1e3, "gathered": t_push * 1e3},
                         "cuda_graph_us": {"gemm_only": None if g_local is None else g_local * 1e3,
                                           "gathered": None if g_push is None else g_push * 1e3,
                                           "note": "20 steps recorded into one CUDA graph, replayed: the eager pace of a step this "
                                                   "short is set by the host (Python + launches), not by the GPU"},
                         "aggregate_gb_per_s_gemm_only": byts / best_local / 1e6, "aggregate_gb_per_s_gathered": byts / best_push / 1e6,
                         "frac_of_hbm_peak_gemm_only": byts / best_local / 1e6 / (world * cx.peaks["hbm_gbs"]),
                         "frac_of_hbm_peak_gathered": byts / best_push / 1e6 / (world * cx.peaks["hbm_gbs"]),
                         "algorithmic_bytes_all_ranks": byts}
    out["decode_sparse_K8192_N28672_nsplit"] = dec
    return out


def end_to_end(cx, nsplit, args, A_h, W_h, sa_h, sw_h, n0, n_len, rows, want_full, ops_step):
    """The public API with HOST buffers: every step copies the activations, the rank's weights and the scales
    from pinned host memory, runs the (N-split) linear and copies the rank's full output back.  Copy-in, GEMM
    and copy-out of neighbouring steps overlap on three streams (two buffer sets); every step still moves all
    of its inputs and its output."""
    torch, dist, ig = cx.torch, cx.dist, cx.ig
    import numpy as np
    world, devn = cx.world, cx.devn
    n_out = n_len if world == 1 else N_TOTAL
    pin = lambda a: torch.from_numpy(a).pin_memory()
    A_p, W_p, sa_p, sw_p = pin(A_h), pin(W_h), pin(sa_h), pin(sw_h)
    NB = 2
    A_e = [torch.empty((M, K), dtype=torch.int8, device=devn) for _ in range(NB)]
    W_e = [torch.empty((n_len, K), dtype=torch.int8, device=devn) for _ in range(NB)]
    sa_e = [torch.empty(M, dtype=torch.float32, device=devn) for _ in range(NB)]
    sw_e = [torch.empty(n_len, dtype=torch.float32, device=devn) for _ in range(NB)]
    D_e = [torch.empty((M, n_len), dtype=torch.float16, device=devn) for _ in range(NB)]
    D_ps = [torch.empty((M, n_out), dtype=torch.float16).pin_memory() for _ in range(NB)]
    layers = None
    if world > 1:
        layers = [nsplit.ColumnShardedLinear(W_e[b], sw_e[b], N_TOTAL, n0, mode="fused") for b in range(NB)]
    s_in, s_mm, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(NB)]       # inputs of the set are on the device
    ev_mm = [torch.cuda.Event() for _ in range(NB)]       # the GEMM of the set is done (inputs free, output ready)
    ev_out = [torch.cuda.Event() for _ in range(NB)]      # the output of the set is back on the host
    step_no = [0]

    def e2e_step():
        b = step_no[0] % NB
        step_no[0] += 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_mm[b])                     # the previous GEMM on this set has read its inputs
            A_e[b].copy_(A_p, non_blocking=True); W_e[b].copy_(W_p, non_blocking=True)
            sa_e[b].copy_(sa_p, non_blocking=True); sw_e[b].copy_(sw_p, non_blocking=True)
            ev_in[b].record(s_in)
        with torch.cuda.stream(s_mm):
            s_mm.wait_event(ev_in[b])
            s_mm.wait_event(ev_out[b])                    # the previous output of this set has left the device
            if world == 1:
                ig.w8a8_linear(A_e[b], W_e[b], D_e[b], sa_e[b], sw_e[b], M, n_len, K)
                res = D_e[b]
            else:
                res = layers[b].forward_fused(A_e[b], sa_e[b])     # symmetric [M x N] output, barrier included
            ev_mm[b].record(s_mm)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_mm[b])
            D_ps[b].copy_(res, non_blocking=True)
            ev_out[b].record(s_out)

    n_e2e = max(6, min(args.steps, 30))
    n_e2e += n_e2e % NB
    for _ in range(2 * NB):
        e2e_step()
    cx.sync()
    step_no[0] = 1                                        # so that the final timed step lands in set 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    cur = torch.cuda.current_stream()
    e0.record(cur)
    for st in (s_in, s_mm, s_out):
        st.wait_event(e0)
    for _ in range(n_e2e):
        e2e_step()
    for st in (s_in, s_mm, s_out):
        done = torch.cuda.Event()
        done.record(st)
        cur.wait_event(done)
    e1.record(cur)
    cx.sync()
    e_ms = cx.max_over_ranks(e0.elapsed_time(e1) / n_e2e)
    got = D_ps[0].numpy()[rows]
    want = want_full if world > 1 else want_full[:, n0:n0 + n_len]
    if not np.array_equal(got.view(np.uint16), np.ascontiguousarray(want).view(np.uint16)):
        raise SystemExit("parity check failed on the end-to-end path")
    path = ("pinned host -> cudaMemcpyAsync -> bm_w8a8_f16 -> cudaMemcpyAsync -> pinned host" if world == 1 else
            "on every rank: pinned host -> cudaMemcpyAsync (activations, weight slab, scales) -> ColumnShardedLinear.forward_fused "
            "(bm_w8a8_f16_gather + group barrier) -> cudaMemcpyAsync of the rank's full [M x N] output -> pinned host")
    return {"value": ops_step / (e_ms * 1e-3) / 1e12, "unit": UNIT,
            "h2d_bytes_per_step": int(M * K + n_len * K + 4 * (M + n_len)), "d2h_bytes_per_step": int(2 * M * n_out),
            "bytes_note": "per rank" if world > 1 else "single GPU", "ms_per_step": e_ms, "steps": n_e2e,
            "path": path + "; copy-in, GEMM and copy-out of neighbouring steps overlap on three streams (two buffer sets)"}


def profile_side_workload(args, ig, oracle, torch, devn):
    """Profiler-friendly run of one side workload: warm-up + steps launches of a single kernel."""
    sid = oracle.stream_id
    if args.workload == "sparse":
        Ms = Ns = Ks = 4096
        comp, nib = oracle.gen_sparse_rows(Ns, Ks, 0, sid("C3", "W"))
        sets = 4
        X_d = [torch.from_numpy(oracle.gen_int8((Ms, Ks), 0, sid("C3", "A"))).to(devn) for _ in range(sets)]
        comp_d = [torch.from_numpy(comp).to(devn) for _ in range(sets)]
        til_d = [ig.sp_pack_meta(torch.from_numpy(nib).to(devn), ig.BM_META_ROWS, Ns, Ks) for _ in range(sets)]
        C_d = [torch.empty((Ms, Ns), dtype=torch.int32, device=devn) for _ in range(sets)]
        fn = lambda i: ig.w8a8_sparse_i32(X_d[i % sets], comp_d[i % sets], til_d[i % sets], C_d[i % sets], Ms, Ns, Ks)
        work = 2.0 * Ms * Ns * Ks
        unit = "dense-equiv TOPS"
    elif args.workload == "online_quant":
        Mo = No = Ko = 4096                  # 3 x (32 + 32) MiB of fp16 operands > L2
        Ao = [torch.rand((Mo, Ko), device=devn, dtype=torch.float16) * 2 - 1 for _ in range(3)]
        Bo = [torch.rand((Ko, No), device=devn, dtype=torch.float16) * 2 - 1 for _ in range(3)]
        Co = torch.empty((Mo, No), dtype=torch.float32, device=devn)
        fn = lambda i: ig.igemm_online_quant(Ao[i % 3], Bo[i % 3], Co, Mo, No, Ko)
        work = 2.0 * Mo * No * Ko
        unit = "TOPS"
    elif args.workload == "hgemm_sparse":
        Mh = Nh = Kh = 4096
        comp_h = [(torch.rand((Mh, Kh // 2), device=devn) * 2 - 1).half() for _ in range(3)]
        B_h = [(torch.rand((Kh, Nh), device=devn) * 2 - 1).half() for _ in range(3)]
        nib_h = torch.from_numpy(oracle.gen_sparse_rows(Mh, Kh, 0, sid("H", "A"))[1]).to(devn)
        til_h = ig.sp_pack_meta(nib_h, ig.BM_META_ROWS_F16, Mh, Kh)
        C_h = torch.empty((Mh, Nh), dtype=torch.float32, device=devn)
        fn = lambda i: ig.hgemm_sparse_tiled(comp_h[i % 3], B_h[i % 3], C_h, til_h, Mh, Nh, Kh, ig.BM_META_TILED)
        work = 2.0 * Mh * Nh * Kh
        unit = "dense-equiv TFLOPS"
    else:
        Nd, Kd, Md = 28672, 8192, args.decode_m
        comp, nib = oracle.gen_sparse_rows(Nd, Kd, 0, sid("C5", "W"))
        comp_0, nib_0 = torch.from_numpy(comp).to(devn), torch.from_numpy(nib).to(devn)
        pk_d = [ig.sp_pack_weights(comp_0, nib_0, ig.BM_META_ROWS, Nd, Kd) for _ in range(2)]
        del comp_0, nib_0
        sw = torch.from_numpy(oracle.gen_scales(Nd, 0, sid("C5", "sw"))).to(devn)
        Xd = torch.from_numpy(oracle.gen_int8((Md, Kd), 0, sid("C5", "X1"))).to(devn)
        sa = torch.from_numpy(oracle.gen_scales(Md, 0, sid("C5", "sa"))).to(devn)
        Dd = torch.empty((Md, Nd), dtype=torch.float16, device=devn)
        fn = lambda i: ig.w8a8_sparse_linear_packed(Xd, pk_d[i % 2], Dd, sa, sw, Md, Nd, Kd)
        work = Nd * Kd / 2 + Nd * Kd / 8 + Md * Kd + 2 * Md * Nd + 4 * (Md + Nd)
        unit = "GB/s"
    torch.cuda.synchronize()                 # set-up (packing kernels) is over before the profiled launches
    for i in range(args.warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    value = work / ms / 1e6 if args.workload == "decode" else work / ms / 1e9
    print(json.dumps({"profile_run": True, "workload": args.workload, "value": value, "unit": unit, "ms_per_step": ms}),
          flush=True)


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the benchmarked kernel (33.654 MB read + 2.532 MB
# written), from the ncu capture of the dense pair kernel at this workload; refreshed with the kernel.
TRAFFIC_BYTES_NCU = 36_187_000
TRAFFIC_DECODE_M1_NCU = 150_725_000      # 146.975 MB read + 3.75 MB written, M = 1
# operand bytes per tensor clock an SM can pull from L2 when all 148 pull at once (TMA fill microbenchmark)
L2_FILL_B_PER_CLK_SM = 75.0


def side_measurements(cx, ig, oracle, torch, devn, peaks, _lib):
    """2:4-sparse 4096^3 and decode-shaped sparse GEMV, reported beside the headline, each with its own roofline
    fraction; then the steps either side of the path and the 8192-token layer chain."""
    out = {}
    timeit = lambda fn, iters, warm=5: cx.timeit(fn, iters, warm)
    sid = oracle.stream_id
    # 2:4-sparse weights at 4096^3, int32 out, against the dense kernel on the same box
    Ms = Ns = Ks = 4096
    comp, nib = oracle.gen_sparse_rows(Ns, Ks, 0, sid("C3", "W"))
    X = oracle.gen_int8((Ms, Ks), 0, sid("C3", "A"))
    sets = 6
    comp_d = [torch.from_numpy(comp).to(devn) for _ in range(sets)]
    til_d = [ig.sp_pack_meta(torch.from_numpy(nib).to(devn), ig.BM_META_ROWS, Ns, Ks) for _ in range(sets)]
    X_d = [torch.from_numpy(X).to(devn) for _ in range(sets)]
    C_d = [torch.empty((Ms, Ns), dtype=torch.int32, device=devn) for _ in range(sets)]
    ms = timeit(lambda i: ig.w8a8_sparse_i32(X_d[i % sets], comp_d[i % sets], til_d[i % sets], C_d[i % sets], Ms, Ns, Ks), 100)
    Wd_d = [torch.from_numpy(oracle.decompress_rows(comp, nib)).to(devn) for _ in range(2)]
    ms_dense = timeit(lambda i: ig.igemm_i32(X_d[i % sets], Wd_d[i % 2], C_d[i % sets], Ms, Ns, Ks, ig.BM_B_NK), 50)
    tops = 2.0 * Ms * Ns * Ks / ms / 1e9
    # per CTA and 256-wide K block the pair kernel stages 50 KiB for 480 tensor clocks of sparse MMA: 107 B/clk/SM
    # asked of an L2 that delivers ~75 — the operand fill, not the tensor pipe, bounds it
    need_b_per_clk = 50 * 1024 / 480.0
    sparse_peak = 2.0 * 2.0 * peaks["bf16_tflops"]
    out["sparse_2to4_4096"] = {"ms": ms, "dense_equiv_tops": tops, "dense_same_box_ms": ms_dense,
                               "ratio_to_dense": ms_dense / ms, "l2": f"{sets} rotating operand sets",
                               "roofline": {"bound": "l2 operand fill", "achieved": tops, "unit": "dense-equiv TOP/s",
                                            "peak": sparse_peak * L2_FILL_B_PER_CLK_SM / need_b_per_clk,
                                            "frac": tops / (sparse_peak * L2_FILL_B_PER_CLK_SM / need_b_per_clk),
                                            "tensor_peak": sparse_peak, "frac_of_tensor_peak": tops / sparse_peak,
                                            "operand_bytes_per_clk_sm_needed": need_b_per_clk,
                                            "operand_bytes_per_clk_sm_l2_ceiling": L2_FILL_B_PER_CLK_SM,
                                            "peak_note": "sparse tensor peak (4 x measured bf16 burst) scaled by the measured L2 fill "
                                                         "ceiling over the bytes per tensor clock this tile shape needs"}}
    del comp_d, til_d, X_d, C_d, Wd_d
    # decode shapes
    Nd, Kd = 28672, 8192
    comp, nib = oracle.gen_sparse_rows(Nd, Kd, 0, sid("C5", "W"))
    # weights in the library's packed form (one-time repack of values + positions into contiguous 20 KiB blocks,
    # bm_sp_pack_weights; same bytes, not part of the step), two copies in rotation: 2 x 147 MB > L2
    comp_0, nib_0 = torch.from_numpy(comp).to(devn), torch.from_numpy(nib).to(devn)
    pk_d = [ig.sp_pack_weights(comp_0, nib_0, ig.BM_META_ROWS, Nd, Kd) for _ in range(2)]
    comp_d = [comp_0]
    til_d = [ig.sp_pack_meta(nib_0, ig.BM_META_ROWS, Nd, Kd)]
    sw = torch.from_numpy(oracle.gen_scales(Nd, 0, sid("C5", "sw"))).to(devn)
    dec = {"weights": "packed blocks (bm_sp_pack_weights), rows dealt to the CTAs in multiples of 8"}
    for Md in (1, 16, 64):
        Xd = torch.from_numpy(oracle.gen_int8((Md, Kd), 0, sid("C5", f"X{Md}"))).to(devn)
        sa = torch.from_numpy(oracle.gen_scales(Md, 0, sid("C5", "sa"))).to(devn)
        Dd = torch.empty((Md, Nd), dtype=torch.float16, device=devn)
        ms = timeit(lambda i: ig.w8a8_sparse_linear_packed(Xd, pk_d[i % 2], Dd, sa, sw, Md, Nd, Kd), 60)
        # same result as the unpacked entry point (bits)
        D2 = torch.empty_like(Dd)
        ig.w8a8_sparse_linear(Xd, comp_d[0], til_d[0], D2, sa, sw, Md, Nd, Kd)
        if not torch.equal(Dd, D2):
            raise SystemExit("parity check failed: packed and unpacked decode paths disagree")
        byts = Nd * Kd / 2 + Nd * Kd / 8 + Md * Kd + 2 * Md * Nd + 4 * (Md + Nd)
        gbs = byts / ms / 1e6
        dec[f"M{Md}"] = {"us": ms * 1e3, "algorithmic_bytes": byts, "gb_per_s": gbs,
                         "frac_of_hbm_peak": gbs / peaks["hbm_gbs"], "frac_of_nominal_8tbs": gbs / NOMINAL_HBM_GBS,
                         "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                      "frac": gbs / peaks["hbm_gbs"],
                                      "traffic": TRAFFIC_DECODE_M1_NCU if Md == 1 else None}}
    out["decode_sparse_K8192_N28672"] = dec
    # host enqueue cost of one launcher call (argument checks, cached tensor maps, cudaLaunchKernelEx), GPU idle-bound
    Xd = torch.from_numpy(oracle.gen_int8((1, Kd), 0, sid("C5", "X1"))).to(devn)
    sa = torch.from_numpy(oracle.gen_scales(1, 0, sid("C5", "sa"))).to(devn)
    Dd = torch.empty((1, Nd), dtype=torch.float16, device=devn)
    torch.cuda.synchronize()
    import ctypes
    L = _lib.load()
    argsv = (Xd.data_ptr(), comp_d[0].data_ptr(), til_d[0].data_ptr(), Dd.data_ptr(), sa.data_ptr(), sw.data_ptr(),
             1, Nd, Kd, Nd, torch.cuda.current_stream().cuda_stream)
    n_calls = 200
    t0 = time.perf_counter()
    for _ in range(n_calls):
        L.bm_w8a8_sparse_f16(*argsv)
    t_host = (time.perf_counter() - t0) / n_calls
    torch.cuda.synchronize()
    h, m_, e_ = ctypes.c_uint64(0), ctypes.c_uint64(0), ctypes.c_uint64(0)
    L.bm_tensor_map_cache_stats(ctypes.byref(h), ctypes.byref(m_), ctypes.byref(e_))
    out["host_enqueue"] = {"us_per_call": t_host * 1e6,
                           "what": "bm_w8a8_sparse_f16 (decode, M = 1) called back to back from one host thread through ctypes; "
                                   "while the GPU is slower than the host this includes waiting for a free launch slot",
                           "tensor_map_cache": {"hits": h.value, "encoded": m_.value, "entries": e_.value}}
    del comp_d, til_d, pk_d, comp_0, nib_0
    # the step before the path: per-token dynamic quantisation fp16 -> int8 (8192 tokens x 4096)
    Mq, Kq = 8192, 4096
    xs = [torch.randn((Mq, Kq), device=devn, dtype=torch.float16) for _ in range(4)]      # 4 x 64 MB > L2
    ms = timeit(lambda i: ig.quantize_rows(xs[i % 4], Mq, Kq), 40)
    qb = 3.0 * Mq * Kq + 4.0 * Mq
    out["quantize_rows_8192x4096"] = {"us": ms * 1e3, "algorithmic_bytes": qb, "gb_per_s": qb / ms / 1e6,
                                      "frac_of_hbm_peak": qb / ms / 1e6 / peaks["hbm_gbs"]}
    del xs
    # weight tooling: magnitude pruning to 2:4 + compression of a 28672 x 8192 int8 matrix (235 MB > L2)
    Rp, Kp = 28672, 8192
    Wp = torch.randint(-127, 128, (Rp, Kp), dtype=torch.int8, device=devn)
    ms = timeit(lambda i: ig.prune_2_4(Wp, Rp, Kp), 20)
    pb = 1.625 * Rp * Kp
    out["prune_2to4_28672x8192"] = {"us": ms * 1e3, "algorithmic_bytes": pb, "gb_per_s": pb / ms / 1e6,
                                    "frac_of_hbm_peak": pb / ms / 1e6 / peaks["hbm_gbs"]}
    del Wp
    # FP16-in GEMM with the reference's per-tile quantisation: two quantising passes + block-scaled GEMM
    Mo = No = Ko = 4096
    Ao = [torch.rand((Mo, Ko), device=devn, dtype=torch.float16) * 2 - 1 for _ in range(3)]
    Bo = [torch.rand((Ko, No), device=devn, dtype=torch.float16) * 2 - 1 for _ in range(3)]
    Co = torch.empty((Mo, No), dtype=torch.float32, device=devn)
    ms = timeit(lambda i: ig.igemm_online_quant(Ao[i % 3], Bo[i % 3], Co, Mo, No, Ko), 40)
    out["online_quant_fp16_4096"] = {"ms": ms, "tops": 2.0 * Mo * No * Ko / ms / 1e9}
    del Ao, Bo, Co
    # FP16 2:4 sparse GEMM (kernels/gemm/hgemm_sparse), 4096^3, metadata tiled once
    Mh = Nh = Kh = 4096
    comp_h = [(torch.rand((Mh, Kh // 2), device=devn) * 2 - 1).half() for _ in range(3)]
    B_h = [(torch.rand((Kh, Nh), device=devn) * 2 - 1).half() for _ in range(3)]
    nib_h = torch.from_numpy(oracle.gen_sparse_rows(Mh, Kh, 0, sid("H", "A"))[1]).to(devn)
    til_h = ig.sp_pack_meta(nib_h, ig.BM_META_ROWS_F16, Mh, Kh)
    C_h = torch.empty((Mh, Nh), dtype=torch.float32, device=devn)
    ms = timeit(lambda i: ig.hgemm_sparse_tiled(comp_h[i % 3], B_h[i % 3], C_h, til_h, Mh, Nh, Kh, ig.BM_META_TILED), 30)
    out["hgemm_sparse_fp16_4096"] = {"ms": ms, "dense_equiv_tflops": 2.0 * Mh * Nh * Kh / ms / 1e9}
    del comp_h, B_h, C_h
    # the four GEMMs of one 8192-token transformer layer, W8A8 -> fp16
    Mc = 8192
    chain = {}
    total_ms, total_ops = 0.0, 0.0
    int8_peak = 2.0 * peaks["bf16_tflops"]
    for name, Kc, Nc in (("qkv", 4096, 12288), ("out", 4096, 4096), ("gate_up", 4096, 22016), ("down", 11008, 4096)):
        Xc = torch.randint(-127, 128, (Mc, Kc), dtype=torch.int8, device=devn)
        Wc = [torch.randint(-127, 128, (Nc, Kc), dtype=torch.int8, device=devn) for _ in range(2)]
        sac = torch.rand(Mc, device=devn) * 0.019 + 0.001
        swc = torch.rand(Nc, device=devn) * 0.019 + 0.001
        Dc = torch.empty((Mc, Nc), dtype=torch.float16, device=devn)
        ms = timeit(lambda i: ig.w8a8_linear(Xc, Wc[i % 2], Dc, sac, swc, Mc, Nc, Kc), 20)
        ops = 2.0 * Mc * Nc * Kc
        chain[name] = {"ms": ms, "tops": ops / ms / 1e9, "frac_of_2x_measured_bf16": ops / ms / 1e9 / int8_peak}
        total_ms += ms
        total_ops += ops
        del Xc, Wc, Dc
    chain["layer"] = {"ms": total_ms, "tops": total_ops / total_ms / 1e9,
                      "frac_of_2x_measured_bf16": total_ops / total_ms / 1e9 / int8_peak}
    out["layer_chain_8192_tokens"] = chain
    out["hbm_peak_gbs"] = peaks["hbm_gbs"]
    return out


if __name__ == "__main__":
    main()
