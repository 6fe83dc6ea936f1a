#!/usr/bin/env python
"""Benchmark of the B200-native INT8 GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE config 2): W8A8 GEMM M=N=K=4096, int8 operands uniform on [-127,127],
per-row activation scale and per-column weight scale ~ U[1e-3, 2e-2], fp16 output
D = half_rn(float(A.W^T) * sa[m]*sw[n]), int32 accumulate.  A "step" is one such GEMM.
With N > 1 the weight columns are split: every rank owns a 4096-column slab (global
N = 4096*N, weak scaling), computes its slab and the fp16 outputs are all-gathered.

Prints ONE JSON line (rank 0).  `value` is dense-equivalent TOPS with operands resident in
HBM; `e2e` is the same metric through the C ABI with HOST buffers (H2D of both operands and
the scales, D2H of the result, inside the timed region).  `--impl reference` times the
reference project's own CPU verification GEMM (cpu_sparse_gemm_int8, compiled in place into
oracle/_ref) on the host cores instead.
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

M = N_LOCAL = K = 4096
METRIC = "INT8 dense-equiv TOPS at 4096^3 (W8A8 dense, fp16 out)"
UNIT = "TOPS"
NOMINAL_INT8_TOPS = 4500.0          # B200 dense INT8 datasheet figure


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


def reference_arm(args, rank: int, world: int) -> None:
    """The reference's own CPU verification GEMM on the host cores (rank 0 only)."""
    if rank != 0:
        return
    import numpy as np
    import oracle
    kind = "reference" if oracle.have_ref() else "port"
    cores = os.cpu_count() or 1
    A = oracle.gen_int8((M, K), 0, oracle.stream_id("C2", "A"))
    B = oracle.gen_int8((K, N_LOCAL), 0, oracle.stream_id("C2", "Wt"))

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
    tops = 2.0 * rows * N_LOCAL * K / dt / 1e12
    sample = f"{rows} of {M} rows of the 4096^3 integer GEMM per step, {cores} host threads on row slabs"
    line = {"impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "s8*s8->s32", "data": "synthetic",
            "config": {"workload": "C2 W8A8 GEMM M=N=K=4096 (integer core on CPU)", "sample": sample},
            "cpu_baseline": {"value": tops, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def cpu_baseline_leg():
    import numpy as np
    import oracle
    kind = "reference" if oracle.have_ref() else "port"
    cores = os.cpu_count() or 1
    A = oracle.gen_int8((M, K), 0, oracle.stream_id("C2", "A"))
    B = oracle.gen_int8((K, N_LOCAL), 0, oracle.stream_id("C2", "Wt"))
    rows = min(M, max(cores * 8, 1024))
    a = np.ascontiguousarray(A[:rows])
    fn = (lambda: oracle.ref_cpu_sparse_gemm_int8(a, B, threads=cores)) if kind == "reference" else \
         (lambda: oracle.igemm(a, B, threads=cores))
    fn()
    reps, t0 = 0, time.perf_counter()
    while reps < 3 or (time.perf_counter() - t0 < 4.0 and reps < 50):
        fn(); reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": 2.0 * rows * N_LOCAL * K / dt / 1e12, "unit": UNIT, "cores": cores, "kind": kind,
            "sample": f"{rows} of {M} rows of the 4096^3 integer GEMM, x{reps}, {cores} host threads on row slabs"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the sparse / decode side measurements")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N > 1: fused = GEMM epilogue stores to all ranks over NVLink; nccl = GEMM then all-gather")
    ap.add_argument("--workload", default="dense", choices=["dense", "sparse", "decode", "online_quant", "hgemm_sparse"],
                    help="with --profile: which kernel to run (dense = the headline; sparse = config 3; "
                         "decode = config 5 at M=1)")
    ap.add_argument("--decode-m", type=int, default=1, help="with --profile --workload decode: number of tokens (1, 16, 64)")
    ap.add_argument("--profile", action="store_true",
                    help="profiler-friendly run: only warm-up + the timed steps of the headline kernel")
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
    import oracle                      # data generators + the cpu_baseline leg only
    import bare_metal_b200 as bm
    from bare_metal_b200 import igemm as ig

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback exists)")
    torch.cuda.set_device(local_rank)
    devn = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=devn)
    bm.build()
    peaks = load_peaks()

    if args.profile and args.workload != "dense":
        profile_side_workload(args, ig, oracle, torch, devn)
        return

    # ---- operands: enough rotating sets that consecutive steps never hit L2 (126 MB) -------------
    n_total = N_LOCAL * world
    set_bytes = M * K + N_LOCAL * K + 2 * M * N_LOCAL
    n_sets = max(2, -(-3 * 126 * 2 ** 20 // set_bytes))          # > 3x L2 in flight
    sid = oracle.stream_id
    A_h = oracle.gen_int8((M, K), 0, sid("C2", "A"))
    W_h = oracle.gen_int8((N_LOCAL, K), 0, sid("C2", f"W{rank}"))
    sa_h = oracle.gen_scales(M, 0, sid("C2", "sa"))
    sw_h = oracle.gen_scales(N_LOCAL, 0, sid("C2", f"sw{rank}"))
    A_d = [torch.from_numpy(A_h).to(devn) for _ in range(n_sets)]
    W_d = [torch.from_numpy(W_h).to(devn) for _ in range(n_sets)]
    sa_d, sw_d = torch.from_numpy(sa_h).to(devn), torch.from_numpy(sw_h).to(devn)
    D_d = [torch.empty((M, N_LOCAL), dtype=torch.float16, device=devn) for _ in range(n_sets)]
    layer = None
    if world > 1:
        from bare_metal_b200 import nsplit
        # every rank owns the 4096-column slab [rank*4096, +4096) of the global weight matrix; the
        # GEMM epilogue stores the slab into every rank's row-major output over NVLink (fused gather)
        layer = nsplit.ColumnShardedLinear(W_d[0], sw_d, n_total, rank * N_LOCAL, mode=args.gather)
        G_blocks = torch.empty((world, M, N_LOCAL), dtype=torch.float16, device=devn)

    def step(i: int):
        s = i % n_sets
        if world == 1:
            ig.w8a8_linear(A_d[s], W_d[s], D_d[s], sa_d, sw_d, M, N_LOCAL, K)
        elif args.gather == "fused":
            layer.W = W_d[s]
            layer.forward_fused(A_d[s], sa_d)
        else:
            layer.W = W_d[s]
            layer.forward_nccl(A_d[s], sa_d, out=G_blocks, local=D_d[s])

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- parity of what is being timed (one step against the CPU oracle on sampled rows) -----------
    step(0)
    torch.cuda.synchronize()
    rows = np.array([0, 1, 127, 128, 2047, 4095])
    want = oracle.dequant_w8a8_f16(oracle.igemm_nt(np.ascontiguousarray(A_h[rows]), W_h), sa_h[rows], sw_h)
    if world == 1:
        got = D_d[0].cpu().numpy()[rows]
    elif args.gather == "fused":
        full = layer._symmetric(M, devn)[0]
        got = full[:, rank * N_LOCAL:(rank + 1) * N_LOCAL].cpu().numpy()[rows]
        # the slab a PEER wrote into this rank's output must match that peer's weights too
        peer = (rank + 1) % world
        Wp = oracle.gen_int8((N_LOCAL, K), 0, sid("C2", f"W{peer}"))
        swp = oracle.gen_scales(N_LOCAL, 0, sid("C2", f"sw{peer}"))
        want_p = oracle.dequant_w8a8_f16(oracle.igemm_nt(np.ascontiguousarray(A_h[rows]), Wp), sa_h[rows], swp)
        got_p = full[:, peer * N_LOCAL:(peer + 1) * N_LOCAL].cpu().numpy()[rows]
        if not np.array_equal(got_p.view(np.uint16), want_p.view(np.uint16)):
            raise SystemExit("parity check failed: the slab stored by a peer GPU disagrees with the CPU oracle")
    else:
        got = G_blocks[rank].cpu().numpy()[rows]
    if not np.array_equal(got.view(np.uint16), want.view(np.uint16)):
        raise SystemExit("parity check failed: the benchmarked kernel disagrees with the CPU oracle")

    # ---- timed region ----------------------------------------------------------------------------
    for i in range(args.warmup):
        step(i)
    sync()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    # keep the region long enough for nvidia-smi to see it: repeat the K steps in rounds
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    t_wall0 = time.time()
    ev0.record()
    for i in range(args.steps):
        step(i)
    ev1.record()
    sync()
    ms_total = ev0.elapsed_time(ev1)
    # extra untimed load so the clock sampler has samples under load even for a short region
    t_load = time.time()
    j = 0
    while not args.profile and time.time() - t_load < 1.5:
        step(j); j += 1
        if j % 64 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    t_wall1 = time.time()
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms_total], dtype=torch.float64, device=devn)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    ops_step = 2.0 * M * n_total * K
    value = ops_step / (ms_step * 1e-3) / 1e12
    if args.profile:
        if rank == 0:
            print(json.dumps({"profile_run": True, "value": value, "unit": UNIT, "ms_per_step": ms_step}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- kernel-only duration for the roofline (the GEMM launch alone, same stream) ----------------
    ke0, ke1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    ke0.record()
    for i in range(args.steps):
        s = i % n_sets
        ig.w8a8_linear(A_d[s], W_d[s], D_d[s], sa_d, sw_d, M, N_LOCAL, K)
    ke1.record()
    torch.cuda.synchronize()
    kern_ms = ke0.elapsed_time(ke1) / args.steps
    achieved = 2.0 * M * N_LOCAL * K / (kern_ms * 1e-3) / 1e12
    int8_peak = 2.0 * peaks["bf16_tflops"]
    roofline = {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TOP/s",
                "frac": achieved / int8_peak,
                "peak_note": f"2 x cuBLAS bf16 burst ({peaks['bf16_tflops']} TFLOP/s, of {peaks['source']}); "
                             f"INT8 runs at twice the bf16 rate on this tensor core",
                "frac_of_nominal_4500": achieved / NOMINAL_INT8_TOPS,
                "kernel": "igemm_dense_pair_kernel<false,EPI_F16_ROWCOL>", "kernel_ms": kern_ms,
                "algorithmic_bytes": set_bytes,
                "traffic": TRAFFIC_BYTES_NCU}

    if world > 1:
        # fused GEMM + gather: the slower of the tensor time and the bytes a rank must RECEIVE over NVLink
        link_gbs = 770.0                                        # measured peer-copy bandwidth per direction
        recv_bytes = 2.0 * M * N_LOCAL * (world - 1)
        t_link_ms = recv_bytes / (link_gbs * 1e9) * 1e3
        target_ms = max(kern_ms, t_link_ms)
        roofline["fused_collective"] = {"bound": "nvlink" if t_link_ms > kern_ms else "tensor",
                                        "recv_bytes_per_rank": recv_bytes, "link_gb_per_s": link_gbs,
                                        "target_ms": target_ms, "achieved_ms": ms_step,
                                        "frac": target_ms / ms_step, "gemm_only_ms": kern_ms}

    # ---- end to end through the C ABI with host buffers --------------------------------------------
    e2e = None
    if rank == 0 or world > 1:
        pin = lambda a: torch.from_numpy(a).pin_memory()
        A_p, W_p, sa_p, sw_p = pin(A_h), pin(W_h), pin(sa_h), pin(sw_h)
        D_p = torch.empty((M, N_LOCAL), dtype=torch.float16).pin_memory()
        # Three streams, two buffer sets: the copy-in of step i+1, the GEMM of step i and the copy-out of
        # step i-1 overlap (PCIe is full duplex); every step still moves all of its inputs and its output.
        NB = 2
        A_e = [torch.empty_like(A_d[0]) for _ in range(NB)]
        W_e = [torch.empty_like(W_d[0]) for _ in range(NB)]
        sa_e = [torch.empty_like(sa_d) for _ in range(NB)]
        sw_e = [torch.empty_like(sw_d) for _ in range(NB)]
        D_e = [torch.empty((M, N_LOCAL), dtype=torch.float16, device=devn) for _ in range(NB)]
        D_ps = [D_p] + [torch.empty((M, N_LOCAL), dtype=torch.float16).pin_memory() for _ in range(NB - 1)]
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
                ig.w8a8_linear(A_e[b], W_e[b], D_e[b], sa_e[b], sw_e[b], M, N_LOCAL, K)
                ev_mm[b].record(s_mm)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_mm[b])
                D_ps[b].copy_(D_e[b], non_blocking=True)
                ev_out[b].record(s_out)

        n_e2e = max(6, min(args.steps, 30))
        n_e2e += n_e2e % NB                                   # the last step lands in D_p (set 0 ... NB-1 in turn)
        for _ in range(2 * NB):
            e2e_step()
        sync()
        step_no[0] = 1                                        # so that the final timed step uses set 0 = D_p
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
        sync()
        e_ms = e0.elapsed_time(e1) / n_e2e
        if world > 1:
            t = torch.tensor([e_ms], dtype=torch.float64, device=devn)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e_ms = float(t.item())
        if not np.array_equal(D_p.numpy()[rows].view(np.uint16), want.view(np.uint16)):
            raise SystemExit("parity check failed on the end-to-end path")
        e2e = {"value": ops_step / (e_ms * 1e-3) / 1e12, "unit": UNIT,
               "h2d_bytes_per_step": int(M * K + N_LOCAL * K + 4 * (M + N_LOCAL)),
               "d2h_bytes_per_step": int(2 * M * N_LOCAL), "ms_per_step": e_ms, "steps": n_e2e,
               "path": "pinned host -> cudaMemcpyAsync -> bm_w8a8_f16 -> cudaMemcpyAsync -> pinned host; "
                       "copy-in, GEMM and copy-out of neighbouring steps overlap on three streams (two buffer sets)"}

    # ---- side measurements: 2:4 sparse 4096^3 and the decode shapes (not the headline) -------------
    extras = {}
    if rank == 0 and not args.no_extras:
        extras = side_measurements(ig, oracle, torch, devn, peaks)

    if rank == 0:
        cpu = None if args.no_cpu_baseline else cpu_baseline_leg()
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "s8*s8->s32 (fp32 scale, fp16 out)", "data": "synthetic",
                "config": {"workload": f"C2 W8A8 GEMM M={M} K={K} N={n_total} ({N_LOCAL} weight columns per GPU)",
                           "parallelism": f"n-split x{world}" + ("" if world == 1 else (
                               " + all-gather of the fp16 output fused into the GEMM epilogue (peer TMA stores)"
                               if args.gather == "fused" else " + NCCL all-gather of the fp16 output")),
                           "l2": f"{n_sets} rotating operand sets ({n_sets * set_bytes / 2**20:.0f} MiB) exceed the 126 MiB L2",
                           "tile": "CTA pairs (cta_group::2), 256x256x128 per pair, 4-stage TMA ring, 2 TMEM accumulators"},
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": args.steps,
                "clocks": clocks, "extras": extras}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


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
        comp_d = [torch.from_numpy(comp).to(devn) for _ in range(2)]
        til_d = [ig.sp_pack_meta(torch.from_numpy(nib).to(devn), ig.BM_META_ROWS, Nd, Kd) for _ in range(2)]
        sw = torch.from_numpy(oracle.gen_scales(Nd, 0, sid("C5", "sw"))).to(devn)
        Xd = torch.from_numpy(oracle.gen_int8((Md, Kd), 0, sid("C5", "X1"))).to(devn)
        sa = torch.from_numpy(oracle.gen_scales(Md, 0, sid("C5", "sa"))).to(devn)
        Dd = torch.empty((Md, Nd), dtype=torch.float16, device=devn)
        fn = lambda i: ig.w8a8_sparse_linear(Xd, comp_d[i % 2], til_d[i % 2], Dd, sa, sw, Md, Nd, Kd)
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


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the benchmarked kernel, from the
# committed ncu capture (profiles/); None until one exists for this kernel build.
TRAFFIC_BYTES_NCU = 36_187_000   # 33.654 MB read + 2.532 MB written (profiles/igemm_dense_pair_w8a8_4096_ncu_full.md)


def side_measurements(ig, oracle, torch, devn, peaks):
    """2:4-sparse 4096^3 (config 3) and decode-shaped sparse GEMV (config 5): reported beside the
    headline, each with its own roofline fraction."""
    out = {}

    def timeit(fn, iters, warm=5):
        for i in range(warm):
            fn(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    sid = oracle.stream_id
    # config 3
    Ms = Ns = Ks = 4096
    comp, nib = oracle.gen_sparse_rows(Ns, Ks, 0, sid("C3", "W"))
    X = oracle.gen_int8((Ms, Ks), 0, sid("C3", "A"))
    sets = 6
    comp_d = [torch.from_numpy(comp).to(devn) for _ in range(sets)]
    til_d = [ig.sp_pack_meta(torch.from_numpy(nib).to(devn), ig.BM_META_ROWS, Ns, Ks) for _ in range(sets)]
    X_d = [torch.from_numpy(X).to(devn) for _ in range(sets)]
    C_d = [torch.empty((Ms, Ns), dtype=torch.int32, device=devn) for _ in range(sets)]
    ms = timeit(lambda i: ig.w8a8_sparse_i32(X_d[i % sets], comp_d[i % sets], til_d[i % sets], C_d[i % sets], Ms, Ns, Ks), 100)
    out["sparse_2to4_4096"] = {"ms": ms, "dense_equiv_tops": 2.0 * Ms * Ns * Ks / ms / 1e9,
                               "l2": f"{sets} rotating operand sets"}
    del comp_d, til_d, X_d, C_d
    # config 5
    Nd, Kd = 28672, 8192
    comp, nib = oracle.gen_sparse_rows(Nd, Kd, 0, sid("C5", "W"))
    comp_d = [torch.from_numpy(comp).to(devn) for _ in range(2)]       # 2 x 147 MB > L2
    til_d = [ig.sp_pack_meta(torch.from_numpy(nib).to(devn), ig.BM_META_ROWS, Nd, Kd) for _ in range(2)]
    sw = torch.from_numpy(oracle.gen_scales(Nd, 0, sid("C5", "sw"))).to(devn)
    dec = {}
    for Md in (1, 16, 64):
        Xd = torch.from_numpy(oracle.gen_int8((Md, Kd), 0, sid("C5", f"X{Md}"))).to(devn)
        sa = torch.from_numpy(oracle.gen_scales(Md, 0, sid("C5", "sa"))).to(devn)
        Dd = torch.empty((Md, Nd), dtype=torch.float16, device=devn)
        ms = timeit(lambda i: ig.w8a8_sparse_linear(Xd, comp_d[i % 2], til_d[i % 2], Dd, sa, sw, Md, Nd, Kd), 60)
        byts = Nd * Kd / 2 + Nd * Kd / 8 + Md * Kd + 2 * Md * Nd + 4 * (Md + Nd)
        gbs = byts / ms / 1e6
        dec[f"M{Md}"] = {"us": ms * 1e3, "algorithmic_bytes": byts, "gb_per_s": gbs,
                         "frac_of_hbm_peak": gbs / peaks["hbm_gbs"],
                         "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                      "frac": gbs / peaks["hbm_gbs"],
                                      "traffic": 150_725_000 if Md == 1 else None}}
    out["decode_sparse_K8192_N28672"] = dec
    del comp_d, til_d
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
    # config 4: the four GEMMs of one 8192-token transformer layer, W8A8 -> fp16
    Mc = 8192
    chain = {}
    total_ms, total_ops = 0.0, 0.0
    for name, Kc, Nc in (("qkv", 4096, 12288), ("out", 4096, 4096), ("gate_up", 4096, 22016), ("down", 11008, 4096)):
        Xc = torch.randint(-127, 128, (Mc, Kc), dtype=torch.int8, device=devn)
        Wc = [torch.randint(-127, 128, (Nc, Kc), dtype=torch.int8, device=devn) for _ in range(2)]
        sac = torch.rand(Mc, device=devn) * 0.019 + 0.001
        swc = torch.rand(Nc, device=devn) * 0.019 + 0.001
        Dc = torch.empty((Mc, Nc), dtype=torch.float16, device=devn)
        ms = timeit(lambda i: ig.w8a8_linear(Xc, Wc[i % 2], Dc, sac, swc, Mc, Nc, Kc), 20)
        ops = 2.0 * Mc * Nc * Kc
        chain[name] = {"ms": ms, "tops": ops / ms / 1e9}
        total_ms += ms
        total_ops += ops
        del Xc, Wc, Dc
    chain["layer"] = {"ms": total_ms, "tops": total_ops / total_ms / 1e9}
    out["layer_chain_8192_tokens"] = chain
    out["hbm_peak_gbs"] = peaks["hbm_gbs"]
    return out


if __name__ == "__main__":
    main()
