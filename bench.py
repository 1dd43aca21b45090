#!/usr/bin/env python
"""Benchmark of the fused-reduce hot path (the reduction sweep configuration).

A step = one pass over the sweep: {sum, max, mean, argmax} x axis {0, 1, -1} x
{A [8192,8192], B [64,4096,1024], B.permute(0,2,1) as a strided view}, each as
ONE fused kernel call with prologue x*1.5+0.25 and epilogue exp (no epilogue
for argmax) = 36 calls, fp32, seeded synthetic N(0,1) inputs.

Metric: fused-reduce HBM GB/s = algorithmic bytes (inputs read once + outputs
written once) / device time, CUDA events on the launching stream, max over
ranks. With N > 1 GPUs every rank runs the sweep on its own tensors (weak
scaling, no collective in the data path).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

`--impl reference` times the reference's CPU backend (its own reduce / binary
templates where they were compiled into oracle/_ref, else the C restatement)
on the host cores, on a bounded sample of the same sweep.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

AFFINE = [("LOAD", 0), ("IMM", 0, 0, 0, 1.5), ("MUL", 0, 1), ("IMM", 0, 0, 0, 0.25), ("ADD", 2, 3)]
EXP_EPI = [("ACC",), ("EXP", 0)]
OPS = ["sum", "max", "mean", "argmax"]
WORKLOAD = ("reduction sweep: sum/max/mean/argmax x axis 0/1/-1 x A[8192,8192], B[64,4096,1024], "
            "B.permute(0,2,1) view; prologue x*1.5+0.25, epilogue exp; one fused kernel per case")
SHAPES = {"A": (8192, 8192), "B": (64, 4096, 1024), "Bp": (64, 1024, 4096)}
# dram__bytes_read.sum + dram__bytes_write.sum per launch, averaged over the launches of one step of
# each kernel family, from the ncu capture summarised in profiles/reduce_sweep_dram_traffic.md
NCU_TRAFFIC_PER_LAUNCH = {"col": 916197568, "row": 672153568}


def case_list():
    """(tensor name, op, axis, algorithmic bytes) in an order that alternates tensors."""
    per = {}
    for name, shape in SHAPES.items():
        per[name] = []
        for ax in (0, 1, -1):
            for op in OPS:
                n_in = int(np.prod(shape))
                n_out = n_in // shape[ax]
                per[name].append((name, op, ax, 4 * n_in + 4 * n_out))
    out = []
    for i in range(12):
        out += [per["A"][i], per["B"][i], per["Bp"][i]]
    return out


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------
def cpu_sweep_sample(budget_s: float, threads: int):
    """The reference CPU backend's eager chain (2 binary kernels, per-axis reduce, exp)
    on cases of the sweep until `budget_s` is spent. Returns (bytes, seconds, desc, kind)."""
    import oracle
    from oracle.chain import fused_reduce_oracle
    kind = "reference" if oracle.have_ref() else "port"
    impl = "ref" if kind == "reference" else "port"
    rng = np.random.default_rng(2)
    A = rng.standard_normal(SHAPES["A"], dtype=np.float32)
    done_bytes, t_total, n = 0, 0.0, 0
    a_cases = [c for c in case_list() if c[0] == "A"]
    while t_total < budget_s:
        for name, op, ax, nbytes in a_cases:
            t0 = time.perf_counter()
            if op == "argmax":
                fused_reduce_oracle([A], op, [ax], False, AFFINE, (), impl=impl)
            else:
                fused_reduce_oracle([A], op, [ax], False, AFFINE, EXP_EPI, impl=impl)
            t_total += time.perf_counter() - t0
            done_bytes += nbytes
            n += 1
            if t_total >= budget_s:
                break
    return done_bytes, t_total, (f"{n} case runs cycling through the 12 cases on A[8192,8192] (eager chain: mul, add, reduce, exp), "
                                 f"{t_total:.1f} s of CPU work, {threads} OpenMP threads"), kind


def run_reference(args, rank: int):
    if rank != 0:
        return
    threads = len(os.sched_getaffinity(0))
    os.environ.setdefault("OMP_NUM_THREADS", str(threads))
    budget = 6.0
    for _ in range(args.warmup if args.warmup < 2 else 1):
        cpu_sweep_sample(0.5, threads)
    vals, ms = [], []
    for _ in range(max(1, min(args.steps, 3))):
        b, t, sample, kind = cpu_sweep_sample(budget, threads)
        vals.append(b / t / 1e9)
        ms.append(t * 1e3)
    v = statistics.median(vals)
    line = {
        "impl": "reference", "metric": "fused-reduce HBM GB/s", "value": v, "unit": "GB/s", "n_gpus": args.gpus, "steps": len(vals),
        "warmup": 1, "ms_per_step": statistics.median(ms), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": v, "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="pgb200", choices=["pgb200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--only", default="", help="comma-separated tensor names (A,B,Bp) to restrict the sweep, for profiling")
    ap.add_argument("--bare", action="store_true", help="diagnostic: no prologue / epilogue (not the benchmark workload)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    from pequegrad_b200 import _lib as L
    from pequegrad_b200 import kernels as K

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # per-rank synthetic tensors (rank-seeded; rank 0 uses the configured seed 2)
    g = torch.Generator(device=dev).manual_seed(2 + rank)
    only = set(filter(None, args.only.split(",")))
    T = {}
    if not only or "A" in only:
        T["A"] = torch.randn(SHAPES["A"], generator=g, device=dev)
    if not only or only & {"B", "Bp"}:
        T["B"] = torch.randn(SHAPES["B"], generator=g, device=dev)
        T["Bp"] = T["B"].permute(0, 2, 1)
    cases = [c for c in case_list() if not only or c[0] in only]
    opcode = {"sum": L.SUM, "max": L.MAX, "mean": L.MEAN, "argmax": L.ARGMAX}
    prepared = []
    for name, op, ax, nbytes in cases:
        if args.bare:
            pr = K.PreparedReduce([T[name]], opcode[op], [ax], False)
        else:
            pr = K.PreparedReduce([T[name]], opcode[op], [ax], False, AFFINE, () if op == "argmax" else EXP_EPI)
        prepared.append((name, op, ax, nbytes, pr))
    bytes_per_step = sum(c[3] for c in cases)
    stream = torch.cuda.current_stream().cuda_stream

    def step():
        for _, _, _, _, pr in prepared:
            pr(stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.2)
    launches0 = L.lib().pgb_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    launches = L.lib().pgb_launch_count() - launches0
    ms_total = e0.elapsed_time(e1)

    # per-case device time (CUDA events around each launch), still under the clock sampler
    reps = max(5, args.steps)
    per_case = []
    for name, op, ax, nbytes, pr in prepared:
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
        for a, b in evs:
            # touch the other big tensor first so nothing of this case's input is left in L2
            other = prepared[0][4] if name != prepared[0][0] else prepared[min(1, len(prepared) - 1)][4]
            other(stream)
            a.record()
            pr(stream)
            b.record()
        torch.cuda.synchronize()
        t = statistics.median(a.elapsed_time(b) for a, b in evs)
        per_case.append({"case": f"{name}.{op}.ax{ax}", "us": round(t * 1e3, 2), "gbs": round(nbytes / t / 1e6, 1),
                         "kernel": pr.plan.split()[0], "bytes": nbytes})
    clocks = sampler.stop()

    # end to end through the public call: pinned host inputs -> device, sweep, results -> host
    host_in = {k: torch.empty(SHAPES[k], dtype=torch.float32).pin_memory() for k in ("A", "B") if k in T}
    for k in host_in:
        host_in[k].copy_(T[k])
    host_out = [torch.empty(pr.out.shape, dtype=pr.out.dtype).pin_memory() for *_, pr in prepared]
    h2d = sum(v.numel() * 4 for v in host_in.values())
    d2h = sum(o.numel() * o.element_size() for o in host_out)

    def e2e_step():
        for k, v in host_in.items():
            T[k].copy_(v, non_blocking=True)
        step()
        for o, (*_, pr) in zip(host_out, prepared):
            o.copy_(pr.out, non_blocking=True)

    e2e_step()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n_e2e = max(2, min(args.steps, 5))
    f0.record()
    for _ in range(n_e2e):
        e2e_step()
    f1.record()
    barrier()
    e2e_ms = f0.elapsed_time(f1) / n_e2e

    ms = torch.tensor([ms_total, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms = float(ms[0]), float(ms[1])
    ms_per_step = ms_total / args.steps
    value = world * bytes_per_step / (ms_per_step * 1e-3) / 1e9
    e2e_value = world * bytes_per_step / (e2e_ms * 1e-3) / 1e9

    if rank == 0:
        peak, peak_src = peaks()
        fam = {}
        for c in per_case:
            f = fam.setdefault(c["kernel"], {"us": 0.0, "bytes": 0, "launches": 0})
            f["us"] += c["us"]
            f["bytes"] += c["bytes"]
            f["launches"] += 1
        dom = max(fam, key=lambda k: fam[k]["us"])
        achieved = fam[dom]["bytes"] / (fam[dom]["us"] * 1e-6) / 1e9
        roofline = {"bound": "hbm", "kernel": f"reduce_{dom}_kernel", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                    "frac": round(achieved / peak, 4), "peak_source": peak_src,
                    "traffic": NCU_TRAFFIC_PER_LAUNCH.get(dom) if not only and not args.bare else None,
                    "algorithmic_bytes_per_launch": int(fam[dom]["bytes"] / fam[dom]["launches"]),
                    "launches_timed": fam[dom]["launches"],
                    "families": {k: {"gbs": round(v["bytes"] / (v["us"] * 1e-6) / 1e9, 1), "launches": v["launches"]} for k, v in fam.items()}}
        cpu = None
        if not args.no_cpu_baseline:
            threads = len(os.sched_getaffinity(0))
            os.environ.setdefault("OMP_NUM_THREADS", str(threads))
            b, t, sample, kind = cpu_sweep_sample(10.0, threads)
            cpu = {"value": round(b / t / 1e9, 3), "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample}
        line = {
            "metric": "fused-reduce HBM GB/s", "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD + (" [diagnostic run: prologue and epilogue left out]" if args.bare else ""),
                       "cases": len(cases), "bytes_per_step": bytes_per_step,
                       "l2": "inputs (268 MB and 1074 MB) are larger than the 126 MB L2; consecutive launches alternate tensors"},
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": round(e2e_ms, 3)},
            "gpu_launches": int(launches),
            "roofline": roofline,
            "cpu_baseline": cpu,
            "frac_of_peak": round(value / world / peak, 4),
        }
        print(json.dumps(line))
        out_dir = ROOT / "gpurun_out"
        if out_dir.exists():
            (out_dir / "bench_cases.json").write_text(json.dumps(per_case, indent=1))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
