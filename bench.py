#!/usr/bin/env python
"""Benchmarks of the hot path: fused reduce kernels, row kernels, int8 MLP, GPT-2 forward.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                  [--workload sweep|mlp|gpt2|rows]

Default workload (`sweep`, the headline): a step = one pass over the reduction
sweep: {sum, max, mean, argmax} x axis {0, 1, -1} x {A [8192,8192],
B [64,4096,1024], B.permute(0,2,1) as a strided view}, each as ONE fused kernel
call with prologue x*1.5+0.25 and epilogue exp (no epilogue for argmax) = 36
calls, fp32, seeded synthetic N(0,1) inputs. Metric: fused-reduce HBM GB/s =
algorithmic bytes (inputs read once + outputs written once) / device time.
The default run also times the other workloads briefly and reports them under
`other_workloads` in the same JSON line.

`mlp`:  int8 quantized MLP 784->1024->1024->10, 65536 rows per GPU (rows/s).
`gpt2`: GPT-2 small forward, 32 x 1024 tokens per GPU, fp16 (tok/s).
`rows`: causal softmax over fp16 [32,12,1024,1024] + LayerNorm over fp32 [16384,768] (GB/s).

Every number is device time from CUDA events on the launching stream, max over
ranks. With N > 1 GPUs every rank runs the workload on its own shard (weak
scaling, no collective in the data path).

`--impl reference` times the reference's CPU backend (its own templates where
they were compiled into oracle/_ref, else the C restatement) on the host
cores, on a bounded sample of the same workload.
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
SWEEP_DESC = ("reduction sweep: sum/max/mean/argmax x axis 0/1/-1 x A[8192,8192], B[64,4096,1024], "
              "B.permute(0,2,1) view; prologue x*1.5+0.25, epilogue exp; one fused kernel per case")
SHAPES = {"A": (8192, 8192), "B": (64, 4096, 1024), "Bp": (64, 1024, 4096)}
# dram__bytes_read.sum + dram__bytes_write.sum per launch, averaged over the launches of one step of
# each kernel family, from the ncu capture summarised in profiles/reduce_sweep_dram_traffic.md
NCU_TRAFFIC_PER_LAUNCH = {"col": 916197568, "row": 672153568}


def sweep_cases():
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


def peaks() -> dict:
    """Roofline denominators: the measured copy bandwidth and bf16 GEMM rate of this pool's B200s when the
    file is there, else the stated fallback. int8 runs on the same tensor pipe at twice the 16-bit rate."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm": float(d["hbm_gbs"]), "f16": float(d["bf16_tflops"]), "f16_sustained": float(d["bf16_tflops_sustained"]),
                "source": "measured"}
    return {"hbm": 6650.0, "f16": 1590.0, "f16_sustained": 1400.0, "source": "fallback"}


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


def host_threads() -> int:
    """All host cores this process may use; torchrun pins OMP_NUM_THREADS to 1 per rank, which the CPU arm (rank 0 only) undoes."""
    n = len(os.sched_getaffinity(0))
    os.environ["OMP_NUM_THREADS"] = str(n)
    try:  # an OpenMP runtime that is already initialised ignores the variable
        import ctypes
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(n)
    except OSError:
        pass
    return n


# ---------------------------------------------------------------------------
# Workloads. Each has: metric, unit, dtype, desc; setup(dev, rank); step(); units_per_step;
# e2e_setup() / e2e_step() with h2d / d2h byte counts; roofline(pk, reps); cpu_sample(budget_s, threads).
class Sweep:
    name, metric, unit, dtype = "sweep", "fused-reduce HBM GB/s", "GB/s", "f32"

    def __init__(self, only="", bare=False):
        self.only = set(filter(None, only.split(",")))
        self.bare = bare
        self.desc = SWEEP_DESC + (" [diagnostic run: prologue and epilogue left out]" if bare else "")

    def setup(self, dev, rank):
        import torch
        from pequegrad_b200 import _lib as L
        from pequegrad_b200 import kernels as K
        # per-rank synthetic tensors (rank-seeded; rank 0 uses the configured seed 2)
        g = torch.Generator(device=dev).manual_seed(2 + rank)
        only, T = self.only, {}
        if not only or "A" in only:
            T["A"] = torch.randn(SHAPES["A"], generator=g, device=dev)
        if not only or only & {"B", "Bp"}:
            T["B"] = torch.randn(SHAPES["B"], generator=g, device=dev)
            T["Bp"] = T["B"].permute(0, 2, 1)
        self.T = T
        self.cases = [c for c in sweep_cases() if not only or c[0] in only]
        opcode = {"sum": L.SUM, "max": L.MAX, "mean": L.MEAN, "argmax": L.ARGMAX}
        self.prepared = []
        for name, op, ax, nbytes in self.cases:
            if self.bare:
                pr = K.PreparedReduce([T[name]], opcode[op], [ax], False)
            else:
                pr = K.PreparedReduce([T[name]], opcode[op], [ax], False, AFFINE, () if op == "argmax" else EXP_EPI)
            self.prepared.append((name, op, ax, nbytes, pr))
        self.bytes_per_step = sum(c[3] for c in self.cases)
        self.units_per_step = self.bytes_per_step / 1e9
        self.stream = torch.cuda.current_stream().cuda_stream
        self.config = {"cases": len(self.cases), "bytes_per_step": self.bytes_per_step,
                       "l2": "inputs (268 MB and 1074 MB) are larger than the 126 MB L2; consecutive launches alternate tensors"}

    def step(self):
        for *_, pr in self.prepared:
            pr(self.stream)

    def e2e_setup(self):
        import torch
        self.host_in = {k: torch.empty(SHAPES[k], dtype=torch.float32).pin_memory() for k in ("A", "B") if k in self.T}
        for k in self.host_in:
            self.host_in[k].copy_(self.T[k])
        self.host_out = [torch.empty(pr.out.shape, dtype=pr.out.dtype).pin_memory() for *_, pr in self.prepared]
        self.h2d = sum(v.numel() * 4 for v in self.host_in.values())
        self.d2h = sum(o.numel() * o.element_size() for o in self.host_out)

    def e2e_step(self):
        for k, v in self.host_in.items():
            self.T[k].copy_(v, non_blocking=True)
        self.step()
        for o, (*_, pr) in zip(self.host_out, self.prepared):
            o.copy_(pr.out, non_blocking=True)

    def roofline(self, pk, reps):
        """Per-case device time (CUDA events around each launch), grouped by kernel family."""
        import torch
        prepared, per_case = self.prepared, []
        for name, op, ax, nbytes, pr in prepared:
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
            for a, b in evs:
                # touch the other big tensor first so nothing of this case's input is left in L2
                other = prepared[0][4] if name != prepared[0][0] else prepared[min(1, len(prepared) - 1)][4]
                other(self.stream)
                a.record()
                pr(self.stream)
                b.record()
            torch.cuda.synchronize()
            t = statistics.median(a.elapsed_time(b) for a, b in evs)
            per_case.append({"case": f"{name}.{op}.ax{ax}", "us": round(t * 1e3, 2), "gbs": round(nbytes / t / 1e6, 1),
                             "kernel": pr.plan.split()[0], "bytes": nbytes})
        self.per_case = per_case
        fam = {}
        for c in per_case:
            f = fam.setdefault(c["kernel"], {"us": 0.0, "bytes": 0, "launches": 0})
            f["us"] += c["us"]
            f["bytes"] += c["bytes"]
            f["launches"] += 1
        dom = max(fam, key=lambda k: fam[k]["us"])
        achieved = fam[dom]["bytes"] / (fam[dom]["us"] * 1e-6) / 1e9
        return {"bound": "hbm", "kernel": f"reduce_{dom}_kernel", "achieved": round(achieved, 1), "peak": pk["hbm"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm"], 4), "peak_source": pk["source"],
                "traffic": NCU_TRAFFIC_PER_LAUNCH.get(dom) if not self.only and not self.bare else None,
                "algorithmic_bytes_per_launch": int(fam[dom]["bytes"] / fam[dom]["launches"]),
                "launches_timed": fam[dom]["launches"],
                "families": {k: {"gbs": round(v["bytes"] / (v["us"] * 1e-6) / 1e9, 1), "launches": v["launches"]} for k, v in fam.items()}}

    def cpu_sample(self, budget_s, threads):
        """The reference CPU backend's eager chain (2 binary kernels, per-axis reduce, exp) on cases of the
        sweep until `budget_s` is spent. Returns (units, seconds, sample description, kind)."""
        import oracle
        from oracle.chain import fused_reduce_oracle
        kind = "reference" if oracle.have_ref() else "port"
        impl = "ref" if kind == "reference" else "port"
        A = np.random.default_rng(2).standard_normal(SHAPES["A"], dtype=np.float32)
        done_bytes, t_total, n = 0, 0.0, 0
        a_cases = [c for c in sweep_cases() if c[0] == "A"]
        while t_total < budget_s:
            for name, op, ax, nbytes in a_cases:
                t0 = time.perf_counter()
                fused_reduce_oracle([A], op, [ax], False, AFFINE, () if op == "argmax" else EXP_EPI, impl=impl)
                t_total += time.perf_counter() - t0
                done_bytes += nbytes
                n += 1
                if t_total >= budget_s:
                    break
        return done_bytes / 1e9, t_total, (f"{n} case runs cycling through the 12 cases on A[8192,8192] (eager chain: mul, add, reduce, exp), "
                                           f"{t_total:.1f} s of CPU work, {threads} OpenMP threads"), kind


def make_workload(args):
    from pequegrad_b200 import workloads as W
    if args.workload == "sweep":
        return Sweep(args.only, args.bare)
    if args.workload == "mlp":
        return W.Mlp(args.rows or W.MLP_ROWS)
    if args.workload == "gpt2":
        return W.Gpt2(args.batch or W.GPT2_BATCH, args.seq or W.GPT2_T)
    return W.Rows()


def run_reference(args, rank: int):
    """The CPU arm: rank 0 alone times bounded samples of the workload on the host cores."""
    if rank != 0:
        return
    threads = host_threads()
    wl = make_workload(args)
    wl.cpu_sample(0.5, threads)
    vals, ms, sample, kind = [], [], "", "port"
    for _ in range(max(1, min(args.steps, 3))):
        u, t, sample, kind = wl.cpu_sample(6.0, threads)
        vals.append(u / t)
        ms.append(t * 1e3)
    v = statistics.median(vals)
    print(json.dumps({
        "impl": "reference", "metric": wl.metric, "value": v, "unit": wl.unit, "n_gpus": args.gpus, "steps": len(vals),
        "warmup": 1, "ms_per_step": statistics.median(ms), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": wl.dtype, "data": "synthetic", "config": {"workload": wl.desc, "sample": sample},
        "cpu_baseline": {"value": v, "unit": wl.unit, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": v, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def timed_steps(fn, n, barrier, nvtx="pgb_other"):
    """Device milliseconds for n calls of fn, CUDA events on the current stream, barrier + synchronize on both sides."""
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    torch.cuda.nvtx.range_push(nvtx)  # lets a profiler pick out the launches of the timed region
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.nvtx.range_pop()
    barrier()
    return e0.elapsed_time(e1)


def quick_other(name, dev, rank, pk, barrier):
    """A short measurement of one of the non-headline workloads for the `other_workloads` report."""
    import torch
    from pequegrad_b200 import workloads as W
    wl = {"mlp": W.Mlp, "gpt2": W.Gpt2, "rows": W.Rows}[name]()
    wl.setup(dev, rank)
    for _ in range(3):
        wl.step()
    n = 5
    ms = timed_steps(wl.step, n, barrier) / n
    rf = wl.roofline(pk, 5)
    out = {"metric": wl.metric, "per_gpu_value": round(wl.units_per_step / (ms * 1e-3), 1), "unit": wl.unit, "ms_per_step": round(ms, 4), "roofline": rf}
    if name == "gpt2":
        out["model_tflops"] = round(wl.flops_per_token * wl.units_per_step / (ms * 1e-3) / 1e12, 1)
    if name == "mlp":
        out["model_tops"] = round(wl.ops_per_row * wl.units_per_step / (ms * 1e-3) / 1e12, 1)
    del wl
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="pgb200", choices=["pgb200", "reference"])
    ap.add_argument("--workload", default="sweep", choices=["sweep", "mlp", "gpt2", "rows"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-others", action="store_true", help="sweep only: skip the short runs of the other workloads")
    ap.add_argument("--only", default="", help="sweep: comma-separated tensor names (A,B,Bp) to restrict the sweep, for profiling")
    ap.add_argument("--bare", action="store_true", help="sweep diagnostic: no prologue / epilogue (not the benchmark workload)")
    ap.add_argument("--rows", type=int, default=0, help="mlp: rows per GPU (default 65536; smaller for profiling)")
    ap.add_argument("--batch", type=int, default=0, help="gpt2: sequences per GPU (default 32; smaller for profiling)")
    ap.add_argument("--seq", type=int, default=0, help="gpt2: tokens per sequence (default 1024)")
    ap.add_argument("--cases-out", default="", help="sweep: write the per-case timings to this JSON file")
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

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    pk = peaks()
    wl = make_workload(args)
    wl.setup(dev, rank)
    for _ in range(args.warmup):
        wl.step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.2)
    launches0 = L.lib().pgb_launch_count()
    ms_total = timed_steps(wl.step, args.steps, barrier, nvtx="pgb_timed")
    launches = L.lib().pgb_launch_count() - launches0
    roofline = wl.roofline(pk, max(5, min(args.steps, 20)))  # per-kernel device times, still under the clock sampler
    clocks = sampler.stop()

    # end to end through the public call: pinned host inputs -> device, the step, results -> host
    wl.e2e_setup()
    wl.e2e_step()
    n_e2e = max(2, min(args.steps, 5))
    e2e_ms = timed_steps(wl.e2e_step, n_e2e, barrier) / n_e2e
    err = K.device_error()
    if err:
        raise SystemExit(f"a GEMM kernel reported device error {err} (a bounded wait ran out)")

    ms = torch.tensor([ms_total, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms = float(ms[0]), float(ms[1])
    ms_per_step = ms_total / args.steps
    value = world * wl.units_per_step / (ms_per_step * 1e-3)
    e2e_value = world * wl.units_per_step / (e2e_ms * 1e-3)

    others = None
    if args.workload == "sweep" and not args.no_others and not args.only and not args.bare:
        del wl.T, wl.prepared
        torch.cuda.empty_cache()
        others = {n: quick_other(n, dev, rank, pk, barrier) for n in ("rows", "mlp", "gpt2")}

    if rank == 0:
        cpu = None
        if not args.no_cpu_baseline:
            threads = host_threads()
            u, t, sample, kind = wl.cpu_sample(10.0, threads)
            cpu = {"value": round(u / t, 3), "unit": wl.unit, "cores": threads, "kind": kind, "sample": sample}
        line = {
            "metric": wl.metric, "value": round(value, 1), "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": dict({"workload": wl.desc}, **wl.config),
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 2), "unit": wl.unit, "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                    "ms_per_step": round(e2e_ms, 3)},
            "gpu_launches": int(launches),
            "roofline": roofline,
            "cpu_baseline": cpu,
        }
        if args.workload == "sweep":
            line["frac_of_peak"] = round(value / world / pk["hbm"], 4)
        if args.workload == "gpt2":
            line["model_tflops_per_gpu"] = round(wl.flops_per_token * wl.units_per_step / (ms_per_step * 1e-3) / 1e12, 1)
        if args.workload == "mlp":
            line["model_tops_per_gpu"] = round(wl.ops_per_row * wl.units_per_step / (ms_per_step * 1e-3) / 1e12, 1)
        if others is not None:
            line["other_workloads"] = others
        print(json.dumps(line))
        if args.cases_out and args.workload == "sweep":
            Path(args.cases_out).write_text(json.dumps(wl.per_case, indent=1))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
