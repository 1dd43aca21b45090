#!/usr/bin/env python
"""Benchmarks of the hot path: fused reduce kernels, row kernels, int8 MLP, GPT-2 forward, README case.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                  [--workload sweep|mlp|gpt2|rows|readme]

Default workload (`sweep`, the headline): a step = one pass over the reduction
sweep: {sum, max, mean, argmax} x axis {0, 1, -1} x {A [8192,8192],
B [64,4096,1024], B.permute(0,2,1) as a strided view}, each as ONE fused kernel
call with prologue x*1.5+0.25 and epilogue exp (no epilogue for argmax) = 36
calls, fp32, seeded synthetic N(0,1) inputs. Metric: fused-reduce HBM GB/s =
algorithmic bytes (inputs read once + outputs written once) / device time.
The default run also times the other workloads briefly and reports them under
`other_workloads` in the same JSON line.

`mlp`:    int8 quantized MLP 784->1024->1024->10, batch 65536 (rows/s).
`gpt2`:   GPT-2 small forward, batch 32 x 1024 tokens, fp16 (tok/s).
`rows`:   causal softmax over fp16 [32,12,1024,1024] + LayerNorm over fp32 [16384,768] (GB/s).
`readme`: the README fusion case, one fused kernel over 16.4 MB (microseconds per call, warm and cold L2).

Every number is device time from CUDA events on the launching stream, max over
ranks. With N > 1 GPUs the SAME fixed problem is partitioned over the ranks
(strong scaling): each rank takes its slice of the same seeded global arrays
through `pequegrad_b200.distrib.shard_tensor`, runs the kernels on it with no
exchange, and the step ends with the final gather (NCCL all-gather), inside
the timed region. `value` includes the gather; `compute_only` is the same
measurement without it.

`--impl reference` times the reference's CPU backend (its own templates where
they were compiled into oracle/_ref, else the C restatement) on the host
cores, on a bounded sample of the same workload. Where the reference's own CUDA
kernels were compiled (oracle/_ref_cuda), the line also carries `reference_cuda`:
their time on this GPU for the same case.
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

def sweep_cases():
    from pequegrad_b200.workloads import sweep_cases as sc
    return sc()


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


def library_record() -> dict:
    """Which native library this process loaded: path inside the repository, size, modification time and a short
    hash, so that a reader of the line can tell a freshly built library from a stale one."""
    import hashlib
    from pequegrad_b200 import _lib as L
    p = L.LIB_PATH
    h = hashlib.sha256(p.read_bytes()).hexdigest()[:16]
    st = p.stat()
    return {"path": str(p.relative_to(ROOT)), "sha16": h, "bytes": st.st_size, "mtime": int(st.st_mtime),
            "version": L.lib().pgb_version().decode()}


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
# CPU arms: the reference's CPU backend (or the C / torch-CPU restatement where the reference has no CPU kernel
# for the workload) on bounded samples. The only place besides tests/ and smoke() that executes oracle/.
# Each returns (units done, seconds, sample description, kind).
def cpu_sample_sweep(budget_s, threads):
    """The reference CPU backend's eager chain (2 binary kernels, per-axis reduce, exp) on cases of the sweep."""
    import oracle
    from oracle.chain import fused_reduce_oracle
    from pequegrad_b200.workloads import AFFINE, EXP_EPI, SHAPES
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


def cpu_sample_mlp(budget_s, threads):
    """The int8 pipeline of the CPU restatement on blocks of 2048 rows."""
    import oracle
    from pequegrad_b200.workloads import MLP_DIMS, mlp_weights
    Ws, bs = mlp_weights()
    prep = [oracle.quantize_weight_per_channel(W) for W in Ws]
    rng = np.random.default_rng(2)
    rows, t_total = 0, 0.0
    while t_total < budget_s:
        h = rng.random((2048, MLP_DIMS[0]), dtype=np.float32)
        t0 = time.perf_counter()
        for i in range(3):
            sx = oracle.quant_scale(oracle.absmax(h))
            h = oracle.dequant_bias_act(oracle.gemm_i8(oracle.quantize_i8(h, sx), prep[i][0]), prep[i][1], sx, bs[i], relu=i < 2)
        t_total += time.perf_counter() - t0
        rows += 2048
    return rows, t_total, f"{rows} rows in blocks of 2048 through the 3-layer int8 pipeline, {t_total:.1f} s of CPU work, {threads} threads", "port"


def cpu_sample_gpt2(budget_s, threads):
    """The fp32 CPU restatement of the model on sequences of 256 tokens."""
    import torch
    from pequegrad_b200 import gpt2 as G
    torch.set_num_threads(threads)
    cfg = G.GPT2Config()
    weights = _CACHE.setdefault("gpt2_w", G.init_weights(cfg, seed=5))
    rounded = _CACHE.setdefault("gpt2_r", G.round_weights_fp16(weights))
    rng = np.random.default_rng(2)
    toks, t_total = 0, 0.0
    while t_total < budget_s:
        idx = rng.integers(0, cfg.vocab_size, (1, 256)).astype(np.int32)
        t0 = time.perf_counter()
        G.reference_forward(cfg, weights, idx, rounded)
        t_total += time.perf_counter() - t0
        toks += 256
    return toks, t_total, f"{toks} tokens as sequences of 256 through the fp32 CPU restatement of the model, {t_total:.1f} s, {threads} threads", "port"


def cpu_sample_rows(budget_s, threads):
    """The CPU restatement of both row kernels on slices of the same tensors."""
    import oracle
    rng = np.random.default_rng(2)
    S = rng.standard_normal((2, 1024, 1024)).astype(np.float16)
    X = rng.standard_normal((4096, 768)).astype(np.float32)
    gm, bt = np.ones(768, np.float32), np.zeros(768, np.float32)
    done, t_total = 0.0, 0.0
    while t_total < budget_s:
        t0 = time.perf_counter()
        oracle.softmax_rows(S, causal=True)
        oracle.layernorm_rows(X, gm, bt, 1e-5)
        t_total += time.perf_counter() - t0
        done += (S.size * 4 + X.size * 8) / 1e9
    return done, t_total, f"softmax over [2,1024,1024] fp16 + LayerNorm over [4096,768] fp32, repeated for {t_total:.1f} s, {threads} threads", "port"


def cpu_sample_readme(budget_s, threads):
    """The README case on the reference's CPU backend, eager (what BASELINE's first config names): permute is a view,
    two binary kernels, the axis reduce, one more binary kernel. Units = calls."""
    import oracle
    from oracle.chain import fused_reduce_oracle
    from pequegrad_b200.workloads import README_EPI, README_PRO
    kind = "reference" if oracle.have_ref() else "port"
    rng = np.random.default_rng(1)
    x = rng.random((1000, 20, 100), dtype=np.float32).transpose(0, 2, 1)
    y = rng.random((1000, 100, 20), dtype=np.float32)
    calls, t_total = 0, 0.0
    while t_total < budget_s:
        t0 = time.perf_counter()
        fused_reduce_oracle([x, y], "sum", [2], False, README_PRO, README_EPI, impl="ref" if kind == "reference" else "port")
        t_total += time.perf_counter() - t0
        calls += 1
    return calls, t_total, f"{calls} calls of the eager chain on the full-size case, {t_total:.1f} s, {threads} OpenMP threads", kind


_CACHE: dict = {}
USE_GRAPHS = True
CPU_SAMPLES = {"sweep": cpu_sample_sweep, "mlp": cpu_sample_mlp, "gpt2": cpu_sample_gpt2, "rows": cpu_sample_rows, "readme": cpu_sample_readme}


def cpu_value(name, units, seconds):
    """The workload's metric from a CPU sample (the README case reports microseconds per call, the others a rate)."""
    return seconds / units * 1e6 if name == "readme" else units / seconds


def reference_cuda_leg(wl, reps=10):
    """Times of the reference's own CUDA kernels on this GPU for the same case (the comparator named in the baseline
    notes): the eager chain mul -> add -> reduce -> exp on A for the sweep, the generated kernel for the README
    case. None where that library was not built (it needs the reference checkout at build time)."""
    from oracle import ref_cuda
    if not ref_cuda.available() or wl.world != 1:
        return None
    import torch
    from pequegrad_b200.workloads import _event_us, _L2Flush
    dev = wl.dev
    if wl.name == "readme":
        x, y = wl.pairs[0]
        out = torch.empty((1000, 100), dtype=torch.float32, device=dev)
        from pequegrad_b200.workloads import _graph_us
        ring = [lambda p=p: ref_cuda.readme_kernel(p[0], p[1], out) for p in wl.pairs]
        warm_us = _graph_us([ring[0]])  # timed like this library's kernel: 48 launches replayed as one graph
        cold_us = _graph_us(ring)
        ok = bool(torch.allclose(ref_cuda.readme_kernel(x, y), wl.calls[0](), rtol=1e-5, atol=1e-4))
        return {"kernel": "the generated reduce_kernel printed in the reference's README, recompiled for sm_100a, its launch geometry",
                "warm_us": round(warm_us, 2), "cold_us": round(cold_us, 2), "matches_pgb": ok, "published_us_on_the_authors_gpu": 272.85}
    if wl.name != "sweep" or "A0" not in wl.S:
        return None
    A = wl.S["A0"]
    flush = _L2Flush(dev)
    res = {}
    total_ref = total_pgb = 0.0
    by_case = {(n, o, a): pr for n, o, a, _, pr in wl.prepared}
    for ax in (0, 1):
        for op in ("sum", "max", "mean"):
            chain = ref_cuda.EagerReduceChain(A, op, [ax])
            chain()
            us = _event_us(chain, reps, flush)
            pgb = by_case[("A", op, ax)]
            pus = _event_us(lambda: pgb(wl.stream), reps, flush)
            got, want = pgb(wl.stream), chain()
            both_inf = torch.isinf(got) & torch.isinf(want)
            ok = bool(torch.allclose(torch.where(both_inf, 0, got), torch.where(both_inf, 0, want), rtol=1e-4 if op != "max" else 0, atol=0))
            res[f"A.{op}.ax{ax}"] = {"reference_cuda_us": round(us, 1), "pgb_us": round(pus, 1), "speedup": round(us / pus, 1), "matches_pgb": ok}
            total_ref += us
            total_pgb += pus
            del chain
    del flush
    return {"kernels": "the reference's eager chain on A[8192,8192]: mult_kernel, add_kernel, sum/max/mean_kernel, exp_kernel_dense "
                       "(csrc/cuda), its launch geometry, metadata uploaded once", "cases": res,
            "total_reference_cuda_us": round(total_ref, 1), "total_pgb_us": round(total_pgb, 1), "speedup": round(total_ref / total_pgb, 1)}


def make_workload(args):
    from pequegrad_b200 import workloads as W
    if args.workload == "sweep":
        wl = W.Sweep(args.only, args.bare)
        wl.lanes = max(1, args.lanes)
        wl.peer_gather = not args.no_peer_gather
        wl.skip = frozenset(filter(None, args.sweep_skip.split(",")))
        return wl
    if args.workload == "mlp":
        return W.Mlp(args.rows or W.MLP_ROWS)
    if args.workload == "gpt2":
        return W.Gpt2(args.batch or W.GPT2_BATCH, args.seq or W.GPT2_T)
    if args.workload == "readme":
        return W.Readme()
    return W.Rows()


def run_reference(args, rank: int):
    """The CPU arm: rank 0 alone times bounded samples of the workload on the host cores."""
    if rank != 0:
        return
    threads = host_threads()
    wl = make_workload(args)
    sample_fn = CPU_SAMPLES[wl.name]
    sample_fn(0.5, threads)
    vals, ms, sample, kind = [], [], "", "port"
    for _ in range(max(1, min(args.steps, 3))):
        u, t, sample, kind = sample_fn(6.0, threads)
        vals.append(cpu_value(wl.name, u, t))
        ms.append(t * 1e3)
    v = statistics.median(vals)
    print(json.dumps({
        "impl": "reference", "metric": wl.metric, "value": v, "unit": wl.unit, "n_gpus": args.gpus, "steps": len(vals),
        "warmup": 1, "ms_per_step": statistics.median(ms), "higher_is_better": wl.name != "readme", "scaling": "strong", "vs_baseline": None,
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


def max_over_ranks(vals, dev, world):
    import torch
    import torch.distributed as dist
    t = torch.tensor(vals, device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t]


def quick_other(name, dev, rank, world, pk, barrier):
    """A short measurement of one of the non-headline workloads for the `other_workloads` report: the same fixed
    problem split over the ranks, device time as the max over ranks, with and without the final gather."""
    import torch
    from pequegrad_b200 import workloads as W
    wl = {"mlp": W.Mlp, "gpt2": W.Gpt2, "rows": W.Rows, "readme": W.Readme}[name]()
    wl.setup(dev, rank, world)
    for _ in range(3):
        wl.step()
    graphs = bool(USE_GRAPHS and hasattr(wl, "enable_graphs") and wl.enable_graphs())
    n = 40 if name == "readme" else 5  # a README step is 16 calls of a few microseconds: more of them per timed region
    ms = timed_steps(wl.step, n, barrier) / n
    ms_c = timed_steps(wl.step_compute, n, barrier) / n
    ms, ms_c = max_over_ranks([ms, ms_c], dev, world)
    rf = wl.roofline(pk, 5) if rank == 0 else None
    barrier()
    if name == "readme":
        out = {"metric": wl.metric, "value": round(ms * 1e3 / wl.units_per_step, 2), "unit": wl.unit, "ms_per_step": round(ms, 5),
               "calls_per_step": int(wl.units_per_step), "cuda_graphs": graphs, "roofline": rf}
    else:
        out = {"metric": wl.metric, "value": round(wl.units_per_step / (ms * 1e-3), 1), "unit": wl.unit, "ms_per_step": round(ms, 4),
               "compute_only": {"value": round(wl.units_per_step / (ms_c * 1e-3), 1), "ms_per_step": round(ms_c, 4)},
               "n_gpus": world, "scaling": "strong", "timing": "max over ranks", "cuda_graphs": graphs, "roofline": rf}
    if name == "gpt2":
        out["model_tflops_per_gpu"] = round(wl.flops_per_token * wl.units_per_step / world / (ms * 1e-3) / 1e12, 1)
    if name == "mlp":
        out["model_tops_per_gpu"] = round(wl.ops_per_row * wl.units_per_step / world / (ms * 1e-3) / 1e12, 1)
    del wl
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="pgb200", choices=["pgb200", "reference"])
    ap.add_argument("--workload", default="sweep", choices=["sweep", "mlp", "gpt2", "rows", "readme"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel of a step separately instead of replaying CUDA graphs")
    ap.add_argument("--no-others", action="store_true", help="sweep only: skip the short runs of the other workloads")
    ap.add_argument("--only", default="", help="sweep: comma-separated tensor names (A,B,Bp) to restrict the sweep, for profiling")
    ap.add_argument("--lanes", type=int, default=2, help="sweep: streams the independent cases of a step alternate over (1 = one after another)")
    ap.add_argument("--no-peer-gather", action="store_true", help="sweep on several GPUs: gather the small results with NCCL too, not with the peer-memory kernel")
    ap.add_argument("--sweep-skip", default="", help="sweep diagnostic on several GPUs: leave out parts of the step (b0, b1 = the gathers, copies) to see what they cost; not the benchmark workload")
    ap.add_argument("--bare", action="store_true", help="sweep diagnostic: no prologue / epilogue (not the benchmark workload)")
    ap.add_argument("--rows", type=int, default=0, help="mlp: rows in total (default 65536; smaller for profiling)")
    ap.add_argument("--batch", type=int, default=0, help="gpt2: sequences in total (default 32; smaller for profiling)")
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
    from pequegrad_b200 import distrib as D
    from pequegrad_b200 import kernels as K

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        D.init("nccl")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    pk = peaks()
    wl = make_workload(args)
    wl.setup(dev, rank, world)
    for _ in range(args.warmup):
        wl.step()
    barrier()
    launches0 = L.lib().pgb_launch_count()
    wl.step()  # one more untimed step, kernel by kernel, to count this library's launches per step
    launches = (L.lib().pgb_launch_count() - launches0) * args.steps
    global USE_GRAPHS
    USE_GRAPHS = not args.no_graph
    # the launches of a step as CUDA graphs (what the reference's jit(use_cuda_graph=True) asks for): the same kernels,
    # one launch per graph; matters where a rank's shard makes the kernels as short as their launch overhead
    graphs = bool(USE_GRAPHS and hasattr(wl, "enable_graphs") and wl.enable_graphs())
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.2)
    ms_total = timed_steps(wl.step, args.steps, barrier, nvtx="pgb_timed")
    ms_compute = timed_steps(wl.step_compute, args.steps, barrier)
    barrier()
    clocks = sampler.stop()
    # per-kernel device times, under a clock record of their own (the peak measurements inside run for seconds at the
    # power cap and would otherwise decide the median of the timed steps' record)
    roofline = None
    if rank == 0:
        sampler = ClockSampler(local_rank)
        sampler.start()
        roofline = wl.roofline(pk, max(5, min(args.steps, 20)))
        roofline["clocks"] = sampler.stop()
    barrier()

    # end to end through the public call: pinned host inputs -> device, the step, results -> host
    wl.e2e_setup()
    wl.e2e_step()
    n_e2e = max(2, min(args.steps, 5))
    e2e_ms = timed_steps(wl.e2e_step, n_e2e, barrier) / n_e2e
    err = K.device_error()
    if err:
        raise SystemExit(f"a GEMM kernel reported device error {err} (a bounded wait ran out)")

    ms_total, ms_compute, e2e_ms, h2d = max_over_ranks([ms_total, ms_compute, e2e_ms, float(wl.h2d)], dev, world)
    ms_per_step = ms_total / args.steps
    ms_compute /= args.steps
    latency = wl.name == "readme"  # a time per call, not a rate
    value = ms_per_step * 1e3 / wl.units_per_step if latency else wl.units_per_step / (ms_per_step * 1e-3)
    e2e_value = e2e_ms * 1e3 if latency else wl.units_per_step / (e2e_ms * 1e-3)  # (the README case's e2e step is one call)

    ref_cuda = None
    if rank == 0 and world == 1 and wl.name in ("sweep", "readme") and not args.only and not args.bare:
        ref_cuda = reference_cuda_leg(wl)

    others = None
    if args.workload == "sweep" and not args.no_others and not args.only and not args.bare:
        per_case = getattr(wl, "per_case", None)
        del wl.S, wl.prepared, wl.buckets, wl.copies, wl.slots
        torch.cuda.empty_cache()
        others = {n: quick_other(n, dev, rank, world, pk, barrier) for n in ("rows", "gpt2") + (("readme",) if world == 1 else ()) + ("mlp",)}  # mlp last: its int8 peak measurement runs for seconds at the power cap
        wl.per_case = per_case

    if rank == 0:
        cpu = None
        if not args.no_cpu_baseline:
            threads = host_threads()
            u, t, sample, kind = CPU_SAMPLES[wl.name](10.0, threads)
            cpu = {"value": round(cpu_value(wl.name, u, t), 3), "unit": wl.unit, "cores": threads, "kind": kind, "sample": sample}
        line = {
            "metric": wl.metric, "value": round(value, 2 if latency else 1), "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5), "higher_is_better": not latency, "scaling": "strong",
            "vs_baseline": round(value / 272.85, 4) if latency else None, "dtype": wl.dtype, "data": "synthetic",
            "config": dict({"workload": wl.desc, "parallelism": f"dp{world}: one fixed problem split over the GPUs, final all-gather inside the timed region"},
                           **wl.config),
            "clocks": clocks,
            "compute_only": {"value": round(ms_compute * 1e3 / wl.units_per_step if latency else wl.units_per_step / (ms_compute * 1e-3), 2 if latency else 1),
                             "unit": wl.unit, "ms_per_step": round(ms_compute, 5),
                             "what": "the same steps without the final gather" if world > 1 else
                                     "one GPU: there is no gather; a second timing of the same steps, taken right after the first"},
            "e2e": {"value": round(e2e_value, 2), "unit": wl.unit, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": wl.d2h,
                    "ms_per_step": round(e2e_ms, 4),
                    "what": "pinned host inputs copied to every rank's shards, the step with its gather, the result read back by rank 0; "
                            "h2d bytes are the sum over ranks"},
            "gpu_launches": int(launches), "cuda_graphs": graphs,
            "library": library_record(),
            "roofline": roofline,
            "cpu_baseline": cpu,
        }
        if ref_cuda is not None:
            line["reference_cuda"] = ref_cuda
        if args.workload == "sweep":
            line["frac_of_peak_per_gpu"] = round(value / world / pk["hbm"], 4)
        if args.workload == "gpt2":
            line["model_tflops_per_gpu"] = round(wl.flops_per_token * wl.units_per_step / world / (ms_per_step * 1e-3) / 1e12, 1)
        if args.workload == "mlp":
            line["model_tops_per_gpu"] = round(wl.ops_per_row * wl.units_per_step / world / (ms_per_step * 1e-3) / 1e12, 1)
        if others is not None:
            line["other_workloads"] = others
        print(json.dumps(line))
        if args.cases_out and args.workload == "sweep":
            Path(args.cases_out).write_text(json.dumps(wl.per_case, indent=1))
    if world > 1:
        barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
