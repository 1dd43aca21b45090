"""The benchmark workloads on the GPU, in the shape `bench.py` drives:

    setup(dev, rank, world); step(); step_compute(); units_per_step; e2e_setup(); e2e_step() with
    h2d / d2h byte counts; roofline(pk, reps) -> dict for the dominant kernel.

Every workload is ONE fixed problem (the configured global size) partitioned over the `world` GPUs
through `distrib.shard_tensor`: each rank slices the same seeded global arrays, runs the kernels on
its shard with no exchange, and `step()` ends with the final gather (NCCL all-gather), after which
every rank holds the whole result. `step_compute()` is the same work without the gather. All inputs
are seeded synthetic tensors of the configured shapes and distributions. Nothing here touches the
CPU oracle: the CPU arms of the benchmark live in `bench.py`.
"""
from __future__ import annotations

import statistics

import numpy as np

MLP_DIMS = [784, 1024, 1024, 10]
MLP_ROWS = 65536
GPT2_BATCH, GPT2_T = 32, 1024

AFFINE = [("LOAD", 0), ("IMM", 0, 0, 0, 1.5), ("MUL", 0, 1), ("IMM", 0, 0, 0, 0.25), ("ADD", 2, 3)]
EXP_EPI = [("ACC",), ("EXP", 0)]
REDUCE_OPS = ["sum", "max", "mean", "argmax"]
SWEEP_DESC = ("reduction sweep: sum/max/mean/argmax x axis 0/1/-1 x A[8192,8192], B[64,4096,1024], "
              "B.permute(0,2,1) view; prologue x*1.5+0.25, epilogue exp; one fused kernel per case")
SHAPES = {"A": (8192, 8192), "B": (64, 4096, 1024), "Bp": (64, 1024, 4096)}
# dram__bytes_read.sum + dram__bytes_write.sum per launch, averaged over the launches of one single-GPU step of
# each kernel family; source and capture commit are stated in profiles/reduce_sweep_dram_traffic.md
NCU_TRAFFIC_PER_LAUNCH = {"col": 916197568, "row": 672153568}
NCU_TRAFFIC_SOURCE = "profiles/reduce_sweep_dram_traffic.md (single-GPU ncu capture; not a value of this run)"
README_PRO = [("LOAD", 0), ("IMM", 0, 0, 0, 2.0), ("ADD", 0, 1), ("LOAD", 1), ("ADD", 2, 3)]
README_EPI = [("ACC",), ("IMM", 0, 0, 0, 3.0), ("MUL", 0, 1)]


def sweep_cases():
    """(tensor name, op, axis, algorithmic bytes of the whole case) in an order that alternates tensors;
    the first twelve are the axis-0 cases."""
    per = {}
    for name, shape in SHAPES.items():
        per[name] = []
        for ax in (0, 1, -1):
            for op in REDUCE_OPS:
                n_in = int(np.prod(shape))
                n_out = n_in // shape[ax]
                per[name].append((name, op, ax, 4 * n_in + 4 * n_out))
    out = []
    for i in range(12):
        out += [per["A"][i], per["B"][i], per["Bp"][i]]
    return out


def _event_us(fn, reps, flush=None):
    """Median device time of fn() in microseconds, CUDA events on the current stream."""
    import torch
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    runway = getattr(torch.cuda, "_sleep", None)  # a spin kernel; without it the timings below are upper bounds
    for a, b in evs:
        if flush is not None:
            flush()
        # The device first spins for ~0.2 ms without touching memory, so that the launch below is already queued when
        # the first event is reached: without this runway the interval also holds the host's time to issue the call
        # (tens of microseconds for a ctypes call), which swamps kernels of 10-60 us.
        if runway is not None:
            runway(400_000)
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    return statistics.median(a.elapsed_time(b) for a, b in evs) * 1e3


def _graph_us(fns, launches=48):
    """Mean device time per call, in microseconds, of `launches` calls cycling through `fns`, replayed as ONE CUDA
    graph between one pair of events. For kernels of a few tens of microseconds: a single launch between two events
    is read with the granularity of the event timestamps (about 2 us here: every single-launch figure of a short
    kernel came out as a multiple of 2.05 us), and kernel-by-kernel launches from Python leave the GPU idle between
    calls. A ring of buffer sets larger than the L2 in `fns` makes every call a cold one. Falls back to
    single-launch timing when the capture fails."""
    import torch
    n = len(fns)

    def run():
        for i in range(launches):
            fns[i % n]()
    g = capture_graph(run)
    if g is None:
        return _event_us(fns[0], 20)
    ts = []
    for _ in range(5):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e3 / launches)
    return statistics.median(ts)


def _graph_us_flushed(fn, flush, rounds=6):
    """Device time of fn() in microseconds when every call comes right after `flush()` (kernels that leave nothing of
    fn's operands in L2): `rounds` x (flush, fn) replayed as one graph, minus `rounds` x flush replayed as another,
    divided by `rounds`. The event pair then brackets milliseconds, not one short kernel, so the timestamps'
    granularity (about 2 us) and the event overhead drop out. Falls back to single-launch timing if a capture fails."""
    import torch

    def both():
        for _ in range(rounds):
            flush()
            fn()

    def only_flush():
        for _ in range(rounds):
            flush()
    g1, g0 = capture_graph(both), capture_graph(only_flush)
    if g1 is None or g0 is None:
        return _event_us(fn, 10, flush)

    def t(g):
        ts = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        return statistics.median(ts)
    return max(0.0, (t(g1) - t(g0)) / rounds)


class _L2Flush:
    """201 MB written, then another 201 MB read: the L2 (126 MB) ends up holding clean lines of unrelated data, as it
    would after the kernels that run between two uses of a buffer. Writing alone leaves the L2 full of dirty lines,
    and their write-back would be charged to the timed kernel's first misses."""

    def __init__(self, dev):
        import torch
        self.buf = torch.zeros((2, 100 << 20), dtype=torch.float16, device=dev)

    def __call__(self):
        self.buf[:1].zero_().add_(1)
        self.sink = self.buf[1:2].amax()


def capture_graph(fn):
    """`fn()` (kernels of this library on the current stream, torch allocations allowed) as a CUDA graph: a step
    then costs one launch instead of one per kernel, which is what bounds the small per-GPU shards of a partitioned
    problem (the reference's `jit(use_cuda_graph=True)` is the same idea, pequegrad/transforms/compile.py:85-118).
    Returns the graph, or None when the capture failed (the caller keeps launching kernel by kernel)."""
    import torch
    try:
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        torch.cuda.synchronize()
        return g
    except Exception:  # noqa: BLE001 - any capture problem leaves the eager path in charge
        torch.cuda.synchronize()
        return None


def _devices(world):
    from . import distrib as D
    return D.default_devices(world)


class Sweep:
    """The 36-case reduction sweep. Partition over P GPUs: every case splits a KEPT axis, so no rank needs
    another's data: A by rows for the axis-1 / -1 cases and by column slabs for axis 0; B along its batch
    dim for axis 1 / -1 and along dim 1 for axis 0; the permuted view is the permute of B's shards. The
    outputs of a step go into two buckets, each gathered by one all-gather: the axis-0 cases (large
    outputs) first, so that their transfer runs under the remaining kernels."""
    name, metric, unit, dtype = "sweep", "fused-reduce HBM GB/s", "GB/s", "f32"

    def __init__(self, only="", bare=False):
        self.only = set(filter(None, only.split(",")))
        self.bare = bare
        self.desc = SWEEP_DESC + (" [diagnostic run: prologue and epilogue left out]" if bare else "")

    def setup(self, dev, rank, world):
        import torch
        from . import _lib as L
        from . import distrib as D
        from . import kernels as K
        self.dev, self.rank, self.world = dev, rank, world
        g = torch.Generator(device=dev).manual_seed(2)  # the same global arrays on every rank
        only, devs, S = self.only, _devices(world), {}
        if not only or "A" in only:
            A = torch.randn(SHAPES["A"], generator=g, device=dev)
            S["A0"], S["A1"] = (D.shard_tensor(A, world, d, devs).shards[0] for d in (0, 1))
            del A
        if not only or only & {"B", "Bp"}:
            B = torch.randn(SHAPES["B"], generator=g, device=dev)
            S["B0"], S["B1"] = (D.shard_tensor(B, world, d, devs).shards[0] for d in (0, 1))
            del B
        self.S = S
        torch.cuda.empty_cache()
        self.cases = [c for c in sweep_cases() if not only or c[0] in only]
        opcode = {"sum": L.SUM, "max": L.MAX, "mean": L.MEAN, "argmax": L.ARGMAX}
        # the first bucket (the large axis-0 results) is gathered by NCCL under the remaining kernels; the second (11 MB)
        # comes after the last kernel, where latency is all that counts: one launch of the peer-memory kernel
        self.buckets = [D.GatherBucket(dev, async_op=True), D.GatherBucket(dev, async_op=True, peer_memory=self.peer_gather)]
        plan = []
        for name, op, ax, nbytes in self.cases:
            base = S[("A" if name == "A" else "B") + ("1" if ax == 0 else "0")]
            x = base.permute(0, 2, 1) if name == "Bp" else base
            gdim = 1 if (name == "Bp" and ax == 0) else 0  # the only case whose kept split axis is not the output's dim 0
            oshape = K.reduced_shape(x.shape, [ax], False)
            bk = self.buckets[0 if ax == 0 else 1]
            idx = bk.add(oshape, torch.int32 if op == "argmax" else torch.float32, gdim)
            plan.append((name, op, ax, nbytes, x, bk, idx, gdim))
        self.prepared, self.copies, self.slots = [], [], []
        for name, op, ax, nbytes, x, bk, idx, gdim in plan:
            self.slots.append((bk, idx))
            out = bk.local_view(idx)
            pro, epi = ((), ()) if self.bare else (AFFINE, () if op == "argmax" else EXP_EPI)
            pr = K.PreparedReduce([x], opcode[op], [ax], False, pro, epi, out=out)
            self.prepared.append((name, op, ax, nbytes // world, pr))
            if gdim != 0 and world > 1:
                full = list(out.shape)
                full[gdim] *= world
                self.copies.append((bk, idx, torch.empty(full, dtype=out.dtype, device=dev)))
        self.n_first = sum(1 for c in self.cases if c[2] == 0)
        self.bytes_per_step = sum(c[3] for c in self.cases)
        self.units_per_step = self.bytes_per_step / 1e9
        self.stream = torch.cuda.current_stream().cuda_stream
        self.gather_bytes = sum(b.nbytes for b in self.buckets) * world
        shard_mb = {k: round(v.numel() * 4 / 1e6) for k, v in S.items()}
        self.config = {"cases": len(self.cases), "bytes_per_step": self.bytes_per_step, "partition": "kept axis of every case split over the GPUs",
                       "streams": "the independent cases of a step alternate over %d streams that fork from and join the timed one" % self.lanes,
                       "gathers": "none (one GPU)" if world == 1 else "axis-0 results: NCCL all-gather under the remaining kernels; the rest: " + self.buckets[1].peer_note,
                       "shard_MB_per_gpu": shard_mb, "gathered_bytes_per_step": self.gather_bytes if world > 1 else 0,
                       "e2e_note": "each rank uploads its row shards of A and B once per step; the second sharding (column slabs of A, dim 1 of B) "
                                   "is made on the devices by one all-to-all each" if world > 1 else
                                   "one GPU: A and B uploaded once per step on a copy stream; A's cases run while B is still on its way, the "
                                   "axis-0 results of B travel back under the remaining kernels; all joined into the timed stream",
                       "l2": ("each rank's shards (%s MB) against a 126 MB L2; consecutive launches alternate tensors, so a case never "
                              "finds its own input in L2 unless the shard is smaller than what ran in between" % "/".join(map(str, shard_mb.values())))}

    graphs = None

    lanes = 2
    peer_gather = True
    skip = frozenset()
    copy_graph = None

    def _launch(self, lo, hi):
        """The cases lo..hi, which do not depend on one another, alternating over `lanes` streams that fork from and
        join the current one: the ramp and the last partial wave of one kernel run under its neighbour's full waves
        (on a shard of an eighth of A a kernel is all ramp and tail)."""
        self._on_lanes([pr for *_, pr in self.prepared[lo:hi]])

    def _on_lanes(self, calls):
        """Independent launches alternating over the lanes (see _launch)."""
        import torch
        if self.lanes <= 1 or len(calls) < 2:
            for fn in calls:
                fn()
            return
        main = torch.cuda.current_stream()
        if getattr(self, "_side", None) is None:
            self._side = [torch.cuda.Stream(device=self.dev) for _ in range(self.lanes - 1)]
        fork = torch.cuda.Event()
        fork.record(main)
        for st in self._side:
            st.wait_event(fork)
        for i, fn in enumerate(calls):
            lane = i % self.lanes
            if lane == 0:
                fn()
            else:
                with torch.cuda.stream(self._side[lane - 1]):
                    fn()
        for st in self._side:
            join = torch.cuda.Event()
            join.record(st)
            main.wait_event(join)

    def enable_graphs(self):
        """The launches of a step as two CUDA graphs (the axis-0 cases, then the rest), with the gathers between them."""
        n = len(self.prepared)
        g = [capture_graph(lambda: self._launch(0, self.n_first)), capture_graph(lambda: self._launch(self.n_first, n))]
        self.graphs = g if all(x is not None for x in g) else None
        if self.graphs is not None and self.copies:
            self._copy_pairs()
            self.copy_graph = capture_graph(self._run_copies)  # None (not captured) leaves the separate launches
        return self.graphs is not None

    def _copy_pairs(self):
        """(source view, destination view) of the permuting copies, built once: the slabs that are not row blocks of
        their result (the permuted view's axis-0 results, gathered along dim 1). int32 results travel as float32
        bit patterns, so that every copy takes the vectorised elementwise kernel."""
        import torch
        if getattr(self, "_pairs", None) is None:
            pairs = []

            def keep(d, s_):
                if d.dtype == torch.int32:
                    d, s_ = d.view(torch.float32), s_.view(torch.float32)
                pairs.append((s_, d))
            for bk, idx, dst in self.copies:
                bk.full(idx, copy_out=dst, copy_fn=keep)
            self._pairs = pairs
        return self._pairs

    def _run_copies(self):
        from . import kernels as K
        if getattr(self, "copy_graph", None) is not None:
            self.copy_graph.replay()
            return
        self._on_lanes([lambda s_=s_, d=d: K.fused_elementwise([s_], [("LOAD", 0)], outs=[d]) for s_, d in self._copy_pairs()])

    def _part(self, i):
        if self.graphs is not None:
            self.graphs[i].replay()
        elif i == 0:
            self._launch(0, self.n_first)
        else:
            self._launch(self.n_first, len(self.prepared))

    def step_compute(self):
        self._part(0)
        self._part(1)

    def step(self):
        if self.world == 1:
            return self.step_compute()
        b0, b1 = self.buckets
        skip = self.skip  # diagnostic only (bench.py --sweep-skip): parts of the step left out to see what they cost
        import torch
        main = torch.cuda.current_stream()
        self._part(0)
        if "b0" not in skip:
            b0.gather()
        copied = None
        if self.copies and "copies" not in skip:
            # the permuting copies (all of them slabs of the first bucket) wait for that bucket's gather on a stream of
            # their own and run under the remaining kernels; the timed stream joins them at the end
            if getattr(self, "_copy_stream", None) is None:
                self._copy_stream = torch.cuda.Stream(device=self.dev)
            start = torch.cuda.Event()
            start.record(main)  # whoever read the copies' destinations in the step before is done
            self._copy_stream.wait_event(start)
            with torch.cuda.stream(self._copy_stream):
                b0.wait()
                self._run_copies()
                copied = torch.cuda.Event()
                copied.record(self._copy_stream)
        self._part(1)
        if "b1" not in skip:
            b1.gather()
        b0.wait()
        b1.wait()
        if copied is not None:
            main.wait_event(copied)

    def results(self):
        """Every case's whole result on this rank after step(): [(case name, tensor)]."""
        res, copies = [], {(id(bk), idx): dst for bk, idx, dst in self.copies}
        for (name, op, ax, _), (bk, idx) in zip(self.cases, self.slots):
            full = copies.get((id(bk), idx))
            if full is None:
                full = bk.full(idx)
                if self.world > 1:  # [world, rows / world, ...] view of the receive buffer
                    full = full.reshape((-1,) + tuple(full.shape[2:]))
            res.append((f"{name}.{op}.ax{ax}", full))
        return res

    def e2e_setup(self):
        import torch
        # Host buffers hold this rank's ROW shards only (dim 0 of A and of B). The second sharding of each tensor
        # (column slabs of A, dim 1 of B, which the axis-0 cases need) is made on the devices from the row shards by
        # one all-to-all each: the bytes cross NVLink once instead of PCIe a second time.
        self.host_in = {k: torch.empty(v.shape, dtype=torch.float32).pin_memory() for k, v in self.S.items() if k.endswith("0")}
        for k, h in self.host_in.items():
            h.copy_(self.S[k])
        self.staging = {k: torch.empty_like(v) for k, v in self.S.items() if k.endswith("0")} if self.world > 1 else {}
        self.reshard_ok = True
        self.host_out = [torch.empty(b.recv.numel(), dtype=torch.uint8).pin_memory() for b in self.buckets] if self.rank == 0 else []
        self.host_out += [torch.empty(dst.shape, dtype=dst.dtype).pin_memory() for _, _, dst in self.copies] if self.rank == 0 else []
        self.h2d = sum(v.numel() * 4 for v in self.host_in.values()) * self.world
        self.d2h = sum(o.numel() * o.element_size() for o in self.host_out)

    def _e2e_step_one_gpu(self):
        """One GPU: the copies run on streams of their own around the timed one. A is uploaded first and its twelve
        cases run while B is still on its way; B's axis-0 cases (134 of the 145 MB of results) run first and their
        results travel to the host under the remaining kernels. Everything is joined into the timed stream at the
        end, so its events bracket the copies too."""
        import torch
        main = torch.cuda.current_stream()
        if getattr(self, "_cp", None) is None:
            self._cp, self._dh = torch.cuda.Stream(device=self.dev), torch.cuda.Stream(device=self.dev)
            names = [c[0] for c in self.cases]
            ax = [c[2] for c in self.cases]
            self._order = ([i for i, n in enumerate(names) if n == "A"],
                           [i for i, n in enumerate(names) if n != "A" and ax[i] == 0],
                           [i for i, n in enumerate(names) if n != "A" and ax[i] != 0])
        start = torch.cuda.Event()
        start.record(main)
        self._cp.wait_event(start)  # the kernels of the step before have read the shards that the uploads overwrite
        self._dh.wait_event(start)
        ups = {}
        with torch.cuda.stream(self._cp):
            for k in sorted(self.host_in):  # "A0" before "B0"
                self.S[k].copy_(self.host_in[k], non_blocking=True)
                ups[k[0]] = torch.cuda.Event()
                ups[k[0]].record(self._cp)
        a_cases, b_first, b_rest = self._order
        if "A" in ups:
            main.wait_event(ups["A"])
        for i in a_cases:
            self.prepared[i][-1]()
        if "B" in ups:
            main.wait_event(ups["B"])
        for i in b_first:
            self.prepared[i][-1]()
        r0 = torch.cuda.Event()
        r0.record(main)
        with torch.cuda.stream(self._dh):
            self._dh.wait_event(r0)
            self.host_out[0].copy_(self.buckets[0].recv, non_blocking=True)
        for i in b_rest:
            self.prepared[i][-1]()
        r1 = torch.cuda.Event()
        r1.record(main)
        with torch.cuda.stream(self._dh):
            self._dh.wait_event(r1)
            self.host_out[1].copy_(self.buckets[1].recv, non_blocking=True)
            done = torch.cuda.Event()
            done.record(self._dh)
        main.wait_event(done)

    def e2e_step(self):
        from . import distrib as D
        from . import kernels as K
        if self.world == 1 and not self.only:
            return self._e2e_step_one_gpu()
        for k, h in self.host_in.items():
            self.S[k].copy_(h, non_blocking=True)
        if self.world > 1 and self.reshard_ok:
            try:
                for name, shape in (("A", SHAPES["A"]), ("B", SHAPES["B"])):
                    if name + "0" in self.S:
                        st = D.ShardedTensor([self.S[name + "0"]], [0], self.world, shape)
                        D.reshard_tensor(st, 1, staging=self.staging[name + "0"], out=self.S[name + "1"],
                                         copy_fn=lambda d, s_: K.fused_elementwise([s_], [("LOAD", 0)], outs=[d]))
            except (RuntimeError, ValueError) as e:  # the same refusal on every rank: upload the second sharding too
                import torch
                self.reshard_ok = False
                self.config["e2e_note"] = f"re-sharding on the devices refused ({e}); both shardings are uploaded from the host"
                self.host_in1 = {k: torch.empty(v.shape, dtype=torch.float32).pin_memory() for k, v in self.S.items() if k.endswith("1")}
                for k, h in self.host_in1.items():
                    h.copy_(self.S[k])
                self.h2d += sum(v.numel() * 4 for v in self.host_in1.values()) * self.world
        if self.world > 1 and not self.reshard_ok:
            for k, h in self.host_in1.items():
                self.S[k].copy_(h, non_blocking=True)
        self.step()
        if self.rank == 0:  # the caller's process reads the gathered results
            srcs = [b.recv for b in self.buckets] + [dst for _, _, dst in self.copies]
            for o, s in zip(self.host_out, srcs):
                o.copy_(s, non_blocking=True)

    def _flushers(self, pr):
        """Cases over other buffers, largest first, that together stream more than the 126 MB L2."""
        own, seen, picked, total = pr.inputs[0].data_ptr(), set(), [], 0
        for *_, o in sorted(self.prepared, key=lambda p: -p[4].inputs[0].numel()):
            ptr = o.inputs[0].data_ptr()
            if ptr == own or ptr in seen:
                continue
            seen.add(ptr)
            picked.append(o)
            total += o.inputs[0].numel() * 4
            if total > 160e6:
                break
        return picked

    def roofline(self, pk, reps):
        """Per-case device time on this rank's shards (each case right after kernels over other buffers, six rounds
        replayed as one graph, the flushing kernels' own time subtracted), grouped by kernel family."""
        prepared, per_case = self.prepared, []
        for name, op, ax, nbytes, pr in prepared:
            fl = self._flushers(pr)  # cases over other buffers: nothing of this case's input is left in L2

            def flush(fl=fl):
                for o in fl:
                    o()
            us = _graph_us_flushed(pr, flush)
            per_case.append({"case": f"{name}.{op}.ax{ax}", "us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1),
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
        full = not self.only and not self.bare and self.world == 1
        return {"bound": "hbm", "kernel": f"reduce_{dom}_kernel", "achieved": round(achieved, 1), "peak": pk["hbm"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm"], 4), "peak_source": pk["source"],
                "traffic": NCU_TRAFFIC_PER_LAUNCH.get(dom) if full else None, "traffic_source": NCU_TRAFFIC_SOURCE if full else None,
                "algorithmic_bytes_per_launch": int(fam[dom]["bytes"] / fam[dom]["launches"]),
                "launches_timed": fam[dom]["launches"],
                "slowest_case": min(per_case, key=lambda c: c["gbs"]),
                "families": {k: {"gbs": round(v["bytes"] / (v["us"] * 1e-6) / 1e9, 1), "launches": v["launches"]} for k, v in fam.items()}}


def mlp_weights(seed=3):
    rng = np.random.default_rng(seed)
    Ws = [(rng.standard_normal((MLP_DIMS[i], MLP_DIMS[i + 1])) * 0.05).astype(np.float32) for i in range(3)]
    bs = [(rng.standard_normal(MLP_DIMS[i + 1]) * 0.05).astype(np.float32) for i in range(3)]
    return Ws, bs


def measure_int8_peak(dev, seconds=4.0):
    """The int8 tensor rate of this GPU, measured the way the bf16 figures of MEASURED_PEAKS.json are: the
    vendor library's int8 GEMM (torch._int_mm, cuBLASLt) on 8192^3, best of 10 launches (burst) and back to
    back for `seconds` (sustained, under the power cap). TOP/s. A library call used as a yardstick only."""
    import time

    import torch
    n = 8192
    a = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=dev)
    b = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=dev).t()  # [K, N] with K contiguous: the layout cuBLASLt wants
    ops = 2.0 * n ** 3
    for _ in range(3):
        torch._int_mm(a, b)
    best = float("inf")
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch._int_mm(a, b)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    per = max(1, int(seconds * 1e3 / best))
    t0 = time.perf_counter()
    e0.record()
    for _ in range(per):
        torch._int_mm(a, b)
    e1.record()
    torch.cuda.synchronize()
    sustained_ms = e0.elapsed_time(e1) / per
    return {"burst": round(ops / best / 1e9, 1), "sustained": round(ops / sustained_ms / 1e9, 1), "unit": "TOP/s",
            "how": f"torch._int_mm int8 8192^3: best of 10, and {per} launches back to back ({time.perf_counter() - t0:.1f} s)"}


class Mlp:
    """int8 quantized MLP 784 -> 1024 -> 1024 -> 10 over `rows` activation rows in total, split by rows over the
    GPUs. The per-tensor activation scale stays global: one all-reduce(max) of a float per layer."""
    name, metric, unit, dtype = "mlp", "int8-MLP rows/s", "rows/s", "i8"

    def __init__(self, rows=MLP_ROWS, use_peers=True):
        self.rows, self.use_peers = rows, use_peers
        self.desc = (f"quantized MLP inference 784->1024->1024->10 with ReLU, batch {rows} row-sharded over the GPUs; weights N(0,0.05) int8 per "
                     "output channel, activations uniform[0,1) fp32 quantized per tensor on the device (absmax over the whole batch); int32 "
                     "accumulate, fused dequant+bias+ReLU")

    def setup(self, dev, rank, world):
        import torch
        from . import distrib as D
        from .qmlp import QuantizedMLP
        self.dev, self.rank, self.world = dev, rank, world
        Ws, bs = mlp_weights()
        self.mlp = QuantizedMLP(Ws, bs, device=dev)
        g = torch.Generator(device=dev).manual_seed(3)
        X = torch.rand((self.rows, MLP_DIMS[0]), generator=g, device=dev)
        self.X = D.shard_tensor(X, world, 0, _devices(world)).shards[0]
        del X
        self.full = torch.empty((self.rows, MLP_DIMS[-1]), dtype=torch.float32, device=dev) if world > 1 else None
        # the exchanges of a step (three maxima of one float, one gather of [rows / P, 10] slabs) go through the
        # peer-memory kernels when the ranks can map one another's memory, else through NCCL
        self.peers, self.peer_note = None, "NCCL"
        if world > 1 and self.use_peers:
            try:
                self.peers = D.PeerGroup(gather_bytes=self.X.shape[0] * MLP_DIMS[-1] * 4)
                self.peer_note = "peer-memory kernels over NVLink (CUDA IPC mappings)"
            except Exception as e:  # noqa: BLE001 - any failure of the mapping leaves the NCCL path
                self.peer_note = f"NCCL (peer mapping unavailable: {type(e).__name__}: {e})"
            flags = [None] * world
            import torch.distributed as dist
            dist.all_gather_object(flags, self.peers is not None)
            if not all(flags):  # all ranks or none
                if self.peers is not None:
                    self.peers.close()
                self.peers = None
        self.units_per_step = self.rows
        self.ops_per_row = 2 * sum(MLP_DIMS[i] * MLP_DIMS[i + 1] for i in range(3))
        self.config = {"rows_total": self.rows, "rows_per_gpu": self.rows // world, "int8_ops_per_step": self.ops_per_row * self.rows,
                       "collectives_per_step": 0 if world == 1 else "3 x all_reduce(max) of one float + 1 all_gather of [rows,10] fp32, by " + self.peer_note,
                       "l2": "activations per layer (51 to 268 MB over all GPUs) against a 126 MB L2; each layer reads what the one before "
                             "wrote, as the pipeline does in use"}

    graphs = None

    def _compute(self):
        self.out = self.mlp.forward_sharded([self.X], peers=self.peers)[0]

    def _full(self):
        self._compute()
        if self.peers is not None:
            self.out_full = self.peers.allgather(self.out).view(self.rows, MLP_DIMS[-1])

    def enable_graphs(self):
        """Whole steps as CUDA graphs when no library collective is inside (one GPU, or the peer-memory kernels)."""
        if self.world > 1 and self.peers is None:
            return False
        g = [capture_graph(self._compute), capture_graph(self._full)]
        ok = all(x is not None for x in g)
        if self.world > 1:  # all ranks or none: the peer kernels of a step must be launched by everyone
            import torch.distributed as dist
            flags = [None] * self.world
            dist.all_gather_object(flags, ok)
            ok = all(flags)
        self.graphs = g if ok else None
        return ok

    def step_compute(self):
        if self.graphs is not None:
            self.graphs[0].replay()
        else:
            self._compute()

    def step(self):
        import torch.distributed as dist
        if self.graphs is not None and (self.world == 1 or self.peers is not None):
            self.graphs[1].replay()
            if self.world == 1:
                self.out_full = self.out
            return
        self.step_compute()
        if self.world == 1:
            self.out_full = self.out
        elif self.peers is not None:
            self.out_full = self.peers.allgather(self.out).view(self.rows, MLP_DIMS[-1])
        else:
            dist.all_gather_into_tensor(self.full, self.out)
            self.out_full = self.full

    def e2e_setup(self):
        import torch
        self.host_x = torch.empty(self.X.shape, dtype=torch.float32).pin_memory()
        self.host_x.copy_(self.X)
        self.step()
        self.host_out = torch.empty(self.out_full.shape, dtype=torch.float32).pin_memory() if self.rank == 0 else None
        self.h2d = self.host_x.numel() * 4 * self.world
        self.d2h = self.host_out.numel() * 4 if self.rank == 0 else 0

    def e2e_step(self):
        self.X.copy_(self.host_x, non_blocking=True)
        self.step()
        if self.rank == 0:
            self.host_out.copy_(self.out_full, non_blocking=True)

    def roofline(self, pk, reps):
        """The 1024 -> 1024 hidden layer's GEMM as the pipeline runs it on this rank's rows: the absmax-only pass and
        the pass that stores requantised int8 (the slower of the two is the reported kernel), plus the fp32-output
        variant for comparison. The peak is the int8 GEMM rate measured on this GPU in this run."""
        from . import kernels as K
        rows = self.X.shape[0]
        wq, ws, bias = self.mlp.layers[1]
        b = self.mlp._buffers(rows, self.X.device)
        xq, amax = b["q"][1], b["amax"]
        flush = _L2Flush(self.X.device)  # nothing of the operands stays in L2
        t_abs = _graph_us_flushed(lambda: K.qlinear_i8(xq, wq, ws, a_absmax=amax[1:2], bias=bias, relu=True, want_out=False, out_absmax=amax[2:3]), flush)
        t_q = _graph_us_flushed(lambda: K.qlinear_i8(xq, wq, ws, a_absmax=amax[1:2], bias=bias, relu=True, out=b["q"][2], out_absmax=amax[2:3]), flush)
        t_f = _graph_us_flushed(lambda: K.qlinear_i8(xq, wq, ws, a_absmax=amax[1:2], bias=bias, relu=True, out=b["h"][1]), flush)
        t_in = _graph_us_flushed(lambda: K.qlinear_i8(b["q"][0], self.mlp.layers[0][0], self.mlp.layers[0][1], a_absmax=amax[0:1], bias=self.mlp.layers[0][2],
                                                      relu=True, out=b["q"][1], out_absmax=amax[1:2]), flush)
        ops = 2.0 * rows * 1024 * 1024
        i8 = measure_int8_peak(self.X.device)
        peak = i8["burst"]
        us = max(t_abs, t_q)
        ach = ops / (us * 1e-6) / 1e12
        tops = lambda t, o=ops: round(o / (t * 1e-6) / 1e12, 1)  # noqa: E731
        other = {"absmax_f32_us": round(_graph_us_flushed(lambda: K.absmax(self.X, out=amax[0:1]), flush), 1),
                 "quantize_input_us": round(_graph_us_flushed(lambda: K.quantize_i8(self.X, absmax_dev=amax[0:1], out=b["q"][0]), flush), 1),
                 "quantize_hidden_us (materialising route only)": round(_graph_us_flushed(lambda: K.quantize_i8(b["h"][1], absmax_dev=amax[2:3], out=b["q"][2]), flush), 1)}
        del flush
        x_bytes = self.X.numel() * 4
        other["absmax_f32_gbs"] = round(x_bytes / other["absmax_f32_us"] / 1e3, 1)
        other["absmax_f32_frac_of_hbm"] = round(other["absmax_f32_gbs"] / pk["hbm"], 4)
        return {"bound": "tensor", "kernel": "gemm_tc_kernel<i8> %dx1024x1024, %s epilogue" % (rows, "int8-requantising" if t_q >= t_abs else "absmax-only"),
                "achieved": round(ach, 1), "peak": peak, "unit": "TOP/s", "frac": round(ach / peak, 4),
                "peak_source": "int8 GEMM rate measured in this run (burst: the kernel is timed alone): " + i8["how"],
                "int8_peak_measured": i8, "frac_of_2x_bf16_burst": round(ach / (2 * pk["f16"]), 4),
                "traffic": None, "us": round(us, 1), "algorithmic_ops_per_launch": ops,
                "variants": {"absmax_only": {"us": round(t_abs, 1), "tops": tops(t_abs), "frac": round(tops(t_abs) / peak, 4)},
                             "int8_out": {"us": round(t_q, 1), "tops": tops(t_q), "frac": round(tops(t_q) / peak, 4)},
                             "fp32_out (written in full)": {"us": round(t_f, 1), "tops": tops(t_f), "frac": round(tops(t_f) / peak, 4)},
                             "input layer K=784, int8_out": {"us": round(t_in, 1), "tops": tops(t_in, 2.0 * rows * 784 * 1024),
                                                              "frac": round(tops(t_in, 2.0 * rows * 784 * 1024) / peak, 4)}},
                "hidden_layer_both_passes_us": round(t_abs + t_q, 1),
                "other_kernels": other}


class Gpt2:
    """GPT-2 small forward (12 layers, 768, 12 heads, vocab 50257) over `batch` sequences of `T` tokens in total,
    whole sequences split over the GPUs; the final gather brings every rank the logits of the whole batch."""
    name, metric, unit, dtype = "gpt2", "GPT-2 tok/s", "tok/s", "f16"

    def __init__(self, batch=GPT2_BATCH, T=GPT2_T):
        self.B, self.T = batch, T
        self.desc = (f"GPT-2 small forward inference from random init N(0,0.02): 12 layers, d_model 768, 12 heads, d_ff 3072, vocab 50257, "
                     f"batch {batch} x {T} token ids uniform in [0,50257), sequences split over the GPUs; fp16 activations and weights, fp32 accumulate")

    def setup(self, dev, rank, world):
        import torch
        from . import distrib as D
        from . import gpt2 as G
        self.dev, self.rank, self.world = dev, rank, world
        self.cfg = G.GPT2Config()
        self.weights = G.init_weights(self.cfg, seed=5)
        self.model = G.GPT2(self.cfg, self.weights, device=dev)
        g = torch.Generator(device=dev).manual_seed(5)
        idx = torch.randint(0, self.cfg.vocab_size, (self.B, self.T), generator=g, device=dev, dtype=torch.int32)
        self.idx = D.shard_tensor(idx, world, 0, _devices(world)).shards[0]
        self.Bl = self.idx.shape[0]
        self.logits_buf = torch.empty((self.Bl, self.T, self.model.vocab_ld), dtype=torch.float16, device=dev)
        self.full = torch.empty((self.B, self.T, self.model.vocab_ld), dtype=torch.float16, device=dev) if world > 1 else None
        self.units_per_step = self.B * self.T
        C, L_, V, T = self.cfg.n_embd, self.cfg.n_layer, self.cfg.vocab_size, self.T
        # multiply-adds x 2 per token: the four Linear layers of a block, the lm_head, and both attention GEMMs over the
        # causal half of the [T, T] square (the average query row sees (T + 1) / 2 keys)
        self.flops_per_token = 2.0 * (L_ * (C * 3 * C + C * C + 2 * C * 4 * C) + C * V) + 2.0 * 2.0 * ((T + 1) / 2.0) * C * L_
        self.config = {"batch_total": self.B, "batch_per_gpu": self.Bl, "seq_len": T, "flops_per_token": self.flops_per_token,
                       "gathered_bytes_per_step": self.full.numel() * 2 if world > 1 else 0,
                       "l2": "activations of a layer (50 to 805 MB over all GPUs) and the 3.3 GB of logits against a 126 MB L2"}

    graph = None

    def _compute(self):
        self.logits = self.model.forward(self.idx, logits_out=self.logits_buf)

    def enable_graphs(self):
        self.graph = capture_graph(self._compute)
        return self.graph is not None

    def step_compute(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self._compute()

    def step(self):
        import torch.distributed as dist
        self.step_compute()
        if self.world > 1:
            dist.all_gather_into_tensor(self.full, self.logits_buf)
            self.logits_full = self.full[:, :, : self.cfg.vocab_size]
        else:
            self.logits_full = self.logits

    def e2e_setup(self):
        import torch
        from . import _lib as L
        from . import kernels as K
        self.host_idx = torch.empty(self.idx.shape, dtype=torch.int32).pin_memory()
        self.host_idx.copy_(self.idx)
        self.step_compute()
        # the result a caller reads back: the greedy next-token id at every position (argmax over the vocabulary, one
        # fused reduce launch over this rank's fp16 logits); with several GPUs the ids, not the logits, are gathered
        self.next_ids = K.PreparedReduce([self.logits], L.ARGMAX, [-1], False)
        self.ids_full = torch.empty((self.B, self.T), dtype=torch.int32, device=self.dev) if self.world > 1 else None
        self.host_ids = torch.empty((self.B, self.T), dtype=torch.int32).pin_memory() if self.rank == 0 else None
        self.h2d = self.host_idx.numel() * 4 * self.world
        self.d2h = self.host_ids.numel() * 4 if self.rank == 0 else 0

    def e2e_step(self):
        import torch.distributed as dist
        self.idx.copy_(self.host_idx, non_blocking=True)
        self.step_compute()
        ids = self.next_ids()
        if self.world > 1:
            dist.all_gather_into_tensor(self.ids_full, ids)
            ids = self.ids_full
        if self.rank == 0:
            self.host_ids.copy_(ids, non_blocking=True)

    def roofline(self, pk, reps):
        """The MLP up-projection GEMM (tokens x 3072 x 768, + bias + tanh GELU, fp16 out) timed alone, and per-kernel shares of a
        layer: each kernel eight times back to back in one graph replay (activations of 50 to 200 MB per kernel against a
        126 MB L2; no launch gaps, as inside the step)."""
        import torch
        from . import kernels as K
        dev = self.idx.device
        Bl = self.Bl
        M, C = Bl * self.T, self.cfg.n_embd
        blk = self.model.blocks[0]
        g = torch.Generator(device=dev).manual_seed(7)
        h = (torch.randn((M, C), generator=g, device=dev) * 0.5).half()
        out = torch.empty((M, 4 * C), dtype=torch.float16, device=dev)
        us = _graph_us([lambda: K.matmul(h, blk["fc_wt"].T, bias=blk["fc_b"], act=2, out=out)], 8)
        flops = 2.0 * M * C * 4 * C
        ach = flops / (us * 1e-6) / 1e12
        parts = {}
        x3 = h.view(Bl, self.T, C)
        qkv = K.matmul(x3, blk["attn_wt"].T, bias=blk["attn_b"])
        H, D = self.cfg.n_head, C // self.cfg.n_head
        q, k, v = (qkv[:, :, i * C:(i + 1) * C].view(Bl, self.T, H, D).permute(0, 2, 1, 3) for i in range(3))
        y = torch.empty((Bl, self.T, C), dtype=torch.float16, device=dev)
        parts["layernorm"] = _graph_us([lambda: K.layernorm_rows(x3, blk["ln1_g"], blk["ln1_b"], 1e-5)], 8)
        parts["qkv_gemm"] = _graph_us([lambda: K.matmul(x3, blk["attn_wt"].T, bias=blk["attn_b"], out=qkv)], 8)
        y_heads = y.view(Bl, self.T, H, D).permute(0, 2, 1, 3)
        parts["fused_attention"] = _graph_us([lambda: K.attention(q, k, v, scale=0.125, causal=True, out=y_heads)], 8)
        parts["proj_gemm"] = _graph_us([lambda: K.matmul(y, blk["proj_wt"].T, bias=blk["proj_b"], residual=x3, out=y)], 8)
        parts["fc_gemm_gelu"] = us
        parts["fc2_gemm"] = _graph_us([lambda: K.matmul(out.view(Bl, self.T, 4 * C), blk["fc2_wt"].T, bias=blk["fc2_b"], residual=x3, out=y)], 8)
        parts["lm_head_gemm"] = _graph_us([lambda: K.matmul(x3, self.model.lm_head_t.T, out=self.logits_buf[:, :, : self.cfg.vocab_size])], 3)
        att_flops = 2.0 * 2.0 * Bl * H * self.T * ((self.T + 1) / 2.0) * D
        return {"bound": "tensor", "kernel": "gemm_tc_kernel<f16> %dx3072x768 + bias + GELU epilogue" % M, "achieved": round(ach, 1),
                "peak": pk["f16_sustained"], "unit": "TFLOP/s", "frac": round(ach / pk["f16_sustained"], 4),
                "peak_source": pk["source"] + " (sustained bf16 cuBLAS rate: the kernel runs inside a long step)", "traffic": None,
                "us": round(us, 1), "algorithmic_flops_per_launch": flops, "kernel_us": {k_: round(v_, 1) for k_, v_ in parts.items()},
                "fused_attention_tflops_causal": round(att_flops / (parts["fused_attention"] * 1e-6) / 1e12, 1)}


class Rows:
    """Causal row softmax over fp16 scores [32,12,1024,1024] and LayerNorm over fp32 [16384,768], one kernel each;
    over several GPUs the scores are split along the batch dim and the LayerNorm rows in blocks."""
    name, metric, unit, dtype = "rows", "softmax+LayerNorm HBM GB/s", "GB/s", "f16/f32"
    SM_SHAPE, LN_SHAPE = (32, 12, 1024, 1024), (16384, 768)

    def __init__(self):
        self.desc = ("row softmax over fp16 scores [32,12,1024,1024] N(0,1) with causal mask; LayerNorm over fp32 [16384,768] N(0,1), "
                     "gamma=1+N(0,0.02), beta=N(0,0.02), eps=1e-5; a single kernel each; rows split over the GPUs")

    def setup(self, dev, rank, world):
        import torch
        from . import distrib as D
        self.dev, self.rank, self.world = dev, rank, world
        g = torch.Generator(device=dev).manual_seed(4)
        devs = _devices(world)
        S = torch.randn(self.SM_SHAPE, generator=g, device=dev).half()
        self.S = D.shard_tensor(S, world, 0, devs).shards[0]
        del S
        X = torch.randn(self.LN_SHAPE, generator=g, device=dev)
        self.X = D.shard_tensor(X, world, 0, devs).shards[0]
        del X
        self.gamma = 1 + 0.02 * torch.randn(768, generator=g, device=dev)
        self.beta = 0.02 * torch.randn(768, generator=g, device=dev)
        T = self.SM_SHAPE[-1]
        n_rows = int(np.prod(self.SM_SHAPE[:-1]))
        # algorithmic bytes: every score read once and every probability written once; a causal kernel may skip the
        # masked half of the reads (the second figure), the roofline is charged with the full count
        self.sm_bytes = 2 * n_rows * T * 2
        self.sm_bytes_triangle = n_rows * (T + 1) // 2 * 2 + n_rows * T * 2
        self.ln_bytes = int(np.prod(self.LN_SHAPE)) * 8 + 768 * 8
        self.units_per_step = (self.sm_bytes + self.ln_bytes) / 1e9
        if world > 1:
            self.sm_full = torch.empty(self.SM_SHAPE, dtype=torch.float16, device=dev)
            self.ln_full = torch.empty(self.LN_SHAPE, dtype=torch.float32, device=dev)
        self.config = {"softmax_bytes": self.sm_bytes, "softmax_bytes_reading_the_triangle_only": self.sm_bytes_triangle,
                       "layernorm_bytes": self.ln_bytes, "gathered_bytes_per_step": (self.sm_bytes // 2 + self.ln_bytes // 2) if world > 1 else 0,
                       "l2": "the scores (805 MB over all GPUs) against a 126 MB L2; the LayerNorm input is flushed by the softmax between launches"}

    def step_compute(self):
        """The two kernels do not depend on one another: the LayerNorm runs on a stream that forks from and joins the
        timed one, under the softmax, where the shard is large enough for that to pay (one or two GPUs: 249 against
        256 us on one; on an eighth of the rows the two event hand-overs cost more than the 4 us kernel they hide:
        73 against 48 us)."""
        import torch
        from . import kernels as K
        if getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream(device=self.S.device)
            self.sm_out = torch.empty_like(self.S)
            self.ln_out = torch.empty_like(self.X)
        if self.world > 2:
            K.softmax_rows(self.S, causal=True, out=self.sm_out)
            K.layernorm_rows(self.X, self.gamma, self.beta, 1e-5, out=self.ln_out)
            return
        main = torch.cuda.current_stream()
        fork = torch.cuda.Event()
        fork.record(main)
        self._side.wait_event(fork)
        with torch.cuda.stream(self._side):
            K.layernorm_rows(self.X, self.gamma, self.beta, 1e-5, out=self.ln_out)
        K.softmax_rows(self.S, causal=True, out=self.sm_out)
        join = torch.cuda.Event()
        join.record(self._side)
        main.wait_event(join)

    def step(self):
        import torch.distributed as dist
        self.step_compute()
        if self.world > 1:
            dist.all_gather_into_tensor(self.sm_full, self.sm_out)
            dist.all_gather_into_tensor(self.ln_full, self.ln_out)

    def e2e_setup(self):
        import torch
        self.host_x = torch.empty(self.X.shape, dtype=torch.float32).pin_memory()
        self.host_x.copy_(self.X)
        self.host_y = torch.empty(self.LN_SHAPE, dtype=torch.float32).pin_memory() if self.rank == 0 else None
        self.h2d = self.host_x.numel() * 4 * self.world
        self.d2h = self.host_y.numel() * 4 if self.rank == 0 else 0

    def e2e_step(self):
        # the scores of an attention layer never leave the device in use; LayerNorm rows go both ways
        self.X.copy_(self.host_x, non_blocking=True)
        self.step()
        if self.rank == 0:
            self.host_y.copy_(self.ln_full if self.world > 1 else self.ln_out, non_blocking=True)

    def roofline(self, pk, reps):
        from . import kernels as K
        flush = _L2Flush(self.dev)
        w = self.world
        sm_us = _event_us(lambda: K.softmax_rows(self.S, causal=True), reps, flush=flush if w > 1 else None)
        ln_single_us = _event_us(lambda: K.layernorm_rows(self.X, self.gamma, self.beta, 1e-5), reps, flush=flush)
        # The LayerNorm launch is short enough for the event timestamps' granularity to matter: time 48 launches in one
        # graph over a ring of five input / output pairs (500 MB over all GPUs' worth of rows: no launch finds its rows
        # in L2). Yardstick: the vendor's device copy of the same tensors (the same bytes, no arithmetic, no row
        # dependency), timed the same way.
        import torch
        ring = [(self.X if i == 0 else self.X.clone(), torch.empty_like(self.X)) for i in range(5 if w == 1 else 9)]
        xd = [(K.desc(a), K.desc(b)) for a, b in ring]
        from . import _lib as L_
        import ctypes as C_
        gd, bd = K.desc(self.gamma), K.desc(self.beta)
        lib = L_.lib()

        def ln_call(i):
            def f():
                L_.check(lib.pgb_layernorm_rows(C_.byref(xd[i][0]), C_.byref(gd), C_.byref(bd), 1e-5, C_.byref(xd[i][1]),
                                                torch.cuda.current_stream().cuda_stream))
            return f
        ln_us = _graph_us([ln_call(i) for i in range(len(ring))])
        copy_us = _graph_us([(lambda a=a, b=b: b.copy_(a)) for a, b in ring])
        del flush, ring
        ach = self.sm_bytes / w / (sm_us * 1e-6) / 1e9
        tri = self.sm_bytes_triangle / w / (sm_us * 1e-6) / 1e9
        ln = self.ln_bytes / w / (ln_us * 1e-6) / 1e9
        return {"bound": "hbm", "kernel": "softmax_rows (causal, fp16, 1024 columns)", "achieved": round(ach, 1), "peak": pk["hbm"], "unit": "GB/s",
                "frac": round(ach / pk["hbm"], 4), "peak_source": pk["source"], "traffic": None, "us": round(sm_us, 1),
                "algorithmic_bytes_per_launch": self.sm_bytes // w,
                "counting_only_the_triangle_read": {"bytes": self.sm_bytes_triangle // w, "gbs": round(tri, 1), "frac": round(tri / pk["hbm"], 4)},
                "layernorm": {"gbs": round(ln, 1), "frac": round(ln / pk["hbm"], 4), "us": round(ln_us, 2), "bytes": self.ln_bytes // w,
                              "timing": "mean of 48 launches replayed as one CUDA graph over a ring of buffers larger than the L2",
                              "single_launch_between_two_events_us": round(ln_single_us, 1),
                              "device_copy_of_the_same_tensor_us": round(copy_us, 2)}}


class Readme:
    """The README fusion case: f(x, y) = sum(permute(x,(0,2,1)) + 2 + y, axis=2) * 3 over x [1000,20,100] and
    y [1000,100,20], one fused kernel. 16.4 MB: it fits the L2 and is bound by launch latency, so the metric is
    the kernel's time: warm (same buffers again and again) and cold (a ring of buffer pairs larger than the L2)."""
    name, metric, unit, dtype = "readme", "README fusion case time per call", "us", "f32"
    RING = 16  # 16 x 16 MB of inputs: nothing of a pair is left in the 126 MB L2 when its turn comes again

    def __init__(self):
        self.desc = ("README JIT fusion case: x float32 [1000,20,100], y float32 [1000,100,20] uniform[0,1); "
                     "sum(permute(x,(0,2,1)) + 2 + y, axis=2) * 3 as a single fused reduce kernel")

    def setup(self, dev, rank, world):
        import torch
        from . import _lib as L
        from . import kernels as K
        self.dev, self.rank, self.world = dev, rank, world
        g = torch.Generator(device=dev).manual_seed(1)
        self.pairs = [(torch.rand((1000, 20, 100), generator=g, device=dev), torch.rand((1000, 100, 20), generator=g, device=dev)) for _ in range(self.RING)]
        self.calls = [K.PreparedReduce([x.permute(0, 2, 1), y], L.SUM, [2], False, README_PRO, README_EPI) for x, y in self.pairs]
        self.stream = torch.cuda.current_stream().cuda_stream
        self.bytes = 8_000_000 + 8_000_000 + 400_000
        self.units_per_step = float(self.RING)  # calls per step
        self.config = {"algorithmic_bytes": self.bytes, "kernel": self.calls[0].plan,
                       "l2": f"a timed step = {self.RING} calls, one per buffer pair of a ring (262 MB in all), so no call finds its inputs in L2; "
                             "value = microseconds per call; the warm time is in roofline"}

    graph = None

    def _ring(self):
        for c in self.calls:
            self.out = c()

    def enable_graphs(self):
        self.graph = capture_graph(self._ring)
        return self.graph is not None

    def step_compute(self):
        """One pass over the ring: RING calls, each on a buffer pair that has left the L2 since its last turn."""
        if self.graph is not None:
            self.graph.replay()
        else:
            self._ring()

    step = step_compute  # 16 MB, launch-latency bound: not partitioned; with several GPUs every rank runs the whole case

    def e2e_setup(self):
        import torch
        x, y = self.pairs[0]
        self.host_x, self.host_y = (torch.empty(t.shape, dtype=torch.float32).pin_memory() for t in (x, y))
        self.host_x.copy_(x)
        self.host_y.copy_(y)
        self.host_out = torch.empty((1000, 100), dtype=torch.float32).pin_memory()
        self.h2d, self.d2h = 16_000_000, 400_000

    def e2e_step(self):
        x, y = self.pairs[0]
        x.copy_(self.host_x, non_blocking=True)
        y.copy_(self.host_y, non_blocking=True)
        self.host_out.copy_(self.calls[0](), non_blocking=True)

    def roofline(self, pk, reps):
        # 48 launches per graph: a single launch of a 10 us kernel is below what two events resolve
        warm = _graph_us([lambda: self.calls[0]()])
        cold = _graph_us([(lambda c=c: c()) for c in self.calls])
        gbs = self.bytes / (cold * 1e-6) / 1e9
        return {"bound": "hbm", "kernel": self.calls[0].plan.split()[0], "achieved": round(gbs, 1), "peak": pk["hbm"], "unit": "GB/s",
                "frac": round(gbs / pk["hbm"], 4), "peak_source": pk["source"], "traffic": None,
                "note": "16.4 MB: 2.5 us at the HBM peak, so launch latency and L2 behaviour decide the time, not the roofline",
                "warm_us": round(warm, 2), "cold_us": round(cold, 2), "warm_gbs_from_l2": round(self.bytes / (warm * 1e-6) / 1e9, 1),
                "algorithmic_bytes_per_launch": self.bytes}
