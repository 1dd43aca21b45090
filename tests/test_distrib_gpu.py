"""The sharding layer over the kernels of this library on real devices.

One GPU: a process that holds every shard (what the reference's emulated devices do,
examples/data_parallel_mlp.py:28-31) runs `pmap` / `shard_tensor` over pgb kernels and must give the
unsharded results. Two GPUs (skipped below that): two processes over NCCL run the same checks and the
benchmark's partitioned workloads, whose gathered results must equal the single-GPU ones."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from pequegrad_b200 import _lib as L
from pequegrad_b200 import distrib as D
from pequegrad_b200 import kernels as K
from pequegrad_b200.workloads import AFFINE, EXP_EPI

pytestmark = pytest.mark.gpu


def _reduce(op, ax, epi=()):
    return lambda t: K.fused_reduce([t], op, [ax], False, AFFINE, epi)


def _check_pmap_over_reduces(x3, devs):
    """x3: [P, rows / P, cols] on the device. Row-sharded fused reduces through pmap == the reduce over all rows."""
    P, r, c = x3.shape
    flat = x3.reshape(P * r, c)
    got = D.pmap(_reduce(L.MAX, 1), devs, [0], out_opts=0)(x3).reshape(-1)
    assert torch.equal(got, _reduce(L.MAX, 1)(flat))
    got = D.pmap(_reduce(L.ARGMAX, 1), devs, [0], out_opts=0)(x3).reshape(-1)
    assert torch.equal(got, _reduce(L.ARGMAX, 1)(flat))
    got = D.pmap(_reduce(L.SUM, 1, EXP_EPI), devs, [0], out_opts=0)(x3).reshape(-1)
    want = _reduce(L.SUM, 1, EXP_EPI)(flat)
    assert torch.allclose(got, want, rtol=1e-5, atol=0)  # the row kernel may split rows differently: not the same bits
    # column reduce with the columns split: shards arrive as [rows, cols / P] slabs and come back side by side
    xt = x3.permute(1, 0, 2)  # [r, P, c]: P column blocks of an [r, P * c] matrix
    got = D.pmap(_reduce(L.MAX, 0), devs, [1], out_opts=0)(xt).reshape(-1)
    assert torch.equal(got, _reduce(L.MAX, 0)(xt.reshape(r, P * c)))
    # the reference's default: outputs averaged over the devices
    got = D.pmap(lambda t: _reduce(L.MEAN, 0)(t), devs, [0])(x3)
    assert torch.allclose(got, flat.mul(1.5).add(0.25).mean(0), rtol=1e-4, atol=1e-5)


def test_one_process_holding_every_shard():
    g = torch.Generator(device="cuda").manual_seed(21)
    for P in (2, 4):
        x3 = torch.randn((P, 96, 1500), generator=g, device="cuda")
        _check_pmap_over_reduces(x3, D.default_devices(P))
    # shard_tensor -> kernels on every shard -> unshard_tensor
    x = torch.randn((1000, 777), generator=g, device="cuda")
    st = D.shard_tensor(x, 4, 0, D.default_devices(4))
    outs = D.ShardedTensor([_reduce(L.MAX, 1)(s) for s in st.shards], [0], 4, [1000])
    assert torch.equal(D.unshard_tensor(outs, 0), _reduce(L.MAX, 1)(x))
    st = D.shard_tensor(x, 3, 1)  # uneven column slabs
    outs = D.ShardedTensor([_reduce(L.ARGMAX, 0)(s) for s in st.shards], [0], 3, [777])
    assert torch.equal(D.unshard_tensor(outs, 0), _reduce(L.ARGMAX, 0)(x))


def test_sweep_on_two_streams_and_as_graphs_gives_the_same_bits():
    # the benchmark launches the independent cases of a step alternately on two streams that fork from and join the
    # timed one, inside CUDA graphs: same results, bit for bit, as one kernel after another
    from pequegrad_b200 import workloads as W
    torch.cuda.set_device(0)
    res = {}
    for lanes, graphs in ((1, False), (2, False), (2, True), (3, True)):
        wl = W.Sweep(only="A,Bp")
        wl.lanes = lanes
        wl.setup(torch.device("cuda:0"), 0, 1)
        if graphs:
            assert wl.enable_graphs()
        wl.step()
        wl.step()
        torch.cuda.synchronize()
        res[(lanes, graphs)] = {k_: v_.clone() for k_, v_ in wl.results()}
        del wl
        torch.cuda.empty_cache()
    base = res[(1, False)]
    assert len(base) == 24
    for key, r in res.items():
        for name, t in r.items():
            assert torch.equal(t.view(torch.int32), base[name].view(torch.int32)), (key, name)


def test_one_gpu_end_to_end_step_with_overlapped_copies_returns_the_steps_results():
    # bench.py's e2e leg on one GPU: uploads on a copy stream, A's cases under B's upload, the axis-0 results copied back
    # under the remaining kernels; the host buffers must hold exactly what a plain step leaves on the device
    from pequegrad_b200 import workloads as W
    torch.cuda.set_device(0)
    wl = W.Sweep()
    wl.setup(torch.device("cuda:0"), 0, 1)
    wl.step()
    torch.cuda.synchronize()
    want = [b.recv.clone() for b in wl.buckets]
    wl.e2e_setup()
    for b in wl.buckets:
        b.recv.zero_()
    for _ in range(3):
        wl.e2e_step()
    torch.cuda.synchronize()
    for have, w, b in zip(wl.host_out, want, wl.buckets):
        assert torch.equal(b.recv, w)
        assert torch.equal(have, w.cpu())
    assert wl.h2d == 4 * (8192 * 8192 + 64 * 4096 * 1024) and wl.d2h == sum(w.numel() for w in want)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      NCCL_NVLS_ENABLE="0")
    try:
        D.init("nccl", timeout_s=120.0)
        dev = torch.device("cuda", rank)
        g = torch.Generator(device=dev).manual_seed(21)
        x3 = torch.randn((world, 96, 1500), generator=g, device=dev)
        _check_pmap_over_reduces(x3, D.default_devices(world))

        # the benchmark's partitioned sweep: gathered results == the unsharded kernels on the global arrays
        from pequegrad_b200 import workloads as W
        wl = W.Sweep()
        wl.setup(dev, rank, world)
        wl.step()
        wl.step()
        torch.cuda.synchronize()
        got = {k_: v_.clone() for k_, v_ in wl.results()}  # the results are views of buffers the next step reuses
        g2 = torch.Generator(device=dev).manual_seed(2)
        T = {"A": torch.randn(W.SHAPES["A"], generator=g2, device=dev)}
        T["B"] = torch.randn(W.SHAPES["B"], generator=g2, device=dev)
        T["Bp"] = T["B"].permute(0, 2, 1)
        opcode = {"sum": L.SUM, "max": L.MAX, "mean": L.MEAN, "argmax": L.ARGMAX}
        for name, op, ax, _ in wl.cases:
            want = K.fused_reduce([T[name]], opcode[op], [ax], False, AFFINE, () if op == "argmax" else EXP_EPI)
            have = got[f"{name}.{op}.ax{ax}"]
            assert have.shape == want.shape, (name, op, ax, have.shape, want.shape)
            if op in ("max", "argmax"):
                assert torch.equal(have, want), (name, op, ax)
            else:
                both_inf = torch.isinf(have) & torch.isinf(want)
                assert torch.allclose(torch.where(both_inf, 0, have), torch.where(both_inf, 0, want), rtol=2e-5, atol=0), (name, op, ax)
        # the end-to-end step: row shards uploaded from the host, the second sharding made by an all-to-all on the
        # devices; the shards it rebuilds must be the ones the set-up made, and the results the same
        b1_before, a1_before = wl.S["B1"].clone(), wl.S["A1"].clone()
        wl.e2e_setup()
        wl.S["B1"].zero_()
        wl.S["A1"].zero_()
        wl.e2e_step()
        torch.cuda.synchronize()
        assert torch.equal(wl.S["B1"], b1_before) and torch.equal(wl.S["A1"], a1_before)
        again = dict(wl.results())
        for k_, v_ in again.items():
            if ".max." in k_ or ".argmax." in k_:
                assert torch.equal(v_, got[k_]), k_
        del wl, T, got, again
        torch.cuda.empty_cache()

        # the peer-memory collectives: a max of one float and a gather of small slabs, many calls in a row
        pg = D.PeerGroup(gather_bytes=3 * 1000 * 4)
        for i in range(50):
            v = torch.tensor([float(rank * 7 + i)], device=dev)
            pg.allreduce_max(v)
            assert float(v) == float((world - 1) * 7 + i), (i, float(v))
            slab = torch.full((3, 1000), float(rank + 10 * i), device=dev)
            got_all = pg.allgather(slab)
            torch.cuda.synchronize()
            assert got_all.shape == (world, 3, 1000)
            assert all(bool((got_all[r] == float(r + 10 * i)).all()) for r in range(world)), i
        assert K.device_error() == 0
        pg.close()

        # the int8 MLP split by rows: the bits of the single-GPU forward over the whole batch,
        # with the exchanges through NCCL and through the peer-memory kernels
        m0 = W.Mlp(rows=16384, use_peers=False)
        m0.setup(dev, rank, world)
        m0.step()
        nccl_out = m0.out_full.clone()
        del m0
        m = W.Mlp(rows=16384)
        m.setup(dev, rank, world)
        assert m.peers is not None, m.peer_note
        m.step()
        m.step()
        assert torch.equal(m.out_full, nccl_out)
        # the same step replayed as a CUDA graph (peer kernels included): same bits, call after call
        assert m.enable_graphs()
        for _ in range(3):
            m.step()
            m.step_compute()
        m.step()
        torch.cuda.synchronize()
        assert torch.equal(m.out_full, nccl_out)
        g3 = torch.Generator(device=dev).manual_seed(3)
        X = torch.rand((16384, 784), generator=g3, device=dev)
        whole = m.mlp.forward_sharded([X])[0]  # one shard per process holding ALL rows: both ranks compute the same thing
        assert torch.equal(m.out_full, whole)
        assert K.device_error() == 0
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, "FAILED " + repr(e) + traceback.format_exc()[-1500:]))
    finally:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_over_nccl():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=600) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        if p.is_alive():
            p.kill()
    assert res == {0: "ok", 1: "ok"}, res


def test_a_peer_that_never_arrives_is_reported_not_waited_for_forever():
    """Failure detection on the device without a fault: rank 0 of a made-up group of two runs the max exchange, but
    the control block standing in for rank 1 is a plain local allocation that nobody ever writes to. The kernel's
    wait for rank 1's contribution must run out (a short poll limit keeps it to about a millisecond), the error
    word must name the peer exchange (role 10), the value must be left alone, and the device must stay usable."""
    import ctypes as C
    lib = L.lib()
    assert K.device_error() == 0
    blocks = []
    for _ in range(2):
        p = C.c_void_p()
        L.check(lib.pgb_peer_alloc(lib.pgb_peer_ctrl_bytes(), C.byref(p)))
        blocks.append(p.value)
    ctrl = (C.c_void_p * 2)(*blocks)
    old = lib.pgb_peer_poll_limit(1 << 12)
    try:
        v = torch.tensor([3.5], device="cuda")
        L.check(lib.pgb_peer_allreduce_max_f32(v.data_ptr(), ctrl, 0, 2, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()  # returns: the wait was bounded
        code = C.c_int(0)
        assert lib.pgb_device_error(C.byref(code), 1) == L.ERR_TIMEOUT
        assert code.value >> 16 == 10 and (code.value & 0xffff) == 0
        assert float(v) == 3.5
        # with a group of one (this rank alone) the same kernel completes: its own contribution is all it needs
        solo = (C.c_void_p * 1)(blocks[0])
        L.check(lib.pgb_peer_allreduce_max_f32(v.data_ptr(), solo, 0, 1, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert K.device_error() == 0 and float(v) == 3.5
    finally:
        lib.pgb_peer_poll_limit(old)
        for b in blocks:
            lib.pgb_peer_free(b)
    x = torch.randn((64, 4096), device="cuda")
    assert torch.equal(K.fused_reduce([x], L.MAX, [1]), x.amax(1))
