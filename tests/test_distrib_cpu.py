"""The sharding layer on two CPU ranks over gloo (the host logic of the multi-GPU path;
the reference tests its "devices" as aliases of one GPU, tests/test_device.py:21-38)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, scenario, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    from pequegrad_b200 import distrib as D
    try:
        D.init("gloo", timeout_s=8.0)
        g = torch.Generator().manual_seed(7)
        x = torch.randn((11, 6, 5), generator=g)  # every rank builds the same "global" tensor; 11 rows split unevenly
        devs = D.default_devices()
        if scenario == "roundtrip":
            for dim in (0, 1, 2, -1):
                st = D.shard_tensor(x, world, dim, devs)
                lo, hi = D.shard_range(x.shape[dim], rank, world)
                assert st.shards[0].shape[dim] == hi - lo and st.shape == list(x.shape) and st.dim == [dim % 3]
                assert torch.equal(D.unshard_tensor(st, dim), x)
                assert torch.equal(D.unshard_tensor(st, None), x)
            assert torch.equal(D.unshard_tensor(D.shard_tensor(x, world, None, devs)), x)
            # four shards over two processes: each process holds two of them
            st = D.shard_tensor(x, 4, 0)
            assert len(st.shards) == 2 and torch.equal(D.unshard_tensor(st, 0), x)
            with pytest.raises(ValueError):
                D.shard_tensor(x, 3, 0)  # 3 shards do not spread over 2 processes
            with pytest.raises(ValueError):
                D.shard_tensor(x, 2, 0, ["cpu:0"])  # num_shards must match the devices
            q.put((rank, "ok"))
        elif scenario == "pmap":
            # the reference's convention: the split dim has one entry per device and is dropped
            y = torch.randn((world, 5, 6), generator=g)
            w = torch.tensor(2.0)
            fn = lambda t, s: (t * 1.5 + 0.25).sum(-1).exp() * s  # noqa: E731
            want = fn(y, w)  # [world, 5]
            assert torch.allclose(D.pmap(fn, devs, [0, None], out_opts=0)(y, w), want)
            assert torch.allclose(D.pmap(fn, devs, [0, None], out_opts=1)(y, w), want.T)
            # default: outputs are averaged over the devices, as the reference does with losses and gradients
            assert torch.allclose(D.pmap(fn, devs, [0, None])(y, w), want.mean(0), atol=1e-6)
            # split along a middle dim; two outputs with different treatment; no collective for "sharded"
            z = torch.randn((4, world, 3), generator=g)
            a, b = D.pmap(lambda t: (t.sum(0), t * 2), devs, [1], out_opts=[0, "sharded"])(z)
            assert torch.allclose(a, z.sum(0)) and len(b) == 1 and torch.equal(b[0], z[:, rank] * 2)
            # four emulated devices on two processes
            z4 = torch.randn((4, 7), generator=g)
            assert torch.allclose(D.pmap(lambda t: t.amax(), D.default_devices(4), [0], out_opts=0)(z4), z4.amax(1))
            for bad in (lambda: D.pmap(fn, devs, [0])(y, w), lambda: D.pmap(fn, devs, [1, None])(y, w),
                        lambda: D.pmap(fn, devs, [0, None], out_opts=3)(y, w), lambda: D.pmap(fn, devs, [0, None], out_opts="cat")(y, w)):
                with pytest.raises(ValueError):
                    bad()
            # sharding the REDUCED axis needs an all-reduce instead
            part = D.shard_tensor(x, world, 0).shards[0].sum(0)
            assert torch.allclose(D.all_reduce(part.clone(), "sum"), x.sum(0), atol=1e-5)
            assert torch.allclose(D.all_reduce([part.clone()], "avg"), x.sum(0) / world, atol=1e-5)
            mx = [s.amax(0) for s in D.shard_tensor(x, 4, 0).shards]  # two local shards per process
            assert torch.equal(D.all_reduce(mx, "max"), x.amax(0)) and all(torch.equal(m, x.amax(0)) for m in mx)
            with pytest.raises(ValueError):
                D.all_reduce(part.clone(), "min")
            with pytest.raises(ValueError):
                D.all_reduce(torch.ones(3, dtype=torch.int32), "avg")
            q.put((rank, "ok"))
        elif scenario == "reshard":
            # rows -> column slabs (and a middle dim of a 3-D tensor) by one all-to-all
            a = torch.randn((8, 6), generator=g)
            cols = D.reshard_tensor(D.shard_tensor(a, world, 0, devs), 1)
            assert cols.dim == [1] and torch.equal(cols.shards[0], D.shard_tensor(a, world, 1, devs).shards[0])
            assert torch.equal(D.unshard_tensor(cols, 1), a)
            b3 = torch.randn((4, 6, 5), generator=g)
            mid = D.reshard_tensor(D.shard_tensor(b3, world, 0, devs), 1)
            assert torch.equal(mid.shards[0], D.shard_tensor(b3, world, 1, devs).shards[0])
            with pytest.raises(ValueError):
                D.reshard_tensor(D.shard_tensor(a, world, 1, devs), 0)
            q.put((rank, "ok"))
        elif scenario == "bucket":
            # several outputs behind one collective: slabs along dim 0 come back as views, other dims as one copy
            bk = D.GatherBucket("cpu")
            i0 = bk.add((3, 5), torch.float32, 0)
            i1 = bk.add((4, 2), torch.int32, 1)
            i2 = bk.add((), torch.float32, 0)
            bk.local_view(i0).copy_(torch.arange(15.0).view(3, 5) + 100 * rank)
            bk.local_view(i1).copy_(torch.arange(8, dtype=torch.int32).view(4, 2) + 10 * rank)
            bk.local_view(i2).fill_(float(rank))
            bk.gather()
            bk.wait()
            f0 = bk.full(i0)
            assert f0.shape == (world, 3, 5) and all(torch.equal(f0[r], torch.arange(15.0).view(3, 5) + 100 * r) for r in range(world))
            f1 = bk.full(i1)
            want1 = torch.cat([torch.arange(8, dtype=torch.int32).view(4, 2) + 10 * r for r in range(world)], 1)
            assert f1.shape == (4, 2 * world) and torch.equal(f1, want1)
            assert torch.equal(bk.full(i2), torch.arange(float(world)))
            # asked for the peer-memory gather where no peer mapping can exist (CPU ranks): every rank falls back to the
            # library collective together, and says so
            bp = D.GatherBucket("cpu", peer_memory=True)
            j0 = bp.add((2, 3), torch.float32, 0)
            bp.local_view(j0).copy_(torch.arange(6.0).view(2, 3) + 7 * rank)
            assert bp.peers is None and bp.peer_note.startswith("NCCL (peer mapping unavailable")
            bp.gather()
            bp.wait()
            g0 = bp.full(j0)
            assert all(torch.equal(g0[r], torch.arange(6.0).view(2, 3) + 7 * r) for r in range(world))
            q.put((rank, "ok"))
        elif scenario == "matmul":
            a, b = torch.randn((8, 6), generator=g), torch.randn((6, 10), generator=g)
            rows = D.shard_tensor(a, world, 0, devs) @ D.shard_tensor(b, world, None, devs)
            cols = D.shard_tensor(a, world, None, devs) @ D.shard_tensor(b, world, 1, devs)
            assert rows.dim == [0] and cols.dim == [1] and rows.shape == [8, 10]
            assert torch.allclose(D.unshard_tensor(rows, 0), a @ b, atol=1e-5)
            assert torch.allclose(D.unshard_tensor(cols, 1), a @ b, atol=1e-5)
            assert np.allclose(cols.numpy(), (a @ b).numpy(), atol=1e-5)
            with pytest.raises(ValueError):
                D.shard_tensor(a, world, 0, devs) @ D.shard_tensor(b, world, 0, devs)
            q.put((rank, "ok"))
        elif scenario == "rank_lost":
            # rank 1 leaves between steps, before the gather: rank 0's gather must fail within the group timeout
            if rank == 1:
                q.put((rank, "left"))
                return
            try:
                D.unshard_tensor(D.shard_tensor(x, world, 0))
                q.put((rank, "gather returned"))
            except Exception as e:  # noqa: BLE001 - any distributed error is the expected outcome
                q.put((rank, "error:" + type(e).__name__))
    except Exception as e:  # noqa: BLE001
        q.put((rank, "FAILED " + repr(e)))
    finally:
        if dist.is_initialized() and scenario != "rank_lost":
            dist.destroy_process_group()


def _run(scenario, world=2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, scenario, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.kill()
    return res


@pytest.mark.parametrize("scenario", ["roundtrip", "pmap", "reshard", "bucket", "matmul"])
def test_two_ranks(scenario):
    assert _run(scenario) == {0: "ok", 1: "ok"}


def test_lost_rank_is_reported_not_waited_for_forever():
    res = _run("rank_lost")
    assert res[1] == "left" and res[0].startswith("error:"), res


def test_single_process_holds_every_shard():
    """Without a process group one process owns all the shards, like the reference's emulated devices."""
    from pequegrad_b200 import distrib as D
    x = torch.arange(24.0).reshape(6, 4)
    assert D.rank_world() == (0, 1)
    assert torch.equal(D.unshard_tensor(D.shard_tensor(x, 1, 0)), x)
    st = D.shard_tensor(x, 3, 0, ["cpu:0", "cpu:1", "cpu:2"])
    assert len(st.shards) == 3 and st.shape == [6, 4] and torch.equal(D.unshard_tensor(st, 0), x)
    st1 = D.shard_tensor(x, 2, 1)
    assert torch.equal(D.unshard_tensor(st1, 1), x) and torch.equal(torch.from_numpy(st1.numpy()), x)
    assert [D.shard_range(10, r, 4) for r in range(4)] == [(0, 2), (2, 5), (5, 7), (7, 10)]
    y = x.reshape(3, 2, 4)
    assert torch.equal(D.pmap(lambda t: t * 2, D.default_devices(3), [0], out_opts=0)(y), y * 2)
    assert torch.equal(D.pmap(lambda t: t.sum(), None, [None])(x), x.sum())
    tot = D.all_reduce([torch.ones(2), torch.full((2,), 3.0)], "avg")
    assert torch.equal(tot, torch.full((2,), 2.0))
