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
        if scenario == "roundtrip":
            for dim in (0, 1, 2, -1):
                st = D.shard_tensor(x, dim)
                lo, hi = D.shard_range(x.shape[dim], rank, world)
                assert st.local.shape[dim] == hi - lo and st.global_shape == tuple(x.shape)
                assert torch.equal(D.unshard_tensor(st), x)
            assert torch.equal(D.unshard_tensor(D.shard_tensor(x, None)), x)
            q.put((rank, "ok"))
        elif scenario == "pmap":
            # row-sharded reduction with prologue and epilogue: no exchange, one gather at the end
            f = D.pmap(lambda t, w: ((t * 1.5 + 0.25).sum(-1).exp() * w), (0, None))
            w = torch.tensor(2.0)
            out = f(x, w)
            assert torch.allclose(out, (x * 1.5 + 0.25).sum(-1).exp() * 2.0)
            st = D.pmap(lambda t: t.amax(1), (0,), gather=False)(x)
            assert st.dim == 0 and st.global_shape == (11, 5)
            # sharding the REDUCED axis needs an all-reduce instead
            part = D.shard_tensor(x, 0).local.sum(0)
            assert torch.allclose(D.all_reduce(part.clone(), "sum"), x.sum(0), atol=1e-5)
            mx = D.shard_tensor(x, 0).local.amax(0)
            assert torch.equal(D.all_reduce(mx.clone(), "max"), x.amax(0))
            q.put((rank, "ok"))
        elif scenario == "matmul":
            a, b = torch.randn((8, 6), generator=g), torch.randn((6, 10), generator=g)
            rows = D.shard_tensor(a, 0) @ D.shard_tensor(b, None)
            cols = D.shard_tensor(a, None) @ D.shard_tensor(b, 1)
            assert torch.allclose(D.unshard_tensor(rows), a @ b, atol=1e-5)
            assert torch.allclose(D.unshard_tensor(cols), a @ b, atol=1e-5)
            q.put((rank, "ok"))
        elif scenario == "rank_lost":
            # rank 1 leaves between steps, before the gather: rank 0's gather must fail within the group timeout
            if rank == 1:
                q.put((rank, "left"))
                return
            try:
                D.unshard_tensor(D.shard_tensor(x, 0))
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


@pytest.mark.parametrize("scenario", ["roundtrip", "pmap", "matmul"])
def test_two_ranks(scenario):
    assert _run(scenario) == {0: "ok", 1: "ok"}


def test_lost_rank_is_reported_not_waited_for_forever():
    res = _run("rank_lost")
    assert res[1] == "left" and res[0].startswith("error:"), res


def test_single_process_is_identity():
    from pequegrad_b200 import distrib as D
    x = torch.arange(12.0).reshape(3, 4)
    assert D.rank_world() == (0, 1)
    assert torch.equal(D.unshard_tensor(D.shard_tensor(x, 0)), x)
    assert [D.shard_range(10, r, 4) for r in range(4)] == [(0, 2), (2, 5), (5, 7), (7, 10)]
    assert torch.equal(D.pmap(lambda t: t * 2, (0,))(x), x * 2)
