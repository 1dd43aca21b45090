"""Batch / row sharding over the GPUs of one box: one process per GPU.

Keeps the API shape of the reference's `pequegrad/distrib`
(`shard_tensor`, `unshard_tensor`, `ShardedTensor`, `all_reduce`,
pequegrad/distrib/sharded_tensor.py:7-95, distrib/__init__.py:4-62) and of
`pmap` (pequegrad/transforms/distrib.py:31-163). The reference emulates its
devices on one GPU and moves data with Python loops; here every rank owns a
real device, computes on its shard with no exchange, and the only collective
on the data path is the final gather (NCCL over NVLink on GPUs, gloo in the
CPU tests). Shards may be uneven: rank r owns rows [r*n//W, (r+1)*n//W).
"""
from __future__ import annotations

import datetime
import os
from typing import Callable, Sequence

import torch
import torch.distributed as dist


def init(backend: str | None = None, timeout_s: float = 600.0) -> tuple[int, int]:
    """Join the process group described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT. Returns (rank, world)."""
    if not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group(backend, timeout=datetime.timedelta(seconds=timeout_s))
    return dist.get_rank(), dist.get_world_size()


def rank_world() -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def shard_range(n: int, rank: int, world: int) -> tuple[int, int]:
    """Half-open row range of `rank` when n rows are split over `world` ranks."""
    return rank * n // world, (rank + 1) * n // world


class ShardedTensor:
    """This rank's shard of a tensor split along `dim` (None = replicated)."""

    def __init__(self, local: torch.Tensor, dim: int | None, global_shape: Sequence[int]):
        self.local, self.dim, self.global_shape = local, dim, tuple(global_shape)

    @property
    def shape(self):
        return self.global_shape

    def __matmul__(self, other: "ShardedTensor") -> "ShardedTensor":
        # 1-D sharded matmul as in the reference (sharded_tensor.py:49-67): one side replicated, the other split
        # by rows (dim 0 of the left operand) or by columns (last dim of the right operand); no communication.
        if self.dim == 0 and other.dim is None:
            out = self.local @ other.local
            return ShardedTensor(out, 0, (self.global_shape[0], other.global_shape[-1]))
        if self.dim is None and other.dim == other.local.dim() - 1:
            out = self.local @ other.local
            return ShardedTensor(out, out.dim() - 1, tuple(self.global_shape[:-1]) + (other.global_shape[-1],))
        raise ValueError("sharded matmul needs one replicated operand and one split by rows (left) or columns (right)")


def shard_tensor(x: torch.Tensor, dim: int | None = 0) -> ShardedTensor:
    """Keep this rank's slice of a tensor every rank holds in full (`dim=None` keeps it replicated)."""
    rank, world = rank_world()
    if dim is None:
        return ShardedTensor(x, None, x.shape)
    dim = dim + x.dim() if dim < 0 else dim
    lo, hi = shard_range(x.shape[dim], rank, world)
    return ShardedTensor(x.narrow(dim, lo, hi - lo), dim, x.shape)


def unshard_tensor(st: ShardedTensor) -> torch.Tensor:
    """The final gather: every rank receives the whole tensor (one all-gather; uneven shards are padded)."""
    rank, world = rank_world()
    if st.dim is None or world == 1:
        return st.local
    n = st.global_shape[st.dim]
    sizes = [shard_range(n, r, world)[1] - shard_range(n, r, world)[0] for r in range(world)]
    biggest = max(sizes)
    loc = st.local.movedim(st.dim, 0).contiguous()
    if loc.shape[0] < biggest:
        pad = torch.zeros((biggest - loc.shape[0],) + tuple(loc.shape[1:]), dtype=loc.dtype, device=loc.device)
        loc = torch.cat([loc, pad], 0)
    bufs = [torch.empty_like(loc) for _ in range(world)]
    dist.all_gather(bufs, loc)
    full = torch.cat([b[:s] for b, s in zip(bufs, sizes)], 0)
    return full.movedim(0, st.dim).contiguous()


def all_reduce(t: torch.Tensor, op: str = "sum") -> torch.Tensor:
    """In-place all-reduce ("sum", "avg", "max"); needed only when a REDUCED axis is what was sharded."""
    rank, world = rank_world()
    if world == 1:
        return t
    if op == "max":
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    else:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        if op == "avg":
            t /= world
    return t


def pmap(f: Callable, argnum_opts: Sequence[int | None], gather: bool = True) -> Callable:
    """Data-parallel map: argument i is split along `argnum_opts[i]` (None = replicated), `f` runs on this
    rank's shards, the outputs are taken as split along dim 0 and, with `gather`, gathered on every rank."""
    def wrapped(*args):
        if len(args) != len(argnum_opts):
            raise ValueError("pmap: one sharding option per argument is required")
        local = [a if d is None else shard_tensor(a, d).local for a, d in zip(args, argnum_opts)]
        out = f(*local)
        outs = out if isinstance(out, (tuple, list)) else (out,)
        rank, world = rank_world()
        n_batch = next((a.shape[d] for a, d in zip(args, argnum_opts) if d is not None), None)
        res = []
        for o in outs:
            gshape = (n_batch,) + tuple(o.shape[1:]) if n_batch is not None else tuple(o.shape)
            st = ShardedTensor(o, 0 if n_batch is not None else None, gshape)
            res.append(unshard_tensor(st) if gather else st)
        return res[0] if not isinstance(out, (tuple, list)) else tuple(res)
    return wrapped
