"""Batch / row sharding over the GPUs of one box.

The API is the reference's `pequegrad/distrib` and `pmap`
(pequegrad/distrib/sharded_tensor.py:7-95, distrib/__init__.py:4-62,
pequegrad/transforms/distrib.py:31-163):

    shard_tensor(x, num_shards, dim, devices) -> ShardedTensor
    unshard_tensor(x, dim, dev)                -> tensor
    pmap(f, devices, argnum_opts)              -> callable
    all_reduce(tensors, op)                    -> tensor

The reference emulates its devices on one GPU and runs them one after another
in Python. Here the shards are spread over processes, one process per GPU
(`torchrun`, `torch.distributed`): with W processes and S shards (S a multiple
of W) process r owns shards [r*S/W, (r+1)*S/W). W == S is the production
layout (one shard per GPU); W == 1 holds every shard on the one device, which
is what the reference's emulated devices do and what lets the same code run
and be tested on a single GPU. Every rank computes on its own shards with no
exchange; the only collective on the data path is the final gather
(`unshard_tensor`, an NCCL all-gather over NVLink; gloo in the CPU tests),
plus `all_reduce` for callers that shard a reduced quantity (the int8 MLP's
per-tensor activation absmax).
"""
from __future__ import annotations

import datetime
import os
from typing import Callable, List, Sequence

import torch
import torch.distributed as dist


def init(backend: str | None = None, timeout_s: float = 600.0) -> tuple[int, int]:
    """Join the process group described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT. Returns (rank, world)."""
    if not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {}
        if backend == "nccl":
            local = int(os.environ.get("LOCAL_RANK", "0"))
            torch.cuda.set_device(local)
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend, timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return dist.get_rank(), dist.get_world_size()


def rank_world() -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def default_devices(num_shards: int | None = None) -> List[str]:
    """One name per shard. Every process computes on its current CUDA device (or the CPU in the gloo tests);
    the names only say how many shards there are, as the reference's emulated `cuda:i` aliases do."""
    _, world = rank_world()
    n = world if num_shards is None else num_shards
    kind = "cuda" if torch.cuda.is_available() else "cpu"
    return [f"{kind}:{i}" for i in range(n)]


def shard_range(n: int, index: int, num_shards: int) -> tuple[int, int]:
    """Half-open range of shard `index` when n rows are split into `num_shards` (uneven splits allowed)."""
    return index * n // num_shards, (index + 1) * n // num_shards


def local_shards(num_shards: int) -> range:
    """Indices of the shards this process owns."""
    rank, world = rank_world()
    if num_shards % world:
        raise ValueError(f"{num_shards} shards cannot be spread evenly over {world} processes")
    per = num_shards // world
    return range(rank * per, (rank + 1) * per)


class ShardedTensor:
    """A tensor split along `dim` (a one-element list, as in the reference; None = replicated).
    `shards` holds the shards this process owns, in shard order."""

    def __init__(self, shards: List[torch.Tensor], dim: List[int] | None = None, num_shards: int | None = None,
                 shape: Sequence[int] | None = None):
        self.shards = list(shards)
        self.dim = dim
        self.num_shards = num_shards if num_shards is not None else len(self.shards) * rank_world()[1]
        if shape is not None:
            self.shape = list(shape)
        elif dim is None:
            self.shape = list(self.shards[0].shape)
        else:
            # what the reference computes (sharded_tensor.py:12-21), valid when every shard is held locally
            self.shape = [sum(s.shape[i] for s in self.shards) if i in dim else self.shards[0].shape[i]
                          for i in range(self.shards[0].dim())]

    def is_replicated(self) -> bool:
        return self.dim is None

    def _zip(self, other, fn):
        if len(self.shards) != len(other.shards):
            raise ValueError("operands are sharded differently")
        return ShardedTensor([fn(a, b) for a, b in zip(self.shards, other.shards)], self.dim or other.dim, self.num_shards)

    def __add__(self, o): return self._zip(o, lambda a, b: a + b)
    def __sub__(self, o): return self._zip(o, lambda a, b: a - b)
    def __mul__(self, o): return self._zip(o, lambda a, b: a * b)
    def __truediv__(self, o): return self._zip(o, lambda a, b: a / b)
    def __neg__(self): return ShardedTensor([-a for a in self.shards], self.dim, self.num_shards, self.shape)

    def __matmul__(self, other: "ShardedTensor") -> "ShardedTensor":
        # 1-D sharded matmul as in the reference (sharded_tensor.py:49-67): both 2-D, one side replicated; the
        # result is split the way the non-replicated operand is. No communication.
        if len(self.shape) != 2 or len(other.shape) != 2 or self.shape[1] != other.shape[0]:
            raise ValueError(f"sharded matmul needs 2-D operands with matching inner sizes, got {self.shape} and {other.shape}")
        if not (self.is_replicated() or other.is_replicated()):
            raise ValueError("one of the tensors must be replicated")
        dim = other.dim if self.is_replicated() else self.dim
        if dim is not None and ((self.is_replicated() and dim != [1]) or (other.is_replicated() and dim != [0])):
            raise ValueError("the left operand may be split by rows or the right operand by columns, nothing else")
        res = [a @ b for a, b in zip(self.shards, other.shards)]
        return ShardedTensor(res, dim, self.num_shards, [self.shape[0], other.shape[1]])

    def numpy(self):
        if self.dim is None:
            return self.shards[0].cpu().numpy()
        if len(self.dim) != 1:
            raise ValueError("only works for 1D sharded tensors")
        return unshard_tensor(self, self.dim[0]).cpu().numpy()

    def __repr__(self):
        return f"ShardedTensor(shape={self.shape}, dim={self.dim}, num_shards={self.num_shards}, local={len(self.shards)})"


def shard_tensor(x: torch.Tensor, num_shards: int, dim: int | None = 0, devices: Sequence | None = None) -> ShardedTensor:
    """Split a tensor that every process holds in full; each process keeps contiguous copies of its own
    shards (`dim=None`: every shard is the whole tensor). Signature of sharded_tensor.py:74-88."""
    if devices is not None and num_shards != len(devices):
        raise ValueError("num_shards must match the number of devices")
    mine = local_shards(num_shards)
    if dim is None:
        return ShardedTensor([x for _ in mine], None, num_shards, x.shape)
    dim = dim + x.dim() if dim < 0 else dim
    if not 0 <= dim < x.dim():
        raise ValueError(f"cannot shard a {x.dim()}-d tensor along dim {dim}")
    shards = []
    for i in mine:
        lo, hi = shard_range(x.shape[dim], i, num_shards)
        shards.append(x.narrow(dim, lo, hi - lo).contiguous())
    return ShardedTensor(shards, [dim], num_shards, x.shape)


def _gather_rows(local: torch.Tensor, rows_per_rank: List[int]) -> torch.Tensor:
    """All-gather of per-process row blocks (dim 0) into one contiguous tensor on every process."""
    rank, world = rank_world()
    if world == 1:
        return local
    local = local.contiguous()
    if len(set(rows_per_rank)) == 1:
        out = torch.empty((sum(rows_per_rank),) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local)
        return out
    # uneven blocks: pad to the largest, gather, drop the padding
    biggest = max(rows_per_rank)
    padded = torch.zeros((biggest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    padded[:local.shape[0]] = local
    recv = torch.empty((world, biggest) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(recv.view((world * biggest,) + tuple(local.shape[1:])), padded)
    return torch.cat([recv[r, :n] for r, n in enumerate(rows_per_rank)], 0)


def unshard_tensor(x: ShardedTensor, dim: int | None = 0, dev=None) -> torch.Tensor:
    """The final gather (sharded_tensor.py:91-97): every process receives the whole tensor, shards
    concatenated along `dim` (None: the dim it was sharded along). One all-gather; a `dim` other
    than 0 costs one extra copy on the device, because the gather delivers whole row blocks."""
    if x.dim is None:
        return x.shards[0]
    if dim is None:
        dim = x.dim[0]
    nd = x.shards[0].dim()
    dim = dim + nd if dim < 0 else dim
    rank, world = rank_world()
    local = x.shards[0] if len(x.shards) == 1 else torch.cat(x.shards, dim)
    if world == 1:
        return local
    per = x.num_shards // world
    n = x.shape[dim]
    sizes = [shard_range(n, (r + 1) * per - 1, x.num_shards)[1] - shard_range(n, r * per, x.num_shards)[0] for r in range(world)]
    if dim == 0:
        return _gather_rows(local, sizes)
    full = _gather_rows(local.movedim(dim, 0).contiguous(), sizes)
    return full.movedim(0, dim).contiguous()


def reshard_tensor(x: ShardedTensor, dim: int, staging: torch.Tensor | None = None, out: torch.Tensor | None = None,
                   copy_fn: Callable | None = None) -> ShardedTensor:
    """The same tensor split along another dim, by ONE all-to-all: every process sends each peer the part of its
    shard that falls into the peer's new slab (data that is already on the GPUs crosses NVLink once, instead of
    being uploaded from the host a second time). One shard per process, even splits, and the old split dim must be
    dim 0, so that the received blocks line up as the new shard without a copy. `staging` / `out` are optional
    preallocated buffers of the shard's size; `copy_fn(dst, src)` replaces the torch copy that packs the blocks."""
    rank, world = rank_world()
    if x.dim is None or len(x.shards) != 1 or x.num_shards != world:
        raise ValueError("reshard_tensor: needs a tensor split along one dim with one shard per process")
    old = x.dim[0]
    nd = x.shards[0].dim()
    dim = dim + nd if dim < 0 else dim
    if old != 0 or not 0 < dim < nd:
        raise ValueError("reshard_tensor: the tensor must be split along dim 0 and the new dim must be another one")
    local = x.shards[0]
    if x.shape[0] % world or x.shape[dim] % world:
        raise ValueError("reshard_tensor: both dims must divide evenly by the number of processes")
    if world == 1:
        return ShardedTensor([local], [dim], 1, x.shape)
    n_new = x.shape[dim] // world
    blk = list(local.shape)
    blk[dim] = n_new
    if staging is None:
        staging = torch.empty([world] + blk, dtype=local.dtype, device=local.device)
    send = staging.view([world] + blk)
    # block s of the send buffer = this shard's rows, new-dim slab s
    src = local.unflatten(dim, (world, n_new)).movedim(dim, 0)
    if copy_fn is None:
        send.copy_(src)
    else:
        copy_fn(send, src)
    if out is None:
        out = torch.empty([world * blk[0]] + blk[1:], dtype=local.dtype, device=local.device)
    dist.all_to_all_single(out.view(-1), send.view(-1))
    return ShardedTensor([out.view([world * blk[0]] + blk[1:])], [dim], world, x.shape)


class GatherBucket:
    """Several sharded outputs gathered by ONE collective. Kernels write their output slabs into views of
    one flat buffer (`local_view`); `gather()` all-gathers that buffer; `full(i)` is output i assembled
    from every process. An output whose slabs are concatenated along dim 0 is returned as a view of the
    receive buffer (strided across processes, no copy); other dims take one permuting copy. With
    `peer_memory=True` the gather is one launch of the peer-memory kernel (`PeerGroup.allgather`, stream-ordered
    on the caller's stream) instead of a library collective: a fraction of its latency, which is what counts for
    a few megabytes at the end of a step; `peer_note` says which of the two is in use."""

    ALIGN = 256

    def __init__(self, device, async_op: bool = False, peer_memory: bool = False):
        self.device, self.async_op, self.peer_memory = device, async_op, peer_memory
        self.specs, self.nbytes = [], 0
        self.local = self.recv = self.work = self.peers = None
        self.peer_note = "NCCL"

    def add(self, local_shape: Sequence[int], dtype: torch.dtype, dim: int = 0) -> int:
        if self.local is not None:
            raise RuntimeError("GatherBucket: add() after the buffers were allocated")
        n = 1
        for s in local_shape:
            n *= int(s)
        es = torch.empty((), dtype=dtype).element_size()
        self.specs.append((self.nbytes, tuple(int(s) for s in local_shape), dtype, dim))
        self.nbytes += (n * es + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        return len(self.specs) - 1

    def _alloc(self):
        if self.local is None:
            _, world = rank_world()
            self.local = torch.empty(max(self.nbytes, self.ALIGN), dtype=torch.uint8, device=self.device)
            if world > 1 and self.peer_memory:
                # every rank comes here at the same point of its set-up: all of them map one another's buffers, or none
                try:
                    self.peers = PeerGroup(gather_bytes=self.local.numel())
                    self.peer_note = "peer-memory kernel over NVLink (CUDA IPC mappings)"
                except Exception as e:  # noqa: BLE001 - any failure of the mapping leaves the NCCL path
                    self.peer_note = f"NCCL (peer mapping unavailable: {type(e).__name__}: {e})"
                flags = [None] * world
                dist.all_gather_object(flags, self.peers is not None)
                if not all(flags):
                    if self.peers is not None:
                        self.peers.close()
                    self.peers = None
            if self.peers is not None:
                self.recv = self.peers.recv[: world * self.local.numel()]
            else:
                self.recv = self.local if world == 1 else torch.empty(world * self.local.numel(), dtype=torch.uint8, device=self.device)

    def local_view(self, i: int) -> torch.Tensor:
        self._alloc()
        off, shape, dtype, _ = self.specs[i]
        n = 1
        for s in shape:
            n *= s
        es = torch.empty((), dtype=dtype).element_size()
        return self.local[off:off + n * es].view(dtype).view(shape)

    def gather(self):
        """Enqueue the all-gather of everything written to the local views so far (stream-ordered)."""
        self._alloc()
        _, world = rank_world()
        if world > 1 and self.peers is not None:
            self.peers.allgather(self.local)  # lands in self.recv, a view of the group's receive buffer
        elif world > 1:
            self.work = dist.all_gather_into_tensor(self.recv, self.local, async_op=self.async_op)

    def wait(self):
        """Make the current stream wait for an asynchronous gather (no host synchronisation)."""
        if self.work is not None:
            self.work.wait()
            self.work = None

    def full(self, i: int, copy_out: torch.Tensor | None = None, copy_fn: Callable | None = None) -> torch.Tensor:
        """Output i of every process, concatenated along its dim. `copy_fn(dst_view, src_view)` replaces
        the torch copy for the outputs that need one (e.g. by a kernel of this library)."""
        _, world = rank_world()
        off, shape, dtype, dim = self.specs[i]
        if world == 1:
            return self.local_view(i)
        es = torch.empty((), dtype=dtype).element_size()
        n = 1
        for s in shape:
            n *= s
        stride0 = self.local.numel() // es
        base = self.recv.view(dtype)
        # [world, *shape] view of the receive buffer: process r's slab starts r * (bytes per process) further on
        inner, acc = [], 1
        for s in reversed(shape):
            inner.append(acc)
            acc *= s
        v = base.as_strided((world,) + shape, (stride0,) + tuple(reversed(inner)), off // es)
        if not shape:
            return v
        if dim == 0:
            return v  # [world, rows/world, ...]: the gathered tensor, split in two along dim 0
        moved = v.movedim(0, dim)  # [.., world, shape[dim], ..]
        tgt = list(shape)
        tgt[dim] *= world
        if copy_out is None:
            copy_out = torch.empty(tgt, dtype=dtype, device=self.device)
        dst = copy_out.view(moved.shape)
        if copy_fn is None:
            dst.copy_(moved)
        else:
            copy_fn(dst, moved)
        return copy_out


class _DevMem:
    """A raw device allocation seen by torch through the CUDA array interface (no copy)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class PeerGroup:
    """Peer-memory collectives between the processes of one box (one GPU each): the kernels of
    `pgb_peer_allreduce_max_f32` / `pgb_peer_allgather` store straight into the other ranks' memory over
    NVLink and wait for the others' stores, one small launch per exchange, instead of a library collective
    (tens of microseconds each, as long as a whole layer of an 8192-row MLP shard). Set-up maps every rank's
    control block and receive buffer into this process with CUDA IPC; the handles travel through the
    process group's host channel. Only for NCCL groups with one shard per process; every rank must issue
    the same sequence of calls."""

    def __init__(self, gather_bytes: int = 0):
        import ctypes as C

        from . import _lib as L
        self.rank, self.world = rank_world()
        if self.world < 2 or self.world > 16 or not torch.cuda.is_available():
            raise RuntimeError("PeerGroup needs 2 to 16 processes with one GPU each")
        lib = L.lib()
        self._lib, self._C = lib, C
        self.gather_bytes = (int(gather_bytes) + 255) // 256 * 256
        self._own, self._opened = [], []

        def alloc(nbytes):
            p = C.c_void_p()
            L.check(lib.pgb_peer_alloc(nbytes, C.byref(p)))
            self._own.append(p.value)
            h = C.create_string_buffer(64)
            L.check(lib.pgb_peer_export(p, h))
            return p.value, h.raw

        ctrl, h_ctrl = alloc(lib.pgb_peer_ctrl_bytes())
        recv, h_recv = alloc(self.gather_bytes * self.world) if self.gather_bytes else (None, b"")
        handles = [None] * self.world
        dist.all_gather_object(handles, (h_ctrl, h_recv))

        def open_(h):
            p = C.c_void_p()
            L.check(lib.pgb_peer_open(h, C.byref(p)))
            self._opened.append(p.value)
            return p.value

        ctrls = [ctrl if r == self.rank else open_(handles[r][0]) for r in range(self.world)]
        recvs = [recv if r == self.rank else (open_(handles[r][1]) if self.gather_bytes else None) for r in range(self.world)]
        self._ctrl = (C.c_void_p * self.world)(*ctrls)
        self._recv = (C.c_void_p * self.world)(*[r or 0 for r in recvs])
        self.recv = torch.as_tensor(_DevMem(recv, self.gather_bytes * self.world), device="cuda") if self.gather_bytes else None
        dist.barrier()  # every mapping exists before anyone's first kernel stores through one

    def allreduce_max(self, value: torch.Tensor) -> torch.Tensor:
        """`value` (one non-negative float32 on this rank's GPU) becomes the maximum over all ranks, in place."""
        from . import _lib as L
        L.check(self._lib.pgb_peer_allreduce_max_f32(value.data_ptr(), self._ctrl, self.rank, self.world, torch.cuda.current_stream().cuda_stream))
        return value

    def allgather(self, local: torch.Tensor) -> torch.Tensor:
        """Every rank's `local` (same shape everywhere, contiguous) stacked along a new dim 0: a view of this
        rank's receive buffer, valid until the next allgather."""
        from . import _lib as L
        nbytes = local.numel() * local.element_size()
        if nbytes > self.gather_bytes or not local.is_contiguous():
            raise ValueError("PeerGroup.allgather: the slab must be contiguous and fit the receive buffer")
        padded = (nbytes + 15) // 16 * 16
        L.check(self._lib.pgb_peer_allgather(local.data_ptr(), padded, self._recv, self._ctrl, self.rank, self.world,
                                             torch.cuda.current_stream().cuda_stream))
        out = self.recv[: padded * self.world].view(self.world, padded)[:, :nbytes]
        return out.view(local.dtype).view((self.world,) + tuple(local.shape)) if padded == nbytes else \
            out.contiguous().view(local.dtype).view((self.world,) + tuple(local.shape))

    def close(self):
        torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier()  # nobody unmaps while a peer's kernel may still store
        for p in self._opened:
            self._lib.pgb_peer_close(p)
        for p in self._own:
            self._lib.pgb_peer_free(p)
        self._opened, self._own = [], []


def all_reduce(tensors, op: str = "sum") -> torch.Tensor:
    """All-reduce over every shard (distrib/__init__.py:4-29): `tensors` is this process's list of per-shard
    tensors (or a single tensor); each of them ends up holding the result, which is also returned.
    "sum" and "avg" as in the reference; "max" is added for the per-tensor activation absmax."""
    if op not in ("sum", "avg", "max"):
        raise ValueError(f"Unknown op {op}")
    ts = [tensors] if isinstance(tensors, torch.Tensor) else list(tensors)
    if op == "avg" and not ts[0].is_floating_point():
        raise ValueError("all_reduce('avg') needs floating-point tensors")
    _, world = rank_world()
    if len(ts) == 1:
        total = ts[0]  # reduced in place
    else:
        total = ts[0].clone()
        for t in ts[1:]:
            if op == "max":
                torch.maximum(total, t, out=total)
            else:
                total.add_(t)
    if world > 1:
        dist.all_reduce(total, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM)
    n = len(ts) * world
    if op == "avg" and n > 1:
        total.div_(n)
    for t in ts:
        if t is not total:
            t.copy_(total)
    return total


def pmap(f: Callable, devices: Sequence | None, argnum_opts: Sequence[int | None], out_opts="avg") -> Callable:
    """Data-parallel map with the reference's calling convention (transforms/distrib.py:31-67,
    examples/data_parallel_mlp.py:38-57): argument i with `argnum_opts[i] = d` must have
    `shape[d] == len(devices)` and shard k receives `arg.select(d, k)`; `None` replicates the argument.

    Outputs: `out_opts="avg"` averages each output over the shards, which is what the reference does with
    its per-device losses and gradients (transforms/distrib.py:150-157). An int d (or one entry per
    output) instead stacks the per-shard outputs along a new dim d on every process — the final gather of
    an inference workload. "sharded" returns this process's per-shard outputs untouched (no collective).
    `f` must not call collectives itself."""
    num = len(devices) if devices is not None else rank_world()[1]

    def wrapped(*args):
        if len(args) != len(argnum_opts):
            raise ValueError(f"Number of args must match argnum_opts: {len(args)} != {len(argnum_opts)}")
        mine = local_shards(num)
        for a, d in zip(args, argnum_opts):
            if d is not None:
                if not isinstance(a, torch.Tensor):
                    raise ValueError("Only tensors can be split")
                if a.shape[d] != num:
                    raise ValueError(f"Splitting dimension must be equal to the number of devices: {a.shape[d]} != {num}")
        per_shard = [f(*[a if d is None else a.select(d, k) for a, d in zip(args, argnum_opts)]) for k in mine]
        is_seq = isinstance(per_shard[0], (tuple, list))
        n_out = len(per_shard[0]) if is_seq else 1
        outs = [[(p[j] if is_seq else p) for p in per_shard] for j in range(n_out)]
        opts = list(out_opts) if isinstance(out_opts, (tuple, list)) else [out_opts] * n_out
        if len(opts) != n_out:
            raise ValueError("pmap: one out_opts entry per output is required")
        res = []
        for shards, opt in zip(outs, opts):
            if opt == "sharded":
                res.append(shards)
            elif opt == "avg":
                res.append(all_reduce([s.clone() for s in shards], "avg"))
            elif isinstance(opt, int):
                nd = shards[0].dim() + 1
                d = opt + nd if opt < 0 else opt
                if not 0 <= d < nd:
                    raise ValueError(f"pmap: cannot stack {nd - 1}-d outputs along dim {opt}")
                stacked = torch.stack(shards, 0)  # [local shards, ...]
                st = ShardedTensor([stacked], [0], rank_world()[1], [num] + list(shards[0].shape))
                res.append(unshard_tensor(st, 0).movedim(0, d))
            else:
                raise ValueError(f"pmap: unknown out_opts entry {opt!r}")
        return tuple(res) if is_seq else res[0]
    return wrapped
