"""TEST INFRASTRUCTURE — the reference's own CUDA kernels as a second oracle and GPU comparator.

Front-end of oracle/_ref_cuda/libpgrefcuda.so (the reference's csrc/cuda reduce / binary / exp /
where kernels and the generated kernel its README prints, compiled from its checkout by
oracle/build.py). torch CUDA tensors serve as device memory; every function launches exactly the
reference's kernel with the reference's launch geometry and nothing else. The eager chain
`eager_reduce_chain` is what the reference runs for `exp(reduce(x * a + b))`: one kernel per
primitive with the scalars as broadcast 4-byte buffers (csrc/ops.cpp:74-89).

Only tests/ and bench.py's comparator leg import this module; the product never does.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "_ref_cuda" / "libpgrefcuda.so"
_lib = None
REDUCE_OPS = {"sum": 0, "max": 1, "mean": 2}
BINARY_OPS = {"add": 0, "mul": 1, "max": 2}


def available() -> bool:
    return LIB_PATH.exists()


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not available():
            raise RuntimeError(f"{LIB_PATH} is not built (it needs a reference checkout at build time)")
        _lib = C.CDLL(str(LIB_PATH))
    return _lib


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _meta(vals, device):
    """A device array of 64-bit values (the reference's size_t / long metadata arrays)."""
    return torch.tensor([int(v) for v in vals] or [0], dtype=torch.int64, device=device)


def _p(t: torch.Tensor):
    return C.c_void_p(t.data_ptr())


class Reduce:
    """`Sum/MaxReduce/Mean::dispatch_cuda` (csrc/cuda/reduce.cu:11-125) of a float32 view, metadata uploaded once."""

    def __init__(self, x: torch.Tensor, op: str, axes):
        assert x.dtype == torch.float32 and x.is_cuda
        nd = x.dim()
        self.axes = [a + nd if a < 0 else a for a in axes]
        self.x, self.op = x, REDUCE_OPS[op]
        self.strides = _meta([s * 4 for s in x.stride()], x.device)
        self.shape = _meta(x.shape, x.device)
        self.d_axes = _meta(self.axes, x.device)
        out_shape = [s for i, s in enumerate(x.shape) if i not in self.axes]
        self.out = torch.empty(out_shape, dtype=torch.float32, device=x.device)
        self.red = 1
        for a in self.axes:
            self.red *= x.shape[a]
        # the kernels index with `int`: the sizes they can address are limited
        assert x.numel() < 2 ** 31 and self.out.numel() < 2 ** 31

    def __call__(self) -> torch.Tensor:
        rc = lib().refcuda_reduce_f32(self.op, _p(self.x), _p(self.out), _p(self.strides), _p(self.shape), self.x.dim(), _p(self.d_axes),
                                      len(self.axes), self.out.numel(), self.red, _stream())
        if rc:
            raise RuntimeError("reference reduce kernel failed to launch")
        return self.out


class Binary:
    """`DEF_BINARY_OP` dispatch (csrc/cuda/binary.cu:51-79): both operands as views of the output's shape."""

    def __init__(self, op: str, a: torch.Tensor, b: torch.Tensor):
        b = b.expand(a.shape)
        self.a, self.b, self.op = a, b, BINARY_OPS[op]
        self.sa = _meta([s * 4 for s in a.stride()], a.device)
        self.sb = _meta([s * 4 for s in b.stride()], a.device)
        self.shape = _meta(a.shape, a.device)
        self.out = torch.empty(a.shape, dtype=torch.float32, device=a.device)
        assert a.numel() * 4 < 2 ** 31  # byte offsets are computed in `int`

    def __call__(self) -> torch.Tensor:
        rc = lib().refcuda_binary_f32(self.op, _p(self.sa), _p(self.sb), _p(self.shape), self.a.dim(), _p(self.a), _p(self.b), _p(self.out),
                                      C.c_long(self.a.numel()), _stream())
        if rc:
            raise RuntimeError("reference binary kernel failed to launch")
        return self.out


def exp_dense(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    out = torch.empty_like(x) if out is None else out
    if lib().refcuda_exp_dense_f32(_p(x), _p(out), C.c_long(x.numel()), _stream()):
        raise RuntimeError("reference exp kernel failed to launch")
    return out


def where(c: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    a, b = a.expand(c.shape), b.expand(c.shape)
    out = torch.empty(c.shape, dtype=torch.float32, device=c.device)
    meta = [_meta([s * 4 for s in t.stride()], c.device) for t in (c, a, b)]
    shape = _meta(c.shape, c.device)
    if lib().refcuda_where_f32(_p(meta[0]), _p(meta[1]), _p(meta[2]), _p(shape), c.dim(), _p(c), _p(a), _p(b), _p(out), C.c_long(c.numel()),
                               _stream()):
        raise RuntimeError("reference where kernel failed to launch")
    return out


class EagerReduceChain:
    """exp(reduce(x * mul + add, axes)) as the reference's eager mode runs it: mult_kernel, add_kernel, the
    reduce kernel, exp_kernel_dense — four launches, two full-size intermediates."""

    def __init__(self, x: torch.Tensor, op: str, axes, mul: float = 1.5, add: float = 0.25, exp: bool = True):
        dev = x.device
        self.m = Binary("mul", x, torch.tensor(mul, dtype=torch.float32, device=dev))
        self.a = Binary("add", self.m.out, torch.tensor(add, dtype=torch.float32, device=dev))
        self.r = Reduce(self.a.out, op, axes)
        self.exp = exp
        self.out = torch.empty_like(self.r.out)

    def __call__(self) -> torch.Tensor:
        self.m()
        self.a()
        self.r()
        return exp_dense(self.r.out, self.out) if self.exp else self.r.out


def readme_kernel(x_buf: torch.Tensor, y: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """The generated kernel of the README fusion case (README.md:93-119): x_buf is the [1000,20,100] buffer,
    y [1000,100,20]; returns sum(permute(x,(0,2,1)) + 2 + y, axis=2) * 3 as [1000,100]."""
    assert tuple(x_buf.shape) == (1000, 20, 100) and tuple(y.shape) == (1000, 100, 20) and x_buf.is_contiguous() and y.is_contiguous()
    out = torch.empty((1000, 100), dtype=torch.float32, device=y.device) if out is None else out
    if lib().refcuda_readme_kernel(_p(x_buf), _p(y), _p(out), _stream()):
        raise RuntimeError("reference README kernel failed to launch")
    return out
