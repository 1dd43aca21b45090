"""Host-side mirror of the reference's operator interface for the hot path.

A `Tensor` is a lazy graph node, as in the reference (csrc/tensor.hpp:361-429):
ops build nodes and infer shapes, nothing runs until `eval()` / `numpy()`.
  * eager evaluation runs ONE kernel per primitive, like `Tensor::eval`
    dispatching each `ADPrimitive::dispatch_cuda` (csrc/tensor.cpp:176-222);
  * `jit(f)` evaluates through the fuser in `fuser.py`, which plays the role of
    `schedule` + `graph_to_ir` (csrc/compiler/scheduler.cpp:100-257,
    csrc/compiler/ir.cpp:839-1286): an elementwise region with at most one
    reduce becomes a single fused kernel call.
Views (permute, broadcast_to, reshape of contiguous data) never copy: they
change strides, which the kernels take as they are ("the permute is implicit
in the kernel", README.md:125). All device work goes through the C ABI.
"""
from __future__ import annotations

import math
from typing import Sequence

import numpy as np
import torch

from . import _lib as L
from . import kernels as K

float32, float16, float64, int32, bfloat16 = torch.float32, torch.float16, torch.float64, torch.int32, torch.bfloat16
_NP2T = {np.dtype(np.float32): float32, np.dtype(np.float64): float64, np.dtype(np.int32): int32, np.dtype(np.float16): float16}

BINARY = {"add": "ADD", "sub": "SUB", "mul": "MUL", "div": "DIV", "pow": "POW", "max": "MAX", "gt": "GT", "lt": "LT", "eq": "EQ",
          "neq": "NEQ", "ge": "GTE", "le": "LTE"}
UNARY = {"exp": "EXP", "log": "LOG", "sin": "SIN", "cos": "COS"}
REDUCE = {"sum": L.SUM, "max_reduce": L.MAX, "mean": L.MEAN, "argmax": L.ARGMAX}
VIEW_OPS = ("permute", "broadcast_to", "reshape")


def _norm_axes(axes, nd):
    if axes is None:
        return tuple(range(nd))
    if isinstance(axes, int):
        axes = (axes,)
    return tuple(a + nd if a < 0 else a for a in axes)


class Tensor:
    """Lazy tensor node. `op == "leaf"` holds device data in `_buf` (a torch CUDA tensor view)."""

    def __init__(self, data=None, *, op="leaf", args=(), attrs=None, shape=None, dtype=None, device="cuda"):
        self.op, self.args, self.attrs = op, tuple(args), attrs or {}
        self._buf = None
        if op == "leaf":
            if isinstance(data, Tensor):
                data = data.eval()._buf
            if isinstance(data, np.ndarray):
                if data.dtype not in _NP2T:
                    data = data.astype(np.float32)
                data = torch.from_numpy(np.ascontiguousarray(data))
            if not isinstance(data, torch.Tensor):
                data = torch.tensor(data, dtype=torch.float32)
            if not data.is_cuda:
                if not torch.cuda.is_available():
                    raise RuntimeError("pequegrad_b200 tensors live on the GPU: no CUDA device is present and there is no CPU backend")
                data = data.cuda()
            self._buf = data
            shape, dtype = tuple(data.shape), data.dtype
        self.shape, self.dtype = tuple(shape), dtype

    # -- construction helpers -------------------------------------------------
    @staticmethod
    def from_numpy(a):
        return Tensor(a)

    @property
    def ndim(self):
        return len(self.shape)

    dim = ndim

    @property
    def strides(self):
        """Byte strides of the evaluated view, as the reference reports them."""
        t = self.eval()._buf
        return tuple(s * t.element_size() for s in t.stride())

    def to(self, device):
        if not str(device).startswith("cuda"):
            raise RuntimeError("only CUDA devices exist in pequegrad_b200")
        return self

    def is_evaled(self):
        return self._buf is not None

    # -- evaluation -----------------------------------------------------------
    def eval(self, fuse: bool = False):
        if self._buf is None:
            from .fuser import evaluate
            evaluate(self, fuse)
        return self

    def numpy(self):
        return self.eval()._buf.cpu().numpy()

    def torch(self):
        return self.eval()._buf

    # -- operators ------------------------------------------------------------
    def __add__(self, o): return add(self, o)
    def __radd__(self, o): return add(o, self)
    def __sub__(self, o): return sub(self, o)
    def __rsub__(self, o): return sub(o, self)
    def __mul__(self, o): return mul(self, o)
    def __rmul__(self, o): return mul(o, self)
    def __truediv__(self, o): return div(self, o)
    def __rtruediv__(self, o): return div(o, self)
    def __pow__(self, o): return pow(self, o)
    def __neg__(self): return mul(self, -1.0)
    def __gt__(self, o): return gt(self, o)
    def __lt__(self, o): return lt(self, o)
    def __ge__(self, o): return ge(self, o)
    def __le__(self, o): return le(self, o)
    def __eq__(self, o): return eq(self, o)  # noqa: PLW1641 - mirrors the reference, which overloads == elementwise
    def __ne__(self, o): return neq(self, o)
    __hash__ = object.__hash__
    def __matmul__(self, o): return matmul(self, o)

    def sum(self, dim=None, keepdim=False): return sum(self, dim, keepdim)  # noqa: A003
    def mean(self, dim=None, keepdim=False): return mean(self, dim, keepdim)
    def max_reduce(self, dim=None, keepdim=False): return max_reduce(self, dim, keepdim)
    def exp(self): return exp(self)
    def log(self): return log(self)
    def relu(self): return max(self, 0.0)  # max(x, 0), pequegrad/tensor.py:162-163
    def astype(self, dt): return astype(self, dt)
    def permute(self, *dims): return permute(self, dims[0] if len(dims) == 1 and not isinstance(dims[0], int) else dims)
    def reshape(self, *shape): return reshape(self, shape[0] if len(shape) == 1 and not isinstance(shape[0], int) else shape)
    def transpose(self, a, b):
        p = list(range(self.ndim)); p[a], p[b] = p[b], p[a]
        return permute(self, p)


def _as_tensor(x, like: Tensor) -> Tensor:
    """Scalars become 0-d Fill tensors, as in the reference (csrc/ops.cpp:81-89)."""
    if isinstance(x, Tensor):
        return x
    return fill((), like.dtype, float(x))


def fill(shape, dtype, value) -> Tensor:
    return Tensor(op="fill", attrs={"value": float(value)}, shape=tuple(shape), dtype=dtype)


def broadcast_to(x: Tensor, shape) -> Tensor:
    shape = tuple(shape)
    if x.shape == shape:
        return x
    pad = len(shape) - x.ndim
    for i, s in enumerate(x.shape):
        if s != 1 and s != shape[pad + i]:
            raise ValueError(f"cannot broadcast {x.shape} to {shape}")
    return Tensor(op="broadcast_to", args=(x,), attrs={"shape": shape}, shape=shape, dtype=x.dtype)


def _binary(name, a, b) -> Tensor:
    ref = a if isinstance(a, Tensor) else b
    a, b = _as_tensor(a, ref), _as_tensor(b, ref)
    if a.dtype != b.dtype:
        raise ValueError(f"{name}: operand dtypes differ ({a.dtype} and {b.dtype})")
    shape = tuple(np.broadcast_shapes(a.shape, b.shape))
    # both operands are broadcast explicitly before the op, as csrc/ops.cpp:74-79 does
    return Tensor(op=name, args=(broadcast_to(a, shape), broadcast_to(b, shape)), shape=shape, dtype=a.dtype)


def add(a, b): return _binary("add", a, b)
def sub(a, b): return _binary("sub", a, b)
def mul(a, b): return _binary("mul", a, b)
def div(a, b): return _binary("div", a, b)
def pow(a, b): return _binary("pow", a, b)  # noqa: A001
def max(a, b): return _binary("max", a, b)  # noqa: A001
def gt(a, b): return _binary("gt", a, b)
def lt(a, b): return _binary("lt", a, b)
def eq(a, b): return _binary("eq", a, b)
def neq(a, b): return _binary("neq", a, b)
def ge(a, b): return _binary("ge", a, b)
def le(a, b): return _binary("le", a, b)


def _unary(name, x): return Tensor(op=name, args=(x,), shape=x.shape, dtype=x.dtype)
def exp(x): return _unary("exp", x)
def log(x): return _unary("log", x)
def sin(x): return _unary("sin", x)
def cos(x): return _unary("cos", x)


def astype(x: Tensor, dt) -> Tensor:
    return x if x.dtype == dt else Tensor(op="astype", args=(x,), attrs={"dtype": dt}, shape=x.shape, dtype=dt)


def where(c, a, b) -> Tensor:
    ref = a if isinstance(a, Tensor) else (b if isinstance(b, Tensor) else c)
    c, a, b = _as_tensor(c, ref), _as_tensor(a, ref), _as_tensor(b, ref)
    shape = tuple(np.broadcast_shapes(c.shape, a.shape, b.shape))
    return Tensor(op="where", args=tuple(broadcast_to(t, shape) for t in (c, a, b)), shape=shape, dtype=a.dtype)


def _reduce(name, x: Tensor, axes, keepdims) -> Tensor:
    ax = _norm_axes(axes, x.ndim)
    shape = K.reduced_shape(x.shape, ax, keepdims)
    dt = int32 if name == "argmax" else x.dtype
    return Tensor(op=name, args=(x,), attrs={"axes": ax, "keepdims": bool(keepdims)}, shape=shape, dtype=dt)


def sum(x, axes=None, keepdims=False): return _reduce("sum", x, axes, keepdims)  # noqa: A001
def mean(x, axes=None, keepdims=False): return _reduce("mean", x, axes, keepdims)
def max_reduce(x, axes=None, keepdims=False): return _reduce("max_reduce", x, axes, keepdims)


def argmax(x, dim=-1):
    """First index of the maximum along one axis (int32). The reference composes this from max_reduce,
    ==, arange and sum with a float result (pequegrad/ops.py:968-978); here it is one reduce kernel."""
    return _reduce("argmax", x, (dim,), False)


def permute(x: Tensor, dims: Sequence[int]) -> Tensor:
    dims = tuple(d + x.ndim if d < 0 else d for d in dims)
    return Tensor(op="permute", args=(x,), attrs={"dims": dims}, shape=tuple(x.shape[d] for d in dims), dtype=x.dtype)


def reshape(x: Tensor, shape) -> Tensor:
    shape = list(shape)
    if -1 in shape:
        known = -int(np.prod(shape))
        shape[shape.index(-1)] = int(np.prod(x.shape)) // known
    if int(np.prod(shape)) != int(np.prod(x.shape)):
        raise ValueError(f"cannot reshape {x.shape} to {tuple(shape)}")
    return Tensor(op="reshape", args=(x,), attrs={"shape": tuple(shape)}, shape=tuple(shape), dtype=x.dtype)


def matmul(a: Tensor, b: Tensor) -> Tensor:
    if a.ndim < 2 or b.ndim < 2:
        raise ValueError("matmul: operands need at least 2 dims")
    if a.shape[-1] != b.shape[-2]:
        raise ValueError(f"matmul: shapes {a.shape} and {b.shape} do not contract")
    batch = a.shape[:-2] if b.ndim == 2 else tuple(np.broadcast_shapes(a.shape[:-2], b.shape[:-2]))
    return Tensor(op="matmul", args=(a, b), shape=batch + (a.shape[-2], b.shape[-1]), dtype=a.dtype)


def sqrt(x): return x ** 0.5  # pequegrad/ops.py:508-509


def softmax(x: Tensor, dim=-1) -> Tensor:
    """Composite exactly as pequegrad/ops.py:259-267. Under `jit` the fuser recognises the chain (over the last axis)
    in the graph, however it was written, and runs it as the one-kernel row softmax."""
    m = x.max_reduce(dim, keepdim=True)
    e = (x - m).exp()
    return e / e.sum(dim, keepdim=True)


def layer_norm(x: Tensor, normalized_shape, eps=1e-5, weight=None, bias=None) -> Tensor:
    """Composite exactly as pequegrad/ops.py:515-551 (biased variance, eps before the square root). Under `jit` the
    fuser recognises the chain in the graph and runs it as the one-kernel row LayerNorm."""
    ns = (normalized_shape,) if isinstance(normalized_shape, int) else tuple(normalized_shape)
    dims = tuple(range(x.ndim - len(ns), x.ndim))
    mu = x.mean(dims, keepdim=True)
    n = float(np.prod(ns))
    var = ((x - mu) ** 2.0).sum(dims, keepdim=True) / n
    y = (x - mu) / sqrt(var + eps)
    if weight is not None:
        y = y * weight
    if bias is not None:
        y = y + bias
    return y


def tanh(x): return 2.0 / (1.0 + exp(-2.0 * x)) - 1.0  # pequegrad/ops.py:159-164


def gelu(x: Tensor) -> Tensor:
    """tanh approximation, pequegrad/ops.py:109-118."""
    y = 0.5 * x * (1.0 + tanh(math.sqrt(2 / math.pi) * (x + 0.044715 * (x ** 3.0))))
    y.attrs = dict(y.attrs, gelu_of=x)  # lets the fuser fold gelu(x @ w + b) into the GEMM's epilogue
    return y


def scaled_dot_product_attention(query: Tensor, key: Tensor, value: Tensor, mask: Tensor | None = None, is_causal: bool = False) -> Tensor:
    """pequegrad/ops.py:792-818: softmax(q k^T / sqrt(d_k) [masked with -1e9]) v. Under `jit`, 16-bit operands with a head
    dim of 64 and no mask tensor become ONE fused attention kernel (which also takes `is_causal`); the composite itself
    refuses `is_causal` as the reference does ("use a mask")."""
    from . import fuser
    d_k = key.shape[-1]
    if (fuser._fuse_composites and mask is None and d_k == 64 and query.shape[-1] == 64 and value.shape[-1] == 64
            and query.dtype in (torch.float16, torch.bfloat16) and 2 <= query.ndim <= 4 and query.shape[:-2] == key.shape[:-2] == value.shape[:-2]):
        return Tensor(op="attention", args=(query, key, value), attrs={"causal": bool(is_causal), "scale": 1.0 / math.sqrt(d_k)},
                      shape=query.shape, dtype=query.dtype)
    if is_causal:
        raise NotImplementedError("Causal attention not implemented yet, use a mask")
    scores = (query @ key.transpose(-2, -1)) / math.sqrt(d_k)
    if mask is not None:
        scores = where(mask, scores, broadcast_to(fill((), scores.dtype, -1e9), scores.shape))
    return softmax(scores, dim=-1) @ value

