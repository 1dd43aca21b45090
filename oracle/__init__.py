"""TEST INFRASTRUCTURE — numpy front-end of the CPU oracle.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs import
this package; the product never does.

`impl="port"` calls the C restatement (oracle/pgoracle.c); `impl="ref"` calls
the reference's own CPU templates (oracle/_ref/libpgref.so) where that library
has been built. numpy arrays carry byte strides, so permuted / broadcast views
are passed exactly as the reference's `View` would describe them.

The functions mirror the reference's eager CPU dispatch:
  reduce      Sum/MaxReduce/Mean::dispatch_cpu, csrc/cpu/reduce.cpp:11-46
              (multi-axis = one single-axis pass per axis, in the given order)
  binary      DEF_BINARY_OP dispatch_cpu, csrc/cpu/binary.cpp:8-39, after the
              explicit broadcast of csrc/ops.cpp:74-79
  where       Where::dispatch_cpu, csrc/cpu/ternary.cpp:6-24
  unary       Exp/Log::dispatch_cpu, csrc/cpu/unary.cpp:14-18
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_DT = {np.dtype(np.int32): 0, np.dtype(np.float32): 2, np.dtype(np.float64): 3}
REDUCE_OPS = {"sum": 0, "max": 1, "mean": 2}
BINARY_OPS = {"add": 0, "sub": 1, "mul": 2, "div": 3, "gt": 4, "lt": 5, "eq": 6, "neq": 7, "ge": 8, "le": 9, "pow": 10, "max": 11}

_libs: dict = {}


def have_ref() -> bool:
    return (HERE / "_ref" / "libpgref.so").exists()


def _lib(impl: str) -> C.CDLL:
    if impl in _libs:
        return _libs[impl]
    path = HERE / "libpgoracle.so" if impl == "port" else HERE / "_ref" / "libpgref.so"
    if not path.exists():
        from . import build as _b
        _b.build()
    if not path.exists():
        raise RuntimeError(f"oracle library {path} is not built")
    L = C.CDLL(str(path))
    _libs[impl] = L
    return L


def _i64(v):
    return (C.c_int64 * max(len(v), 1))(*[int(x) for x in v])


def _p(a: np.ndarray):
    return C.c_void_p(a.ctypes.data)


def reduce_axis(x: np.ndarray, op: str, axis: int, impl: str = "port") -> np.ndarray:
    """One pass of the reference's reduce: contiguous output, `axis` kept with extent 1."""
    axis = axis + x.ndim if axis < 0 else axis
    shape = list(x.shape)
    out_shape = shape.copy()
    out_shape[axis] = 1
    out = np.empty(out_shape, dtype=x.dtype)
    rc = _lib(impl).orc_reduce_axis(_p(x), _p(out), _i64(x.strides), _i64(shape), x.ndim, axis, REDUCE_OPS[op], _DT[x.dtype])
    if rc != 0:
        raise RuntimeError(f"reduce_cpu not implemented for {x.dtype}")
    return out


def reduce(x: np.ndarray, op: str, axes, keepdims: bool = False, impl: str = "port") -> np.ndarray:
    if axes is None:
        axes = list(range(x.ndim))
    if isinstance(axes, int):
        axes = [axes]
    cur = x
    for a in axes:
        cur = reduce_axis(cur, op, a, impl)
    if not keepdims:
        nd = x.ndim
        cur = cur.reshape([s for i, s in enumerate(cur.shape) if i not in {(a + nd) % nd for a in axes}])
    return cur


def binary(op: str, a: np.ndarray, b: np.ndarray, impl: str = "port") -> np.ndarray:
    shape = np.broadcast_shapes(a.shape, b.shape)
    a, b = np.broadcast_to(a, shape), np.broadcast_to(b, shape)
    if a.dtype != b.dtype:
        raise ValueError("binary ops need equal dtypes")
    out = np.empty(shape, dtype=a.dtype)
    rc = _lib(impl).orc_binary(_p(a), _p(b), _p(out), _i64(a.strides), _i64(b.strides), _i64(out.strides), _i64(shape), len(shape),
                               BINARY_OPS[op], _DT[a.dtype])
    if rc != 0:
        raise RuntimeError(f"binary op not implemented for {a.dtype}")
    return out


def where(c: np.ndarray, a: np.ndarray, b: np.ndarray, impl: str = "port") -> np.ndarray:
    shape = np.broadcast_shapes(c.shape, a.shape, b.shape)
    c, a, b = (np.broadcast_to(t, shape) for t in (c, a, b))
    out = np.empty(shape, dtype=a.dtype)
    rc = _lib(impl).orc_where(_p(c), _p(a), _p(b), _p(out), _i64(c.strides), _i64(a.strides), _i64(b.strides), _i64(out.strides),
                              _i64(shape), len(shape), _DT[a.dtype])
    if rc != 0:
        raise RuntimeError(f"where_cpu not implemented for {a.dtype}")
    return out


def unary(op: str, x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    rc = _lib("port").orc_unary(_p(x), _p(out), C.c_int64(x.size), 0 if op == "exp" else 1, _DT[x.dtype])
    if rc != 0:
        raise RuntimeError(f"{op} not implemented for {x.dtype}")
    return out


def matmul_i32(a: np.ndarray, b: np.ndarray, impl: str = "port") -> np.ndarray:
    a, b = np.ascontiguousarray(a, np.int32), np.ascontiguousarray(b, np.int32)
    M, K = a.shape
    N = b.shape[1]
    out = np.empty((M, N), np.int32)
    _lib(impl).orc_matmul_i32(_p(a), _p(b), _p(out), C.c_int64(M), C.c_int64(N), C.c_int64(K), C.c_int64(1))
    return out


def matmul_f32(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a, b = np.ascontiguousarray(a, np.float32), np.ascontiguousarray(b, np.float32)
    M, K = a.shape
    N = b.shape[1]
    out = np.empty((M, N), np.float32)
    _lib("port").orc_matmul_f32(_p(a), _p(b), _p(out), C.c_int64(M), C.c_int64(N), C.c_int64(K), C.c_int64(1))
    return out


def argmax(x: np.ndarray, axis: int) -> np.ndarray:
    assert x.dtype == np.float32
    axis = axis + x.ndim if axis < 0 else axis
    out_shape = [s for i, s in enumerate(x.shape) if i != axis]
    out = np.empty(out_shape, np.int32)
    _lib("port").orc_argmax_f32(_p(x), _p(out), _i64(x.strides), _i64(x.shape), x.ndim, axis)
    return out


# --- int8 quantised linear --------------------------------------------------
def absmax(x: np.ndarray) -> float:
    x = np.ascontiguousarray(x, np.float32)
    f = _lib("port").orc_absmax_f32
    f.restype = C.c_float
    return float(f(_p(x), C.c_int64(x.size)))


def quant_scale(amax: float) -> np.float32:
    return np.float32(max(np.float32(amax), np.float32(1e-6))) / np.float32(127)


def quantize_i8(x: np.ndarray, scale) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    q = np.empty(x.shape, np.int8)
    _lib("port").orc_quantize_i8(_p(x), _p(q), C.c_int64(x.size), C.c_float(float(scale)))
    return q


def quantize_weight_per_channel(w: np.ndarray):
    """w: [K, N] fp32 (the reference's Linear layout, pequegrad/modules.py:221-225).
    Returns (wq [N, K] int8, scale [N] fp32)."""
    wt = np.ascontiguousarray(w.T, np.float32)
    amax = np.maximum(np.abs(wt).max(axis=1), np.float32(1e-6)).astype(np.float32)
    scale = (amax / np.float32(127)).astype(np.float32)
    q = np.clip(np.rint(wt / scale[:, None]), -127, 127).astype(np.int8)
    return q, scale


def gemm_i8(a: np.ndarray, w: np.ndarray) -> np.ndarray:
    a, w = np.ascontiguousarray(a, np.int8), np.ascontiguousarray(w, np.int8)
    M, K = a.shape
    N = w.shape[0]
    acc = np.empty((M, N), np.int32)
    _lib("port").orc_gemm_i8(_p(a), _p(w), _p(acc), C.c_int64(M), C.c_int64(N), C.c_int64(K))
    return acc


def dequant_bias_act(acc: np.ndarray, w_scale: np.ndarray, a_scale, bias, relu: bool) -> np.ndarray:
    acc = np.ascontiguousarray(acc, np.int32)
    w_scale = np.ascontiguousarray(w_scale, np.float32)
    M, N = acc.shape
    out = np.empty((M, N), np.float32)
    b = np.ascontiguousarray(bias, np.float32) if bias is not None else None
    _lib("port").orc_dequant_bias_act(_p(acc), _p(w_scale), C.c_float(float(a_scale)), _p(b) if b is not None else None,
                                      1 if relu else 0, _p(out), C.c_int64(M), C.c_int64(N))
    return out


# --- row composites -----------------------------------------------------------
def softmax_rows(x: np.ndarray, causal: bool = False) -> np.ndarray:
    x32 = np.ascontiguousarray(x, np.float32)
    C_ = x32.shape[-1]
    rows = x32.size // C_
    y = np.empty_like(x32)
    _lib("port").orc_softmax_rows_f32(_p(x32), _p(y), C.c_int64(rows), C.c_int64(C_), C.c_int64(x32.shape[-2] if causal else 0))
    return y


def layernorm_rows(x: np.ndarray, gamma, beta, eps: float = 1e-5) -> np.ndarray:
    x32 = np.ascontiguousarray(x, np.float32)
    C_ = x32.shape[-1]
    rows = x32.size // C_
    y = np.empty_like(x32)
    g = np.ascontiguousarray(gamma, np.float32) if gamma is not None else None
    b = np.ascontiguousarray(beta, np.float32) if beta is not None else None
    _lib("port").orc_layernorm_rows_f32(_p(x32), _p(g) if g is not None else None, _p(b) if b is not None else None, C.c_float(eps), _p(y),
                                        C.c_int64(rows), C.c_int64(C_))
    return y
