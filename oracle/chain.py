"""TEST INFRASTRUCTURE — the reference CPU backend's EAGER CHAIN for a fused region.

A fused kernel of the product replaces a chain of separate reference kernels;
this module evaluates the same chain op by op with the oracle's CPU kernels
(one strided binary / unary / where kernel per instruction, then one reduce
pass per axis, csrc/cpu/binary.cpp, unary.cpp, ternary.cpp, reduce.cpp:24-37).
"""
from __future__ import annotations

import numpy as np

import oracle

# program op name -> how the CPU oracle evaluates it (one reference CPU kernel per op,
# as the eager path does: csrc/cpu/binary.cpp, unary.cpp, ternary.cpp)
_BIN = {"ADD": "add", "MUL": "mul", "MAX": "max", "SUB": "sub", "DIV": "div", "GT": "gt", "LT": "lt", "EQ": "eq",
        "POW": "pow", "LTE": "le", "NEQ": "neq", "GTE": "ge"}


def eval_program(prog, inputs, acc=None, impl="port"):
    """Evaluate a pgb program on numpy arrays with the oracle's eager kernels.
    Returns the list of all values."""
    dtype = inputs[0].dtype if inputs else acc.dtype
    shape = np.broadcast_shapes(*[i.shape for i in inputs]) if inputs else acc.shape
    if acc is not None:
        shape = np.broadcast_shapes(shape, acc.shape)
    vals = []
    for ins in prog:
        ins = tuple(ins) + (0,) * (5 - len(ins))
        op, a, b, c, imm = ins
        if op == "LOAD":
            v = inputs[a]
        elif op == "IMM":
            v = np.broadcast_to(np.array(imm, dtype=dtype), shape)
        elif op == "ACC":
            v = acc
        elif op in ("EXP", "LOG"):
            v = oracle.unary(op.lower(), np.ascontiguousarray(vals[a]))
        elif op == "CAST_I32":
            v = vals[a].astype(np.int32).astype(dtype)  # C truncation, csrc/cpu/view_helpers.hpp:33-55
        elif op == "CAST_F16":
            v = vals[a].astype(np.float16).astype(dtype)
        elif op == "CAST_F32":
            v = vals[a].astype(np.float32).astype(dtype)
        elif op == "SIN":
            v = np.sin(vals[a])
        elif op == "COS":
            v = np.cos(vals[a])
        elif op in _BIN:
            v = oracle.binary(_BIN[op], vals[a], vals[b], impl=impl)
        elif op == "WHERE":
            v = oracle.where(vals[a], vals[b], vals[c], impl=impl)
        else:
            raise ValueError(op)
        vals.append(v)
    return vals


def fused_reduce_oracle(inputs, op, axes, keepdims, prologue=(), epilogue=(), impl="port"):
    """The eager chain the reference runs for a fused region: prologue kernels,
    per-axis reduce passes, epilogue kernels."""
    x = eval_program(prologue, inputs, impl=impl)[-1] if prologue else inputs[0]
    if op == "argmax":
        (ax,) = axes
        r = oracle.argmax(np.asarray(x), ax)
        if keepdims:
            r = np.expand_dims(r, ax)
        return r
    r = oracle.reduce(np.asarray(x), op, list(axes), keepdims, impl=impl)
    if epilogue:
        r = eval_program(epilogue, [], acc=r, impl=impl)[-1]
    return np.asarray(r)


def fused_reduce_truth(inputs, op, axes, keepdims, prologue=(), impl="port"):
    """fp64-accumulating twin of a sum / mean: the prologue is evaluated by the same
    fp32 eager kernels, the accumulation is exact to fp64. A long fp32 serial sum
    (what the reference CPU path does) drifts by more than 1e-5 relative, so this
    is the ground truth the 1e-5 bound is checked against; the reference's own
    distance from it is reported by `reference_sum_error`."""
    x = eval_program(prologue, inputs, impl=impl)[-1] if prologue else inputs[0]
    x64 = np.asarray(x, dtype=np.float64)
    ax = tuple(a % x64.ndim for a in axes)
    r = x64.sum(axis=ax, keepdims=keepdims)
    if op == "mean":
        r = r / np.prod([x64.shape[a] for a in ax])
    return r


def reference_sum_error(inputs, op, axes, prologue=(), impl="port"):
    """max relative distance of the reference's fp32 serial sum from the fp64 truth."""
    ref = fused_reduce_oracle(inputs, op, axes, False, prologue, impl=impl).astype(np.float64)
    tru = fused_reduce_truth(inputs, op, axes, False, prologue, impl=impl)
    return float(np.max(np.abs(ref - tru) / np.maximum(np.abs(tru), 1e-30)))
