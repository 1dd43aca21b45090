"""Shared test helpers: seeded inputs, the eager-chain oracle, tolerances."""
from __future__ import annotations

import numpy as np

import oracle

# program op name -> how the CPU oracle evaluates it (one reference CPU kernel per op,
# as the eager path does: csrc/cpu/binary.cpp, unary.cpp, ternary.cpp)
_BIN = {"ADD": "add", "MUL": "mul", "MAX": "max", "SUB": "sub", "DIV": "div", "GT": "gt", "LT": "lt", "EQ": "eq",
        "POW": "pow", "LTE": "le", "NEQ": "neq", "GTE": "ge"}


def ref_test_inputs(shapes, dtype=np.float32):
    """The reference's own test inputs: seed 1337, uniform[0.5, 0.9) (tests/test_ops.py:32-41)."""
    np.random.seed(1337)
    if np.issubdtype(dtype, np.floating):
        return [np.random.uniform(low=0.5, high=0.9, size=s).astype(dtype) for s in shapes]
    return [np.random.randint(1, 4, size=s).astype(dtype) for s in shapes]


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


def assert_close(got, want, rtol, atol=None, what=""):
    """rtol/atol comparison as the reference's tests do (assert_allclose(rtol=tol, atol=tol)),
    treating equal infinities as equal."""
    got, want = np.asarray(got), np.asarray(want)
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    atol = rtol if atol is None else atol
    both_inf = np.isinf(got) & np.isinf(want) & (np.sign(got) == np.sign(want))
    g = np.where(both_inf, 0, got).astype(np.float64)
    w = np.where(both_inf, 0, want).astype(np.float64)
    err = np.abs(g - w)
    bound = atol + rtol * np.abs(w)
    bad = ~(err <= bound)
    if bad.any():
        i = np.unravel_index(np.argmax(np.where(bad, err - bound, -np.inf)), got.shape)
        raise AssertionError(f"{what}: {bad.sum()} of {got.size} outside rtol={rtol} atol={atol}; worst at {i}: got {got[i]!r} want {want[i]!r}")
