"""Shared test helpers: seeded inputs, the eager-chain oracle, tolerances."""
from __future__ import annotations

import numpy as np

import oracle

from oracle.chain import eval_program, fused_reduce_oracle  # noqa: F401


def ref_test_inputs(shapes, dtype=np.float32):
    """The reference's own test inputs: seed 1337, uniform[0.5, 0.9) (tests/test_ops.py:32-41)."""
    np.random.seed(1337)
    if np.issubdtype(dtype, np.floating):
        return [np.random.uniform(low=0.5, high=0.9, size=s).astype(dtype) for s in shapes]
    return [np.random.randint(1, 4, size=s).astype(dtype) for s in shapes]


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
