"""Generates tests/golden/ref_cpu_vectors.npz.

Run in a container that has the reference checkout (it needs
oracle/_ref/libpgref.so, i.e. the reference's own CPU templates compiled from
their sources):  python tests/golden/make_golden.py

Vectors (inputs are regenerated from the seed at test time, only outputs are stored):
  * reducers / binary ops / where on the reference's own test cases
    (tests/test_ops.py:106-138, 160-194, 276-300: seed 1337, uniform[0.5,0.9)
    or randint(1,4)), computed by the REFERENCE CPU templates;
  * the same on permuted and broadcast views (what the fused kernels receive);
  * the README fusion formula (README.md:59-63) on a [50,20,100] slice-sized case,
    evaluated as the reference CPU backend's eager chain;
  * softmax / layer_norm / gelu on the reference's composite-test shapes
    (tests/test_high_level_ops.py:100-121, 354-367, 529-544), computed by torch
    CPU — the oracle the reference's tests themselves use.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import oracle  # noqa: E402
from helpers import fused_reduce_oracle, ref_test_inputs  # noqa: E402

REDUCE_SHAPES = [(2, 3), (3, 4), (4, 5)]
REDUCE_AXES = [(0, 1), (1, 0), (0,), (1,), (-1,), (-1, -2), None]
BINARY = ["add", "mul", "sub", "div", "pow", "gt", "lt", "neq", "max"]
VIEW_CASES = {  # name -> (base shape, permutation)
    "perm102": ((3, 4, 5), (1, 0, 2)),
    "perm021": ((6, 4, 5), (0, 2, 1)),
    "perm210": ((3, 4, 5), (2, 1, 0)),
}


def main():
    if not oracle.have_ref():
        raise SystemExit("oracle/_ref/libpgref.so is missing: run oracle/build.py where the reference checkout is present")
    out = {}
    for dt_name, dt in (("f32", np.float32), ("f64", np.float64), ("i32", np.int32)):
        for shape in REDUCE_SHAPES:
            (x,) = ref_test_inputs([shape], dt)
            s = "x".join(map(str, shape))
            for op in ("sum", "mean", "max"):
                for ai, axes in enumerate(REDUCE_AXES):
                    for kd in (0, 1):
                        out[f"reduce/{op}/{dt_name}/{s}/a{ai}/k{kd}"] = oracle.reduce(x, op, axes, bool(kd), impl="ref")
            a, b = ref_test_inputs([shape, shape], dt)
            for op in BINARY:
                if dt == np.int32 and op in ("div", "pow"):
                    continue
                out[f"binary/{op}/{dt_name}/{s}"] = oracle.binary(op, a, b, impl="ref")
            c, a, b = ref_test_inputs([shape, shape, shape], dt)
            out[f"where/{dt_name}/{s}"] = oracle.where((c > 0.7).astype(dt) if dt != np.int32 else (c > 2).astype(dt), a, b, impl="ref")
    for name, (shape, perm) in VIEW_CASES.items():
        (x,) = ref_test_inputs([shape], np.float32)
        v = x.transpose(perm)
        for op in ("sum", "mean", "max"):
            for ax in range(3):
                out[f"view/{name}/{op}/ax{ax}"] = oracle.reduce(v, op, [ax], False, impl="ref")
        (y,) = ref_test_inputs([(v.shape[0], 1, v.shape[2])], np.float32)
        out[f"view/{name}/add_bcast"] = oracle.binary("add", v, y, impl="ref")
    # README fusion formula, reference CPU eager chain
    rng = np.random.default_rng(1)
    x = rng.random((50, 20, 100), dtype=np.float32)
    y = rng.random((50, 100, 20), dtype=np.float32)
    pro = [("LOAD", 0), ("IMM", 0, 0, 0, 2.0), ("ADD", 0, 1), ("LOAD", 1), ("ADD", 2, 3)]
    epi = [("ACC",), ("IMM", 0, 0, 0, 3.0), ("MUL", 0, 1)]
    out["readme_fusion/50x20x100"] = fused_reduce_oracle([x.transpose(0, 2, 1), y], "sum", [2], False, pro, epi, impl="ref")

    # composites: torch CPU, as the reference's tests do
    import torch
    import torch.nn.functional as F
    for shape, ns in [((2, 3, 4), (4,)), ((2, 3, 4), (3, 4)), ((5, 10), (10,)), ((4, 768), (768,))]:
        (x,) = ref_test_inputs([shape], np.float32)
        s = "x".join(map(str, shape))
        out[f"layer_norm/{s}/n{len(ns)}"] = F.layer_norm(torch.from_numpy(x), ns, eps=1e-5).numpy()
    for shape in [(2, 3), (8, 1024)]:
        (x,) = ref_test_inputs([shape], np.float32)
        out["softmax/" + "x".join(map(str, shape))] = torch.softmax(torch.from_numpy(x), -1).numpy()
    (x,) = ref_test_inputs([(2, 3)], np.float32)
    out["gelu_tanh/2x3"] = F.gelu(torch.from_numpy(x), approximate="tanh").numpy()
    np.savez_compressed(Path(__file__).with_name("ref_cpu_vectors.npz"), **out)
    print(f"wrote {len(out)} vectors")


if __name__ == "__main__":
    main()
