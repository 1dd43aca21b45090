"""GPU parity of the fused elementwise kernel (binary-broadcast, unary, where,
astype and fused programs) through the C ABI. + - * / comparisons, max and where
are bit-exact against the reference CPU templates; exp/log/pow within rel 1e-5."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close, eval_program, ref_test_inputs
from pequegrad_b200 import kernels as K
from test_reduce_gpu import dev

pytestmark = pytest.mark.gpu
GOLD = np.load(Path(__file__).parent / "golden" / "ref_cpu_vectors.npz")
BIN = {"add": "ADD", "mul": "MUL", "sub": "SUB", "div": "DIV", "pow": "POW", "gt": "GT", "lt": "LT", "neq": "NEQ", "max": "MAX",
       "eq": "EQ", "ge": "GTE", "le": "LTE"}
DT = {"f32": np.float32, "f64": np.float64, "i32": np.int32}


def ew(inputs, prog, **kw):
    shape = np.broadcast_shapes(*[i.shape for i in inputs])
    ins = [dev(np.broadcast_to(i, shape)) for i in inputs]
    return [o.cpu().numpy() for o in K.fused_elementwise(ins, prog, shape=tuple(shape), **kw)]


def test_binary_ops_on_the_reference_test_cases():
    # tests/test_ops.py:106-138 inputs; vectors computed by the reference CPU templates
    for dt in ("f32", "f64", "i32"):
        for shape in [(2, 3), (3, 4), (4, 5)]:
            a, b = ref_test_inputs([shape, shape], DT[dt])
            s = "x".join(map(str, shape))
            for name, op in BIN.items():
                key = f"binary/{name}/{dt}/{s}"
                if key not in GOLD.files:
                    continue
                (got,) = ew([a, b], [("LOAD", 0), ("LOAD", 1), (op, 0, 1)])
                if name == "pow":
                    assert_close(got, GOLD[key], 1e-6)
                else:
                    assert np.array_equal(got, GOLD[key]), key
            c, a, b = ref_test_inputs([shape, shape, shape], DT[dt])
            cond = (c > 0.7).astype(DT[dt]) if dt != "i32" else (c > 2).astype(DT[dt])
            (got,) = ew([cond, a, b], [("LOAD", 0), ("LOAD", 1), ("LOAD", 2), ("WHERE", 0, 1, 2)])
            assert np.array_equal(got, GOLD[f"where/{dt}/{s}"])


@pytest.mark.parametrize("shape", [(1000,), (33, 65), (16, 1024), (7, 9, 256), (4, 6, 8, 128), (3, 1, 5, 2, 64)])
def test_broadcast_permuted_and_sliced_operands(shape):
    rng = np.random.default_rng(21)
    x = rng.standard_normal(shape).astype(np.float32)
    ops = ["add", "sub", "mul", "div", "max", "gt", "le", "eq"]
    # full operand, scalar operand (the reference's Fill + broadcast, csrc/ops.cpp:81-89), row and column vectors
    others = [rng.standard_normal(shape).astype(np.float32), np.float32(1.5) * np.ones((1,) * len(shape), np.float32)]
    if len(shape) >= 2:
        others.append(rng.standard_normal((1,) * (len(shape) - 1) + (shape[-1],)).astype(np.float32))
        others.append(rng.standard_normal(shape[:-1] + (1,)).astype(np.float32))
        others.append(np.ascontiguousarray(rng.standard_normal(shape).astype(np.float32).swapaxes(-1, -2)).swapaxes(-1, -2))
    big = rng.standard_normal([s + 2 for s in shape]).astype(np.float32)
    others.append(big[tuple(slice(1, 1 + s) for s in shape)])
    for y in others:
        for name in ops:
            (got,) = ew([x, y], [("LOAD", 0), ("LOAD", 1), (BIN[name], 0, 1)])
            want = oracle.binary(name, x, np.broadcast_to(y, shape))
            assert np.array_equal(got, want), (shape, name, y.shape, y.strides)


def test_fused_programs_chain_tree_and_multi_output():
    rng = np.random.default_rng(22)
    x = rng.random((64, 512), dtype=np.float32) + 0.5
    y = rng.random((64, 512), dtype=np.float32) + 0.5
    chain = [("LOAD", 0), ("IMM", 0, 0, 0, 1.5), ("MUL", 0, 1), ("LOAD", 1), ("ADD", 2, 3), ("IMM", 0, 0, 0, 0.0), ("MAX", 4, 5)]
    (got,) = ew([x, y], chain)
    assert np.array_equal(got, eval_program(chain, [x, y])[-1])
    heavy = [("LOAD", 0), ("LOG", 0), ("LOAD", 1), ("MUL", 1, 2), ("EXP", 3)]  # x ** y the long way
    (got,) = ew([x, y], heavy)
    assert_close(got, eval_program(heavy, [x, y])[-1], 1e-5)
    tree = [("LOAD", 0), ("LOAD", 1), ("ADD", 0, 1), ("SUB", 0, 1), ("MUL", 2, 3), ("EXP", 3)]
    got = ew([x, y], tree, out_vals=[4, 5], out_dtypes=[torch.float32, torch.float32])
    vals = eval_program(tree, [x, y])
    assert np.array_equal(got[0], vals[4])
    assert_close(got[1], vals[5], 1e-5)
    # round() as the reference composes it: (x + 0.5) -> int32 -> float (pequegrad/ops.py:947-948)
    z = (rng.standard_normal((33, 100)) * 4).astype(np.float32)
    rnd = [("LOAD", 0), ("IMM", 0, 0, 0, 0.5), ("ADD", 0, 1), ("CAST_I32", 2)]
    (got,) = ew([z], rnd)
    assert np.array_equal(got, (z + np.float32(0.5)).astype(np.int32).astype(np.float32))


def test_astype_and_half_precision():
    rng = np.random.default_rng(23)
    x = (rng.standard_normal((40, 256)) * 10).astype(np.float32)
    ident = [("LOAD", 0)]
    (got,) = ew([x], ident, out_dtypes=[torch.int32])
    assert np.array_equal(got, x.astype(np.int32))  # float -> int truncates, csrc/cuda/unary.cuh:104-117
    (got,) = ew([x], ident, out_dtypes=[torch.float16])
    assert np.array_equal(got, x.astype(np.float16))
    (got,) = ew([x], ident, out_dtypes=[torch.float64])
    assert np.array_equal(got, x.astype(np.float64))
    h = x.astype(np.float16)
    (got,) = ew([h], ident, out_dtypes=[torch.float32])
    assert np.array_equal(got, h.astype(np.float32))
    (got,) = ew([h, h], [("LOAD", 0), ("LOAD", 1), ("MUL", 0, 1)])
    assert np.array_equal(got, (h.astype(np.float32) * h.astype(np.float32)).astype(np.float16))
    xi = rng.integers(-9, 9, (50, 30)).astype(np.int32)
    yi = rng.integers(1, 9, (50, 30)).astype(np.int32)
    (got,) = ew([xi, yi], [("LOAD", 0), ("LOAD", 1), ("DIV", 0, 1)])
    assert np.array_equal(got, oracle.binary("div", xi, yi))  # C truncation


def test_large_contiguous_and_errors():
    x = torch.randn(1 << 24, device="cuda")
    (y,) = K.fused_elementwise([x], [("LOAD", 0), ("IMM", 0, 0, 0, 1.5), ("MUL", 0, 1), ("IMM", 0, 0, 0, 0.25), ("ADD", 2, 3)])
    assert torch.equal(y, x * 1.5 + 0.25)
    with pytest.raises(ValueError):
        K.fused_elementwise([x], [("LOAD", 1)])
    with pytest.raises(ValueError):
        K.fused_elementwise([x], [("LOAD", 0)], shape=(5,))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.int32])
@pytest.mark.parametrize("shape,perm", [((70, 130), (1, 0)), ((3, 65, 7, 64), (0, 2, 3, 1)), ((2, 5, 100, 64), (0, 1, 3, 2)),
                                        ((2, 3, 4, 33, 65), (2, 0, 1, 4, 3)), ((1, 129, 1, 63), (3, 2, 1, 0))])
def test_copy_of_a_permuted_view_is_bit_exact(shape, perm, dtype):
    # `as_contiguous` of a transpose: the tiled shared-memory path (input contiguous along another dim than the output)
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(shape, generator=g) * 100).to(dtype).cuda()
    v = x.permute(perm)
    (got,) = K.fused_elementwise([v], [("LOAD", 0)])
    assert got.is_contiguous() and got.shape == v.shape
    assert torch.equal(got, v.contiguous())
    # a sliced, permuted view (the V of an attention head inside a packed qkv buffer)
    if len(shape) == 4:
        w = x[..., : shape[-1] // 2 + 1].permute(perm)
        (got,) = K.fused_elementwise([w], [("LOAD", 0)])
        assert torch.equal(got, w.contiguous())
