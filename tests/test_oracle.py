"""The CPU oracle against (1) the committed golden vectors made by the
reference's own CPU templates, (2) those templates live where they are built,
(3) torch CPU, the oracle the reference's tests use (tests/test_ops.py:20-80)."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close, fused_reduce_oracle, ref_test_inputs

GOLD = np.load(Path(__file__).parent / "golden" / "ref_cpu_vectors.npz")
REDUCE_SHAPES = [(2, 3), (3, 4), (4, 5)]
REDUCE_AXES = [(0, 1), (1, 0), (0,), (1,), (-1,), (-1, -2), None]
DT = {"f32": np.float32, "f64": np.float64, "i32": np.int32}
IMPLS = ["port"] + (["ref"] if oracle.have_ref() else [])


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("dt", ["f32", "f64", "i32"])
def test_reducers_match_reference_vectors(impl, dt):
    for shape in REDUCE_SHAPES:
        (x,) = ref_test_inputs([shape], DT[dt])
        s = "x".join(map(str, shape))
        for op in ("sum", "mean", "max"):
            for ai, axes in enumerate(REDUCE_AXES):
                for kd in (0, 1):
                    want = GOLD[f"reduce/{op}/{dt}/{s}/a{ai}/k{kd}"]
                    got = oracle.reduce(x, op, axes, bool(kd), impl=impl)
                    assert got.shape == want.shape and np.array_equal(got, want), (op, shape, axes, kd)


@pytest.mark.parametrize("impl", IMPLS)
def test_binary_where_match_reference_vectors(impl):
    for dt in ("f32", "f64", "i32"):
        for shape in REDUCE_SHAPES:
            s = "x".join(map(str, shape))
            a, b = ref_test_inputs([shape, shape], DT[dt])
            for op in ["add", "mul", "sub", "div", "pow", "gt", "lt", "neq", "max"]:
                key = f"binary/{op}/{dt}/{s}"
                if key in GOLD.files:
                    assert np.array_equal(oracle.binary(op, a, b, impl=impl), GOLD[key]), key
            c, a, b = ref_test_inputs([shape, shape, shape], DT[dt])
            cond = (c > 0.7).astype(DT[dt]) if dt != "i32" else (c > 2).astype(DT[dt])
            assert np.array_equal(oracle.where(cond, a, b, impl=impl), GOLD[f"where/{dt}/{s}"])


@pytest.mark.parametrize("impl", IMPLS)
def test_views_match_reference_vectors(impl):
    cases = {"perm102": ((3, 4, 5), (1, 0, 2)), "perm021": ((6, 4, 5), (0, 2, 1)), "perm210": ((3, 4, 5), (2, 1, 0))}
    for name, (shape, perm) in cases.items():
        (x,) = ref_test_inputs([shape], np.float32)
        v = x.transpose(perm)
        for op in ("sum", "mean", "max"):
            for ax in range(3):
                assert np.array_equal(oracle.reduce(v, op, [ax], False, impl=impl), GOLD[f"view/{name}/{op}/ax{ax}"])
        (y,) = ref_test_inputs([(v.shape[0], 1, v.shape[2])], np.float32)
        assert np.array_equal(oracle.binary("add", v, y, impl=impl), GOLD[f"view/{name}/add_bcast"])


def test_readme_fusion_vector():
    rng = np.random.default_rng(1)
    x = rng.random((50, 20, 100), dtype=np.float32)
    y = rng.random((50, 100, 20), dtype=np.float32)
    pro = [("LOAD", 0), ("IMM", 0, 0, 0, 2.0), ("ADD", 0, 1), ("LOAD", 1), ("ADD", 2, 3)]
    epi = [("ACC",), ("IMM", 0, 0, 0, 3.0), ("MUL", 0, 1)]
    got = fused_reduce_oracle([x.transpose(0, 2, 1), y], "sum", [2], False, pro, epi)
    assert np.array_equal(got, GOLD["readme_fusion/50x20x100"])
    # third opinion in fp64
    want = ((x.transpose(0, 2, 1).astype(np.float64) + 2 + y).sum(2) * 3)
    assert_close(got, want, 1e-5)


def test_reducers_against_torch_like_the_reference_tests():
    # tests/test_ops.py:160-194 protocol: seed 1337, uniform[0.5,0.9), tol 1e-5
    for shape in REDUCE_SHAPES:
        (x,) = ref_test_inputs([shape], np.float64)
        for axes in REDUCE_AXES:
            for kd in (False, True):
                t = torch.from_numpy(x)
                dim = list(range(x.ndim)) if axes is None else list(axes)
                assert_close(oracle.reduce(x, "sum", axes, kd), torch.sum(t, dim=dim, keepdim=kd).numpy(), 1e-5)
                assert_close(oracle.reduce(x, "mean", axes, kd), torch.mean(t, dim=dim, keepdim=kd).numpy(), 1e-5)
                assert_close(oracle.reduce(x, "max", axes, kd), torch.amax(t, dim=dim, keepdim=kd).numpy(), 1e-5)


def test_composites_against_torch_vectors():
    # layer_norm: tests/test_high_level_ops.py:100-121 (tol 1e-4 there); softmax :354-367
    for shape, nlast in [((2, 3, 4), 1), ((2, 3, 4), 2), ((5, 10), 1), ((4, 768), 1)]:
        (x,) = ref_test_inputs([shape], np.float32)
        s = "x".join(map(str, shape))
        rows = x.reshape(-1, int(np.prod(shape[-nlast:])))
        got = oracle.layernorm_rows(rows, None, None, 1e-5).reshape(shape)
        assert_close(got, GOLD[f"layer_norm/{s}/n{nlast}"], 1e-4)
    for shape in [(2, 3), (8, 1024)]:
        (x,) = ref_test_inputs([shape], np.float32)
        assert_close(oracle.softmax_rows(x), GOLD["softmax/" + "x".join(map(str, shape))], 1e-5)


def test_softmax_causal_and_argmax_restatements():
    rng = np.random.default_rng(7)
    s = rng.standard_normal((2, 3, 16, 16)).astype(np.float32)
    got = oracle.softmax_rows(s, causal=True)
    mask = np.tril(np.ones((16, 16), bool))
    want = torch.softmax(torch.from_numpy(np.where(mask, s, -np.inf)), -1).numpy()
    assert_close(got, want, 1e-6)
    assert (got[..., ~mask] == 0).all()
    x = rng.standard_normal((5, 7, 9)).astype(np.float32)
    x[0, :, 0] = 3.0  # ties: first index wins
    for ax in range(3):
        assert np.array_equal(oracle.argmax(x.transpose(0, 2, 1), ax), x.transpose(0, 2, 1).argmax(ax))


def test_int8_linear_restatement():
    rng = np.random.default_rng(3)
    W = (rng.standard_normal((64, 48)) * 0.05).astype(np.float32)
    X = rng.random((33, 64), dtype=np.float32)
    b = (rng.standard_normal(48) * 0.05).astype(np.float32)
    wq, ws = oracle.quantize_weight_per_channel(W)
    assert wq.shape == (48, 64) and np.abs(wq).max() == 127
    sx = oracle.quant_scale(oracle.absmax(X))
    xq = oracle.quantize_i8(X, sx)
    assert np.array_equal(xq, np.clip(np.rint(X / sx), -127, 127).astype(np.int8))
    acc = oracle.gemm_i8(xq, wq)
    assert np.array_equal(acc, xq.astype(np.int64) @ wq.astype(np.int64).T)
    # the reference's generic matmul template gives the same int32 accumulators
    assert np.array_equal(acc, oracle.matmul_i32(xq.astype(np.int32), wq.T.astype(np.int32)))
    h = oracle.dequant_bias_act(acc, ws, sx, b, True)
    assert_close(h, np.maximum(X @ W + b, 0), 5e-2, 5e-2)  # quantisation error only
