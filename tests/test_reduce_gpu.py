"""GPU parity of the fused reduce kernels, called through the C ABI, against the
CPU oracle (the reference CPU backend's eager chain) on the same seeded inputs.

Tolerances: fp32 sums / means rel 1e-5 (+ the same absolute floor the
reference's tests use); max and argmax bit-exact; fp16 inputs 2e-2.
"""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close, eval_program, fused_reduce_oracle
from oracle.chain import fused_reduce_truth
from pequegrad_b200 import _lib as L
from pequegrad_b200 import kernels as K

pytestmark = pytest.mark.gpu
GOLD = np.load(Path(__file__).parent / "golden" / "ref_cpu_vectors.npz")
OPS = {"sum": L.SUM, "max": L.MAX, "mean": L.MEAN, "argmax": L.ARGMAX}

AFFINE = [("LOAD", 0), ("IMM", 0, 0, 0, 1.5), ("MUL", 0, 1), ("IMM", 0, 0, 0, 0.25), ("ADD", 2, 3)]
EXP_EPI = [("ACC",), ("EXP", 0)]
EXP_PRO = [("LOAD", 0), ("IMM", 0, 0, 0, 0.5), ("MUL", 0, 1), ("EXP", 2)]            # chain with a transcendental
TREE_PRO = [("LOAD", 0), ("IMM", 0, 0, 0, 1.0), ("ADD", 0, 1), ("IMM", 0, 0, 0, 2.0), ("SUB", 0, 3), ("MUL", 2, 4)]  # not a chain


def dev(a):
    """numpy view -> CUDA tensor view with the same strides (storage copied once)."""
    base = a
    while isinstance(base.base, np.ndarray):
        base = base.base
    t = torch.from_numpy(np.ascontiguousarray(base) if not base.flags.c_contiguous else base).cuda()
    if base is a:
        return t
    es = a.itemsize
    off = (a.__array_interface__["data"][0] - base.__array_interface__["data"][0]) // es
    return torch.as_strided(t.view(-1), a.shape, [s // es for s in a.strides], off)


def run_case(inputs, op, axes, keepdims=False, prologue=(), epilogue=(), rtol=1e-5, exact=None, what=""):
    ins = [dev(i) for i in inputs]
    if epilogue and op in ("sum", "mean") and any(i[0] == "EXP" for i in epilogue):
        # exp turns an absolute error of the accumulator into a relative one (and overflows for
        # long sums), so the accumulators are compared first, then the epilogue given them
        pre = K.fused_reduce(ins, OPS[op], axes, keepdims, prologue).cpu().numpy()
        want_pre = fused_reduce_oracle(inputs, op, axes, keepdims, prologue)
        scale = max(1.0, float(np.abs(want_pre).max()))
        assert_close(pre, want_pre, rtol, rtol * scale, what + " (accumulators)")
        got = K.fused_reduce(ins, OPS[op], axes, keepdims, prologue, epilogue).cpu().numpy()
        assert_close(got, eval_program(epilogue, [], acc=pre)[-1], rtol, 0.0, what + " (epilogue)")
        return
    want = fused_reduce_oracle(inputs, op, axes, keepdims, prologue, epilogue)
    got = K.fused_reduce(ins, OPS[op], axes, keepdims, prologue, epilogue).cpu().numpy()
    if exact is None:
        exact = op in ("max", "argmax") and not any(i[0] in ("EXP", "LOG", "POW") for i in list(prologue) + list(epilogue))
    if exact:
        assert got.shape == want.shape and np.array_equal(got, want), f"{what}: not bit-exact"
    else:
        scale = max(1.0, float(np.abs(want[np.isfinite(want)]).max())) if np.isfinite(want).any() else 1.0
        assert_close(got, want, rtol, rtol * scale, what)


def views(rng, shape):
    """contiguous, permuted, broadcast and offset-sliced views of the same logical shape."""
    x = rng.standard_normal(shape).astype(np.float32)
    out = [("contig", x)]
    nd = len(shape)
    if nd >= 2:
        perm = list(range(nd))[::-1]
        base = rng.standard_normal([shape[p] for p in perm]).astype(np.float32)
        out.append(("reversed", base.transpose(np.argsort(perm))))
    if nd == 3:
        base = rng.standard_normal((shape[0], shape[2], shape[1])).astype(np.float32)
        out.append(("perm021", base.transpose(0, 2, 1)))
        out.append(("bcast1", np.broadcast_to(rng.standard_normal((shape[0], 1, shape[2])).astype(np.float32), shape)))
    big = rng.standard_normal([s + 3 for s in shape]).astype(np.float32)
    out.append(("sliced", big[tuple(slice(1, 1 + s) for s in shape)]))
    return out


@pytest.mark.parametrize("shape", [(7,), (5, 9), (33, 70), (3, 5, 7), (6, 40, 130), (2, 3, 4, 5)])
def test_small_shapes_all_axes_all_views(shape):
    rng = np.random.default_rng(11)
    nd = len(shape)
    axes_list = [[a] for a in range(nd)] + [[-1]]
    if nd >= 2:
        axes_list += [[0, 1], [1, 0], list(range(nd)), [0, nd - 1]]
    for vname, x in views(rng, shape):
        for axes in axes_list:
            for op in ("sum", "max", "mean"):
                for kd in (False, True):
                    run_case([x], op, axes, kd, what=f"{vname} {shape} {op} {axes} kd={kd}")
            if len(axes) == 1:
                run_case([x], "argmax", axes, False, what=f"{vname} {shape} argmax {axes}")
                run_case([x], "argmax", axes, True, what=f"{vname} {shape} argmax kd {axes}")


@pytest.mark.parametrize("pro,epi", [(AFFINE, EXP_EPI), (EXP_PRO, ()), (TREE_PRO, [("ACC",), ("IMM", 0, 0, 0, 3.0), ("MUL", 0, 1)]), ((), EXP_EPI)])
@pytest.mark.parametrize("shape,axis", [((257, 384), 1), ((257, 384), 0), ((12, 130, 260), 1), ((12, 130, 260), 2), ((12, 130, 260), 0)])
def test_prologue_epilogue_programs(shape, axis, pro, epi):
    rng = np.random.default_rng(12)
    x = (rng.standard_normal(shape) * 0.5).astype(np.float32)
    for op in ("sum", "max", "mean"):
        run_case([x], op, [axis], False, pro, epi, what=f"{shape} ax{axis} {op}")
    # argmax only behind exact arithmetic: expf differs in the last bit between libms and could move a tie
    run_case([x], "argmax", [axis], False, () if pro is EXP_PRO else pro, (), what=f"{shape} ax{axis} argmax")
    # same through a permuted view
    if len(shape) == 3:
        xp = np.ascontiguousarray(x.transpose(0, 2, 1)).transpose(0, 2, 1)
        run_case([xp], "sum", [axis], False, pro, epi, what=f"perm {shape} ax{axis}")


def test_readme_fusion_case_and_golden_vector():
    # README.md:59-63: sum(permute(x,(0,2,1)) + 2 + y, axis 2) * 3
    pro = [("LOAD", 0), ("IMM", 0, 0, 0, 2.0), ("ADD", 0, 1), ("LOAD", 1), ("ADD", 2, 3)]
    epi = [("ACC",), ("IMM", 0, 0, 0, 3.0), ("MUL", 0, 1)]
    rng = np.random.default_rng(1)
    x = rng.random((50, 20, 100), dtype=np.float32)
    y = rng.random((50, 100, 20), dtype=np.float32)
    got = K.fused_reduce([dev(x.transpose(0, 2, 1)), dev(y)], L.SUM, [2], False, pro, epi).cpu().numpy()
    assert_close(got, GOLD["readme_fusion/50x20x100"], 1e-5)
    rng = np.random.default_rng(1)
    x = rng.random((1000, 20, 100), dtype=np.float32)
    y = rng.random((1000, 100, 20), dtype=np.float32)
    run_case([x.transpose(0, 2, 1), y], "sum", [2], False, pro, epi, what="README fusion case")
    # two-input fast paths: both contiguous along the reduced / kept dim
    a = rng.standard_normal((300, 512)).astype(np.float32)
    b = rng.standard_normal((300, 512)).astype(np.float32)
    bc = np.broadcast_to(rng.standard_normal((300, 1)).astype(np.float32), (300, 512))
    two = [("LOAD", 0), ("LOAD", 1), ("MUL", 0, 1)]
    for ax in (0, 1):
        run_case([a, b], "sum", [ax], False, two, what=f"two-input ax{ax}")
        run_case([a, bc], "max", [ax], False, two, what=f"broadcast operand ax{ax}")


def test_epilogue_operand_and_output_dtype():
    rng = np.random.default_rng(13)
    x = rng.standard_normal((64, 200)).astype(np.float32)
    w = rng.standard_normal((64, 1)).astype(np.float32)
    epi = [("ACC",), ("LOAD", 0), ("MUL", 0, 1)]
    got = K.fused_reduce([dev(x)], L.SUM, [1], True, (), epi, epi_inputs=[dev(w)]).cpu().numpy()
    assert_close(got, x.astype(np.float64).sum(1, keepdims=True) * w, 1e-5, 1e-4)
    got16 = K.fused_reduce([dev(x)], L.MEAN, [0], False, out_dtype=torch.float16).cpu().numpy()
    assert got16.dtype == np.float16
    assert_close(got16.astype(np.float32), x.mean(0), 2e-2, 2e-3)


def test_other_dtypes_match_the_reference_dispatch():
    rng = np.random.default_rng(14)
    xd = rng.standard_normal((37, 41))
    xi = rng.integers(-50, 50, (37, 41)).astype(np.int32)
    for ax in (0, 1):
        for op in ("sum", "max", "mean"):
            run_case([xd], op, [ax], rtol=1e-12, what=f"f64 {op}")
            run_case([xi], op, [ax], exact=True, what=f"i32 {op}")
    xh = rng.standard_normal((64, 1024)).astype(np.float16)
    for ax in (0, 1):
        got = K.fused_reduce([dev(xh)], L.SUM, [ax]).cpu().numpy().astype(np.float32)
        assert_close(got, xh.astype(np.float32).sum(ax), 2e-2, 2e-2 * 32)
        got = K.fused_reduce([dev(xh)], L.ARGMAX, [ax]).cpu().numpy()
        assert np.array_equal(got, xh.astype(np.float32).argmax(ax))


@pytest.mark.parametrize("shape,axis", [((4, 1 << 20), 1), ((3, 100003), 1), ((1 << 16, 260), 0), ((5000, 33), 0), ((2, 3000, 96), 1), ((1 << 21,), 0)])
def test_split_reductions_and_workspace(shape, axis):
    rng = np.random.default_rng(15)
    x = rng.standard_normal(shape).astype(np.float32)
    xd = dev(x)
    for op in ("sum", "max", "mean", "argmax"):
        pro = AFFINE if op != "argmax" else ()
        got = K.fused_reduce([xd], OPS[op], [axis], False, pro).cpu().numpy()
        if op in ("max", "argmax"):
            assert np.array_equal(got, fused_reduce_oracle([x], op, [axis], False, pro)), (shape, op)
        else:
            # a million-term fp32 serial sum (the reference CPU loop) is itself off by more than 1e-5;
            # the bound is checked against the fp64-accumulating twin
            want = fused_reduce_truth([x], op, [axis], False, pro)
            assert_close(got, want, 1e-5, 1e-5 * max(1.0, float(np.abs(want).max())), f"{shape} {op}")
    # caller-provided workspace gives the same bits as the library's own
    out_shape = [s for i, s in enumerate(shape) if i != axis]
    need = K.reduce_workspace_bytes(xd, out_shape, L.SUM, [axis])
    a = K.fused_reduce([xd], L.SUM, [axis])
    if need:
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        b = K.fused_reduce([xd], L.SUM, [axis], workspace=ws)
        assert torch.equal(a, b)
        with pytest.raises(RuntimeError):
            K.fused_reduce([xd], L.SUM, [axis], workspace=ws[: need // 2])
    # determinism: same input twice -> identical bits
    assert torch.equal(a, K.fused_reduce([xd], L.SUM, [axis]))


def test_ties_nonfinite_and_guard_bands():
    x = np.zeros((16, 512), np.float32)
    x[:, 100] = 5.0
    x[:, 400] = 5.0  # tie: first index wins
    assert (K.fused_reduce([dev(x)], L.ARGMAX, [1]).cpu().numpy() == 100).all()
    assert (K.fused_reduce([dev(x.T)], L.ARGMAX, [0]).cpu().numpy() == 100).all()
    y = np.full((8, 300), -np.inf, np.float32)
    assert (K.fused_reduce([dev(y)], L.ARGMAX, [1]).cpu().numpy() == 0).all()
    assert np.isneginf(K.fused_reduce([dev(y)], L.MAX, [1]).cpu().numpy()).all()
    # outputs must not be written outside their extent
    big = torch.full((3, 1000), 7.0, device="cuda")
    xin = torch.randn(1000, 700, device="cuda")
    K.fused_reduce([xin], L.SUM, [1], out=big[1])
    assert (big[0] == 7).all() and (big[2] == 7).all()
    assert_close(big[1].cpu().numpy(), xin.cpu().numpy().astype(np.float64).sum(1), 1e-5, 1e-4)


def test_reduction_sweep_shapes_full_size():
    """The benchmark's tensors: A [8192,8192], B [64,4096,1024] and B.permute(0,2,1),
    prologue x*1.5+0.25, epilogue exp. A is compared with the oracle outright;
    B through oracle slabs and size-independent properties."""
    rng = np.random.default_rng(2)
    A = rng.standard_normal((8192, 8192), dtype=np.float32)
    Ad = dev(A)
    Apro = np.ascontiguousarray(eval_program(AFFINE, [A])[-1])  # the two eager prologue kernels, once
    for ax in (0, 1, -1):
        for op in ("sum", "max", "mean"):
            want = oracle.reduce(Apro, op, [ax])
            pre = K.fused_reduce([Ad], OPS[op], [ax], False, AFFINE).cpu().numpy()
            if op == "max":
                assert np.array_equal(pre, want)
            else:
                assert_close(pre, want, 1e-5, 1e-5 * float(np.abs(want).max()), f"A {op} ax{ax}")
            post = K.fused_reduce([Ad], OPS[op], [ax], False, AFFINE, EXP_EPI).cpu().numpy()
            # exp of a sum near 2048 overflows to +inf on both sides (equal infinities count as equal), and where it does
            # not, exp turns the accumulator's 1e-5 * max|sum| absolute slack into a relative one: hence 3e-3 for sum.
            # mean (|acc| near 0.25) and max keep 1e-5.
            assert_close(post, oracle.unary("exp", want), 3e-3 if op == "sum" else 1e-5, 0.0, f"A exp {op} ax{ax}")
            if op != "max":  # the epilogue itself, given the kernel's own accumulators, at 1e-5
                assert_close(post, oracle.unary("exp", pre), 1e-5, 0.0, f"A exp({op}) of its own accumulator ax{ax}")
        assert np.array_equal(K.fused_reduce([Ad], L.ARGMAX, [ax], False, AFFINE).cpu().numpy(), oracle.argmax(Apro, ax))
    del Ad, Apro


def test_reduction_sweep_B_and_its_permuted_view_full_outputs():
    """B [64,4096,1024] and B.permute(0,2,1) (a strided view), every op x axis of the sweep, with the exp epilogue:
    the WHOLE output of every case against the reference CPU backend's eager chain on the same array."""
    g = torch.Generator(device="cuda").manual_seed(2)
    B = torch.randn((64, 4096, 1024), generator=g, device="cuda")
    Bh = B.cpu().numpy()
    Bpro = np.ascontiguousarray(eval_program(AFFINE, [Bh])[-1])  # the two eager prologue kernels, once (1 GB)
    for name, T, Tpro in (("B", B, Bpro), ("Bp", B.permute(0, 2, 1), Bpro.transpose(0, 2, 1))):
        for ax in (0, 1, 2):
            n = T.shape[ax]
            for op in ("sum", "max", "mean"):
                want = oracle.reduce(Tpro, op, [ax])  # one strided CPU reduce pass, as csrc/cpu/reduce.cpp does
                pre = K.fused_reduce([T], OPS[op], [ax], False, AFFINE).cpu().numpy()
                if op == "max":
                    assert np.array_equal(pre, want), (name, op, ax)
                else:
                    assert_close(pre, want, 1e-5, 1e-5 * float(np.abs(want).max()), f"{name} {op} ax{ax}")
                post = K.fused_reduce([T], OPS[op], [ax], False, AFFINE, EXP_EPI).cpu().numpy()
                # sums of up to 4096 terms reach a few hundred: exp overflows on both sides or magnifies the
                # accumulator's absolute slack, so the epilogue is checked on the kernel's own accumulators
                assert_close(post, oracle.unary("exp", pre), 1e-5, 0.0, f"{name} exp({op}) ax{ax}")
                if op != "sum":
                    assert_close(post, oracle.unary("exp", want), 1e-5, 0.0, f"{name} exp {op} ax{ax} vs the chain")
            am = K.fused_reduce([T], L.ARGMAX, [ax], False, AFFINE).cpu().numpy()
            assert np.array_equal(am, oracle.argmax(Tpro, ax)), (name, "argmax", ax)
        # size-independent property: halves of the reduced axis recombine
        for ax in (0, 1, 2):
            n = T.shape[ax]
            lo, hi = T.narrow(ax, 0, n // 2), T.narrow(ax, n // 2, n - n // 2)
            m2 = torch.maximum(K.fused_reduce([lo], L.MAX, [ax], False, AFFINE), K.fused_reduce([hi], L.MAX, [ax], False, AFFINE))
            assert torch.equal(K.fused_reduce([T], L.MAX, [ax], False, AFFINE), m2), (name, ax)


def check_ragged(inputs, op, pro, rtol, what):
    got = K.fused_reduce([dev(i) for i in inputs], OPS[op], [1], False, pro).cpu().numpy()
    # the kernels compute 16-bit inputs in fp32; the CPU chain has no 16-bit kernels, so it gets the upcast values
    half = inputs[0].dtype == np.float16
    wide = [i.astype(np.float32) for i in inputs]
    if op == "argmax" or (op == "max" and not half):
        assert np.array_equal(got, fused_reduce_oracle(wide, op, [1], False, pro)), what
    elif op == "max":  # the fp32 maximum, rounded once to the 16-bit output
        assert_close(got.astype(np.float32), fused_reduce_oracle(wide, op, [1], False, pro), rtol, rtol, what)
    else:  # long fp32 serial sums drift: the bound is checked against the fp64-accumulating twin
        want = fused_reduce_truth(wide, op, [1], False, pro)
        assert_close(got.astype(np.float64), want, rtol, rtol * max(1.0, float(np.abs(want).max())), what)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("cols,pitch", [(50257, 50264), (1003, 1008), (37, 40), (20483, 20488)])
def test_ragged_rows_in_an_aligned_pitch(cols, pitch, dtype):
    """Row length not a multiple of the vector width inside a 16-byte-aligned row pitch (the GPT-2 logits
    layout): whole vectors plus an element-wise end. What lies in the padding must not be read as data."""
    rng = np.random.default_rng(21)
    rows = 48 if cols > 30000 else 131
    base = rng.standard_normal((rows, pitch)).astype(dtype)
    base[:, cols:] = 1e4  # larger than any element: a kernel that reads the padding fails max, argmax and sum
    x = base[:, :cols]
    rtol = 1e-5 if dtype == np.float32 else 2e-2
    for op in ("sum", "max", "argmax", "mean"):
        check_ragged([x], op, (), rtol, f"ragged {cols}/{pitch} {op}")
    check_ragged([x], "sum", AFFINE, rtol, f"ragged {cols}/{pitch} affine")
    check_ragged([x], "max", AFFINE, rtol, f"ragged {cols}/{pitch} affine max")
    check_ragged([x], "sum", EXP_PRO, rtol, f"ragged {cols}/{pitch} exp")
    y = rng.standard_normal((rows, cols)).astype(dtype)  # second operand: contiguous, so its rows are unaligned
    two = [("LOAD", 0), ("LOAD", 1), ("MUL", 0, 1)]
    check_ragged([x, y], "sum", two, rtol, f"ragged {cols}/{pitch} two inputs")
    y2 = rng.standard_normal((rows, pitch)).astype(dtype)[:, :cols]  # both operands on the vector path
    check_ragged([x, y2], "sum", two, rtol, f"ragged {cols}/{pitch} two aligned inputs")
    check_ragged([x, y2], "argmax", two, rtol, f"ragged {cols}/{pitch} two aligned inputs argmax")


def test_ragged_row_split_across_ctas():
    rng = np.random.default_rng(22)
    z = rng.standard_normal((3, 1000004)).astype(np.float32)
    z[:, 1000001:] = 1e4
    for op in ("argmax", "sum", "max"):
        check_ragged([z[:, :1000001]], op, (), 1e-5, f"ragged split {op}")


@pytest.mark.parametrize("shape", [(7, 100, 20), (3, 5, 33, 6), (40, 9, 128), (2, 300, 7), (1000, 12, 3), (5, 64, 12), (5, 64, 24),
                                   (3, 52, 36), (4, 40, 22), (6, 16, 16)])
def test_short_reduced_axis_with_operands_of_opposite_orientation(shape):
    """x read through a permute of its last two dims against a plain y (the README case's shape of problem): the
    operands disagree on which of the innermost kept axis and the short reduced axis is contiguous; every op, a
    chain prologue and an epilogue, odd sizes and rows that 128-bit loads cannot fetch."""
    rng = np.random.default_rng(31)
    *lead, J, Kr = shape
    xbuf = rng.standard_normal(tuple(lead) + (Kr, J)).astype(np.float32)
    x = np.swapaxes(xbuf, -1, -2)  # logical [.., J, K], stored [.., K, J]
    y = rng.standard_normal(shape).astype(np.float32)
    ax = len(shape) - 1
    pro = [("LOAD", 0), ("IMM", 0, 0, 0, 2.0), ("ADD", 0, 1), ("LOAD", 1), ("MUL", 2, 3)]
    epi = [("ACC",), ("IMM", 0, 0, 0, 3.0), ("MUL", 0, 1)]
    xd, yd = dev(x), dev(y)
    out_shape = K.reduced_shape(shape, [ax], False)
    od = torch.empty(out_shape, device="cuda")
    assert K.describe_reduce([K.desc(xd), K.desc(yd)], K.desc(od), L.SUM, [ax], pro).startswith("short")
    for op in ("sum", "max", "mean"):
        run_case([x, y], op, [ax], False, pro, epi, what=f"plane {shape} {op}")
        run_case([y, x], op, [ax], True, pro, (), what=f"plane swapped {shape} {op}")
    run_case([x, y], "argmax", [ax], False, pro, (), what=f"plane {shape} argmax")
