"""No-GPU checks of the boundary: the library loads, exports every symbol the
header declares, validates arguments, plans the configured workloads onto the
intended kernel families, and refuses to compute without a device."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest
import torch

from pequegrad_b200 import _lib as L

ROOT = Path(__file__).resolve().parents[1]
F32 = 4


def _t(shape, strides_elems=None, dtype=L.F32, es=4, ptr=4096):
    if strides_elems is None:
        strides_elems, acc = [], 1
        for s in reversed(shape):
            strides_elems.append(acc)
            acc *= s
        strides_elems.reverse()
    return L.make_tensor(ptr, dtype, shape, [s * es for s in strides_elems])


def _describe(x, out_shape, op, axes, prologue=(), out_dtype=L.F32):
    from pequegrad_b200 import kernels as K
    es = {L.F64: 8, L.F16: 2}.get(out_dtype, 4)
    return K.describe_reduce([x] if not isinstance(x, list) else x, _t(out_shape, dtype=out_dtype, es=es), op, axes, prologue)


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "pgb200.h").read_text()
    declared = set(re.findall(r"PGB_API\s+[\w\s\*]+?\b(pgb_\w+)\s*\(", header))
    assert declared and declared == set(L.EXPORTS)
    lib = L.lib()
    for name in declared:
        assert getattr(lib, name) is not None
    assert b"sm_100a" in lib.pgb_version()
    assert lib.pgb_status_string(L.ERR_UNSUPPORTED) == b"not implemented"


AFFINE = [("LOAD", 0), ("IMM", 0, 0, 0, 1.5), ("MUL", 0, 1), ("IMM", 0, 0, 0, 0.25), ("ADD", 2, 3)]


@pytest.mark.parametrize("case,expect", [
    # reduction sweep shapes: A [8192,8192]; B [64,4096,1024]; Bp = B.permute(0,2,1)
    (("A", 1), "row"), (("A", 0), "col"),
    (("B", 2), "row"), (("B", 1), "col"), (("B", 0), "col"),
    (("Bp", 1), "row"), (("Bp", 2), "col"), (("Bp", 0), "col"),
])
def test_planner_families_for_the_reduction_sweep(case, expect):
    name, axis = case
    if name == "A":
        shape, strides = (8192, 8192), None
    elif name == "B":
        shape, strides = (64, 4096, 1024), None
    else:
        shape, strides = (64, 1024, 4096), [4096 * 1024, 1, 1024]
    out_shape = [s for i, s in enumerate(shape) if i != axis]
    for op in (L.SUM, L.MAX, L.MEAN, L.ARGMAX):
        d = _describe(_t(shape, strides), out_shape, op, [axis], AFFINE, L.I32 if op == L.ARGMAX else L.F32)
        assert d.startswith(expect), d
        assert "vec=4" in d and "chain" in d, d
    d = _describe(_t(shape, strides), out_shape, L.SUM, [axis])
    assert "ident" in d, d


def test_planner_split_and_workspace():
    from pequegrad_b200 import kernels as K
    # few long rows -> split across CTAs with a second stage
    d = _describe(_t((4, 1 << 22)), (4,), L.SUM, [1])
    assert d.startswith("row") and "split=1 " not in d, d
    assert K.reduce_workspace_bytes(_t((4, 1 << 22)), (4,), L.SUM, [1]) > 0
    assert K.reduce_workspace_bytes(_t((8192, 8192)), (8192,), L.SUM, [1]) == 0
    # full reduction merges to one row
    d = _describe(_t((64, 4096, 1024)), (), L.SUM, [0, 1, 2])
    assert d.startswith("row") and "R1=1" in d, d
    # unaligned base pointer or odd row length -> scalar loads, still coalesced
    assert "vec=1" in _describe(_t((64, 1001)), (64,), L.SUM, [1])
    assert "vec=1" in _describe(_t((64, 1024), ptr=4100), (64,), L.SUM, [1])
    # f64 and i32 take the generic kernel (reference: PG_DISPATCH_ALL_TYPES)
    assert _describe(_t((64, 64), dtype=L.F64, es=8), (64,), L.SUM, [1], out_dtype=L.F64).startswith("generic")


def test_readme_fusion_plans():
    # x: permute(0,2,1) view of [1000,20,100]; y contiguous [1000,100,20]; sum over axis 2
    x = _t((1000, 100, 20), [2000, 1, 100])
    y = _t((1000, 100, 20))
    pro = [("LOAD", 0), ("IMM", 0, 0, 0, 2.0), ("ADD", 0, 1), ("LOAD", 1), ("ADD", 2, 3)]
    d = _describe([x, y], (1000, 100), L.SUM, [2], pro)
    assert d, d


def test_argument_errors_are_reported_like_the_reference():
    lib = L.lib()
    x = _t((4, 5))
    out = _t((4,))
    ax = (C.c_int32 * 1)(3)
    buf = C.create_string_buffer(256)
    pro, n = L.make_program([])
    st = lib.pgb_fused_reduce_describe(C.byref(x), 1, C.byref(out), L.SUM, ax, 1, pro, 0, buf, 256)
    assert st == L.ERR_INVALID_ARG and b"axis out of range" in lib.pgb_last_error()
    with pytest.raises(ValueError):
        L.check(st)
    ax = (C.c_int32 * 1)(1)
    bad = _t((5,))
    st = lib.pgb_fused_reduce_describe(C.byref(x), 1, C.byref(bad), L.SUM, ax, 1, pro, 0, buf, 256)
    assert st == L.ERR_INVALID_ARG and b"output shape" in lib.pgb_last_error()
    # operands may only refer to earlier values
    pro, n = L.make_program([("LOAD", 0), ("ADD", 0, 1)])
    st = lib.pgb_fused_reduce_describe(C.byref(x), 1, C.byref(out), L.SUM, ax, 1, pro, n, buf, 256)
    assert st == L.ERR_INVALID_ARG and b"later value" in lib.pgb_last_error()
    # argmax needs one axis and an int32 output
    st = lib.pgb_fused_reduce_describe(C.byref(x), 1, C.byref(out), L.ARGMAX, ax, 1, pro, 0, buf, 256)
    assert st == L.ERR_INVALID_ARG and b"int32" in lib.pgb_last_error()


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-device behaviour")
def test_compute_calls_fail_loudly_without_a_device():
    lib = L.lib()
    x, out = _t((4, 5)), _t((4,))
    ax = (C.c_int32 * 1)(1)
    pro, _ = L.make_program([])
    st = lib.pgb_fused_reduce(C.byref(x), 1, C.byref(out), L.SUM, ax, 1, pro, 0, None, 0, pro, 0, None, 0, None)
    assert st == L.ERR_CUDA and b"no CPU fallback" in lib.pgb_last_error()
    with pytest.raises(RuntimeError):
        L.check(st)
    from pequegrad_b200 import kernels as K
    with pytest.raises(RuntimeError):
        K.fused_reduce([torch.zeros(4, 5)], L.SUM, [1])


def test_tensor_core_entry_points_validate_their_arguments():
    """Host-side validation of matmul / qlinear / attention / quantise: shapes, dtypes and layouts are checked before any device call."""
    lib = L.lib()
    f16 = lambda shape, strides=None, ptr=4096: _t(shape, strides, dtype=L.F16, es=2, ptr=ptr)  # noqa: E731
    i8 = lambda shape: _t(shape, None, dtype=L.I8, es=1)  # noqa: E731

    def err(st, code, text):
        assert st == code, (st, lib.pgb_last_error())
        assert text in lib.pgb_last_error(), lib.pgb_last_error()

    # matmul: dtype the reference does not have either, mismatching contraction dims, unknown activation
    a32i, o32i = _t((8, 16), dtype=L.I32), _t((8, 8), dtype=L.I32)
    err(lib.pgb_matmul(C.byref(a32i), C.byref(_t((16, 8), dtype=L.I32)), None, 0, 1.0, None, C.byref(o32i), None), L.ERR_UNSUPPORTED,
        b"matmul_cuda not implemented for int32")
    a64 = _t((8, 16), dtype=L.F64, es=8)
    err(lib.pgb_matmul(C.byref(a64), C.byref(_t((12, 8), dtype=L.F64, es=8)), None, 0, 1.0, None, C.byref(_t((8, 8), dtype=L.F64, es=8)), None),
        L.ERR_INVALID_ARG, b"contraction dims differ")
    a, out = f16((8, 16)), f16((8, 24))
    err(lib.pgb_matmul(C.byref(a), C.byref(f16((24, 8), (1, 24))), None, 0, 1.0, None, C.byref(out), None), L.ERR_INVALID_ARG, b"contraction dims differ")
    err(lib.pgb_matmul(C.byref(a), C.byref(f16((16, 24), (1, 16))), None, 7, 1.0, None, C.byref(out), None), L.ERR_INVALID_ARG, b"unknown activation")
    err(lib.pgb_matmul(C.byref(a), C.byref(f16((16, 24), (1, 16))), None, 0, 1.0, None, C.byref(f16((8, 20))), None), L.ERR_INVALID_ARG,
        b"output shape does not match")
    # qlinear: int8 operands, something to write, an absmax for an int8 output
    err(lib.pgb_qlinear_i8(C.byref(a), C.byref(i8((24, 16))), None, 1.0, None, None, 0, C.byref(_t((8, 24))), None, None, None), L.ERR_UNSUPPORTED,
        b"must be int8")
    err(lib.pgb_qlinear_i8(C.byref(i8((8, 16))), C.byref(i8((24, 16))), None, 1.0, None, None, 0, None, None, None, None), L.ERR_INVALID_ARG,
        b"nothing to write")
    err(lib.pgb_qlinear_i8(C.byref(i8((8, 16))), C.byref(i8((24, 16))), None, 1.0, None, None, 0, C.byref(i8((8, 24))), None, None, None), L.ERR_INVALID_ARG,
        b"device absmax")
    err(lib.pgb_qlinear_i8(C.byref(i8((8, 16))), C.byref(i8((24, 32))), None, 1.0, None, None, 0, C.byref(_t((8, 24))), None, None, None), L.ERR_INVALID_ARG,
        b"contraction dims differ")
    # attention: head dim, dtype, agreement of the operands, scale
    q = f16((2, 4, 32, 64))
    err(lib.pgb_attention(C.byref(f16((2, 4, 32, 32))), C.byref(q), C.byref(q), 0.125, 1, C.byref(q), None), L.ERR_UNSUPPORTED, b"head dim of 64")
    q32 = _t((2, 4, 32, 64))
    err(lib.pgb_attention(C.byref(q32), C.byref(q32), C.byref(q32), 0.125, 1, C.byref(q32), None), L.ERR_UNSUPPORTED, b"attention not implemented for float32")
    err(lib.pgb_attention(C.byref(q), C.byref(f16((2, 4, 16, 64))), C.byref(q), 0.125, 1, C.byref(q), None), L.ERR_INVALID_ARG, b"disagree")
    # quantise: fp32 in, int8 out, one size
    err(lib.pgb_quantize_i8(C.byref(_t((8, 16))), None, 0.5, C.byref(i8((8, 8))), None), L.ERR_INVALID_ARG, b"one size")
    err(lib.pgb_quantize_i8(C.byref(_t((8, 16))), None, 0.0, C.byref(i8((8, 16))), None), L.ERR_INVALID_ARG, b"positive scale")
