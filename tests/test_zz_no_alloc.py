"""The allocation-free fused reduce (`pgb_fused_reduce_noalloc`), through the C ABI.

Some callers of this library may not allocate device memory: a host whose own
arena already owns the whole GPU, a serving loop that keeps allocator calls off
its hot path, a plugin that is only handed pointers. For them the split
reductions keep their partial results in a fixed array inside the library
instead of a workspace. This test checks that the variant gives exactly the
bits of the regular entry point, on two calls in a row (the second call finds
the first call's partials still in the array), for every reduce op, and that a
problem whose partials do not fit is refused cleanly.

The file sorts last on purpose: a run that stops at the first failure has
already been through every other test by the time it gets here.
"""
import ctypes as C

import pytest
import torch

from pequegrad_b200 import _lib as L
from pequegrad_b200 import kernels as K

pytestmark = pytest.mark.gpu

AFFINE = [("LOAD", 0), ("IMM", 0, 0, 0, 1.5), ("MUL", 0, 1), ("IMM", 0, 0, 0, 0.25), ("ADD", 2, 3)]
EXP_EPI = [("ACC",), ("EXP", 0)]


def _out_like(ref):
    return torch.full_like(ref, -7)


@pytest.mark.parametrize("shape,axis", [((4, 1 << 20), 1), ((1 << 16, 260), 0), ((2, 3000, 96), 1), ((300, 500), 1)])
def test_matches_the_allocating_entry_point_twice_in_a_row(shape, axis):
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(shape, generator=g, device="cuda")
    y = torch.randn(shape, generator=g, device="cuda")
    out_shape = [s for i, s in enumerate(shape) if i != axis]
    uses_scratch = K.reduce_workspace_bytes(x, out_shape, L.SUM, [axis]) > 0
    assert uses_scratch or shape == (300, 500)  # the last case needs no scratch at all and must work too
    for op in (L.SUM, L.MAX, L.MEAN, L.ARGMAX):
        epi = () if op == L.ARGMAX else EXP_EPI
        for t in (x, y):  # two calls in a row through the same scratch, different data
            want = K.fused_reduce([t], op, [axis], False, AFFINE, epi)
            got = K.fused_reduce_noalloc([t], op, [axis], _out_like(want), AFFINE, epi)
            # same kernels, same partition of the work: identical bits (NaN-free inputs; inf == inf)
            assert torch.equal(got, want), (shape, axis, op)
    # and again on the first tensor: stale partials of the previous call must not leak in
    want = K.fused_reduce([x], L.SUM, [axis], False, AFFINE)
    got = K.fused_reduce_noalloc([x], L.SUM, [axis], _out_like(want), AFFINE)
    assert torch.equal(got, want)


def test_refuses_what_does_not_fit():
    # a column argmax over 300 000 columns is split in two and keeps (value, index) partials:
    # 2 x 300 000 x 8 B = 4.8 MB, more than the 4 MiB array; the sum of the same tensor (2.4 MB) fits
    big = torch.randn((128, 300000), device="cuda")
    n = 300000
    assert K.reduce_workspace_bytes(big, [n], L.SUM, [0]) <= L.NOALLOC_SCRATCH_BYTES
    out = torch.empty(n, device="cuda")
    K.fused_reduce_noalloc([big], L.SUM, [0], out)
    assert torch.equal(out, K.fused_reduce([big], L.SUM, [0]))
    need = K.reduce_workspace_bytes(big, [n], L.ARGMAX, [0], out_dtype=torch.int32)
    assert need > L.NOALLOC_SCRATCH_BYTES
    idx = torch.full((n,), -3, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="built-in array holds"):
        K.fused_reduce_noalloc([big], L.ARGMAX, [0], idx)
    torch.cuda.synchronize()
    assert (idx == -3).all()  # refused before anything was launched
    # the regular entry point still handles it, with a workspace of the caller's or its own
    assert torch.equal(K.fused_reduce([big], L.ARGMAX, [0]).long(), big.argmax(0))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_two_inputs_half_precision_and_programs_the_fast_kernels_refuse(dtype):
    """More shapes of call through the built-in array: two inputs, fp16 inputs, and a prologue that is not a chain
    (it runs on the generic kernel, which needs no scratch although the planner, asked without the prologue, reserved some)."""
    g = torch.Generator(device="cuda").manual_seed(6)
    a = torch.randn((6, 1 << 18), generator=g, device="cuda").to(dtype)
    b = torch.randn((6, 1 << 18), generator=g, device="cuda").to(dtype)
    two = [("LOAD", 0), ("LOAD", 1), ("MUL", 0, 1)]
    tree = [("LOAD", 0), ("IMM", 0, 0, 0, 1.0), ("ADD", 0, 1), ("IMM", 0, 0, 0, 2.0), ("SUB", 0, 3), ("MUL", 2, 4)]
    for ins, pro in (([a, b], two), ([a], tree), ([a], AFFINE)):
        for op in (L.SUM, L.MAX, L.ARGMAX):
            for _ in range(2):
                want = K.fused_reduce(ins, op, [1], False, pro)
                got = K.fused_reduce_noalloc(ins, op, [1], _out_like(want), pro)
                assert torch.equal(got, want), (dtype, op, len(ins))


class _DefaultPool:
    """The device's default stream-ordered memory pool, read through the CUDA runtime: every cudaMallocAsync of this
    library draws from it, so its high-water mark shows whether a call allocated."""
    USED_CURRENT, USED_HIGH = 7, 8  # cudaMemPoolAttrUsedMemCurrent, cudaMemPoolAttrUsedMemHigh

    def __init__(self):
        self.rt = C.CDLL("libcudart.so.12")
        self.pool = C.c_void_p()
        assert self.rt.cudaDeviceGetDefaultMemPool(C.byref(self.pool), torch.cuda.current_device()) == 0

    def get(self, attr):
        v = C.c_uint64(0)
        assert self.rt.cudaMemPoolGetAttribute(self.pool, attr, C.byref(v)) == 0
        return v.value

    def reset_high(self):
        v = C.c_uint64(0)
        assert self.rt.cudaMemPoolSetAttribute(self.pool, self.USED_HIGH, C.byref(v)) == 0

    def free_bytes(self):
        f, t = C.c_size_t(0), C.c_size_t(0)
        assert self.rt.cudaMemGetInfo(C.byref(f), C.byref(t)) == 0
        return f.value


def test_the_call_allocates_nothing_on_the_device():
    x = torch.randn((4, 1 << 20), device="cuda")
    need = K.reduce_workspace_bytes(x, [4], L.SUM, [1])
    assert need > 0
    want = K.fused_reduce([x], L.SUM, [1], False, AFFINE, EXP_EPI)
    out = _out_like(want)
    K.fused_reduce_noalloc([x], L.SUM, [1], out, AFFINE, EXP_EPI)  # first call on the device: looks up the array's address
    torch.cuda.synchronize()
    pool = _DefaultPool()
    # control: the regular entry point without a caller workspace takes its partials from the pool, and the probe sees it
    pool.reset_high()
    base = pool.get(pool.USED_CURRENT)
    K.fused_reduce([x], L.SUM, [1], False, AFFINE, EXP_EPI, out=out)
    torch.cuda.synchronize()
    assert pool.get(pool.USED_HIGH) >= base + need
    # the variant: no stream-ordered allocation (the pool's high-water mark does not move) and no plain one either
    pool.reset_high()
    base, free0 = pool.get(pool.USED_CURRENT), pool.free_bytes()
    for _ in range(3):
        K.fused_reduce_noalloc([x], L.SUM, [1], out, AFFINE, EXP_EPI)
    torch.cuda.synchronize()
    assert pool.get(pool.USED_HIGH) == base and pool.get(pool.USED_CURRENT) == base
    assert pool.free_bytes() >= free0  # nothing was taken from the device by cudaMalloc either
    assert torch.equal(out, want)
