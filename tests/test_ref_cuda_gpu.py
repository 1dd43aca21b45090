"""The reference's own CUDA kernels (csrc/cuda reduce / binary / exp / where, and the generated kernel its README
prints), compiled from its checkout into oracle/_ref_cuda, as a second oracle: the fused kernels of this library
against the eager chain of reference kernels on the same device arrays. Sums differ in summation order on both
sides (64 strided threads per output there), hence rel 1e-5 with the absolute floor the reference's tests use;
max is bit-exact."""
import numpy as np
import pytest
import torch

from helpers import assert_close
from oracle import ref_cuda
from pequegrad_b200 import _lib as L
from pequegrad_b200 import kernels as K
from pequegrad_b200.workloads import AFFINE, EXP_EPI, README_EPI, README_PRO

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref_cuda was not built (needs the reference checkout)")]
OPS = {"sum": L.SUM, "max": L.MAX, "mean": L.MEAN}


def _views(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(shape, generator=g, device="cuda")
    views = [("contiguous", x)]
    if len(shape) == 3:
        views.append(("permuted", torch.randn((shape[0], shape[2], shape[1]), generator=g, device="cuda").permute(0, 2, 1)))
        views.append(("sliced", torch.randn((shape[0], shape[1], shape[2] + 5), generator=g, device="cuda")[:, :, 3:3 + shape[2]]))
    else:
        views.append(("transposed", torch.randn((shape[1], shape[0]), generator=g, device="cuda").t()))
    return views


@pytest.mark.parametrize("shape", [(37, 129), (257, 384), (12, 130, 66), (5, 7, 1030)])
def test_fused_reduce_matches_the_reference_cuda_chain(shape):
    for what, x in _views(shape, 11):
        for ax in range(len(shape)):
            for op in ("sum", "max", "mean"):
                want = ref_cuda.EagerReduceChain(x, op, [ax], exp=False)().cpu().numpy()
                got = K.fused_reduce([x], OPS[op], [ax], False, AFFINE).cpu().numpy()
                if op == "max":
                    assert np.array_equal(got, want), (what, shape, ax)
                else:
                    assert_close(got, want, 1e-5, 1e-5 * float(np.abs(want).max()), f"{what} {shape} {op} ax{ax}")
                # the exp epilogue, against the reference's exp kernel applied to the same accumulators
                post = K.fused_reduce([x], OPS[op], [ax], False, AFFINE, EXP_EPI)
                want_post = ref_cuda.exp_dense(torch.from_numpy(got).cuda())
                assert_close(post.cpu().numpy(), want_post.cpu().numpy(), 1e-5, 0.0, f"{what} {shape} exp({op}) ax{ax}")


def test_multi_axis_and_elementwise_kernels():
    g = torch.Generator(device="cuda").manual_seed(12)
    x = torch.randn((6, 20, 33), generator=g, device="cuda")
    for axes in ([0, 2], [1, 2], [0, 1, 2]):
        want = ref_cuda.Reduce(x, "sum", axes)().cpu().numpy()
        got = K.fused_reduce([x], L.SUM, axes).cpu().numpy()
        assert_close(got, want, 1e-5, 1e-5 * float(np.abs(want).max()), f"axes {axes}")
    # binary-broadcast and where: bit-exact
    y = torch.randn((20, 1), generator=g, device="cuda")
    for name, prog in (("add", "ADD"), ("mul", "MUL"), ("max", "MAX")):
        want = ref_cuda.Binary(name, x, y.expand(x.shape))()
        (got,) = K.fused_elementwise([x, y.expand(x.shape)], [("LOAD", 0), ("LOAD", 1), (prog, 0, 1)])
        assert torch.equal(got, want), name
    c = (x > 0).float()
    want = ref_cuda.where(c, x, y)
    (got,) = K.fused_elementwise([c, x, y.expand(x.shape)], [("LOAD", 0), ("LOAD", 1), ("LOAD", 2), ("WHERE", 0, 1, 2)])
    assert torch.equal(got, want)


def test_readme_kernel_and_sweep_tensor_A():
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.rand((1000, 20, 100), generator=g, device="cuda")
    y = torch.rand((1000, 100, 20), generator=g, device="cuda")
    want = ref_cuda.readme_kernel(x, y).cpu().numpy()
    got = K.fused_reduce([x.permute(0, 2, 1), y], L.SUM, [2], False, README_PRO, README_EPI).cpu().numpy()
    assert_close(got, want, 1e-5, 1e-5 * float(np.abs(want).max()), "README fusion case")
    # the sweep's A [8192,8192], all three axes
    g = torch.Generator(device="cuda").manual_seed(2)
    A = torch.randn((8192, 8192), generator=g, device="cuda")
    for ax in (0, 1, -1):
        for op in ("sum", "max", "mean"):
            want = ref_cuda.EagerReduceChain(A, op, [ax], exp=False)().cpu().numpy()
            got = K.fused_reduce([A], OPS[op], [ax], False, AFFINE).cpu().numpy()
            if op == "max":
                assert np.array_equal(got, want), (op, ax)
            else:
                assert_close(got, want, 1e-5, 1e-5 * float(np.abs(want).max()), f"A {op} ax{ax}")
