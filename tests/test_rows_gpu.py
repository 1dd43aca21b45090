"""GPU parity of the single-kernel row softmax and LayerNorm through the C ABI."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close, ref_test_inputs
from pequegrad_b200 import kernels as K

pytestmark = pytest.mark.gpu
GOLD = np.load(Path(__file__).parent / "golden" / "ref_cpu_vectors.npz")


def test_reference_composite_cases():
    # tests/test_high_level_ops.py:100-121, 354-367: torch CPU is the reference's own oracle
    for shape in [(2, 3, 4), (5, 10), (4, 768)]:
        (x,) = ref_test_inputs([shape], np.float32)
        got = K.layernorm_rows(torch.from_numpy(x).cuda(), None, None, 1e-5).cpu().numpy()
        assert_close(got, GOLD["layer_norm/" + "x".join(map(str, shape)) + "/n1"], 1e-4)
    for shape in [(2, 3), (8, 1024)]:
        (x,) = ref_test_inputs([shape], np.float32)
        got = K.softmax_rows(torch.from_numpy(x).cuda()).cpu().numpy()
        assert_close(got, GOLD["softmax/" + "x".join(map(str, shape))], 1e-5)


@pytest.mark.parametrize("C", [1, 7, 64, 100, 768, 1000, 1024, 2048, 4096, 5000])
def test_layernorm_fp32(C):
    rng = np.random.default_rng(31)
    x = rng.standard_normal((37, C)).astype(np.float32)
    g = (1 + 0.02 * rng.standard_normal(C)).astype(np.float32)
    b = (0.02 * rng.standard_normal(C)).astype(np.float32)
    xd, gd, bd = (torch.from_numpy(t).cuda() for t in (x, g, b))
    got = K.layernorm_rows(xd, gd, bd, 1e-5).cpu().numpy()
    x64 = x.astype(np.float64)
    mu = x64.mean(1, keepdims=True)
    want = (x64 - mu) / np.sqrt(x64.var(1, keepdims=True) + 1e-5) * g + b
    assert_close(got, want, 1e-5, 2e-5)
    assert_close(got, oracle.layernorm_rows(x, g, b, 1e-5), 1e-5, 2e-5)
    got = K.layernorm_rows(xd, None, None, 1e-5).cpu().numpy()
    assert_close(got, (x64 - mu) / np.sqrt(x64.var(1, keepdims=True) + 1e-5), 1e-5, 2e-5)


def test_layernorm_configured_shape():
    rng = np.random.default_rng(4)
    x = rng.standard_normal((16384, 768), dtype=np.float32)
    g = (1 + 0.02 * rng.standard_normal(768)).astype(np.float32)
    b = (0.02 * rng.standard_normal(768)).astype(np.float32)
    got = K.layernorm_rows(*(torch.from_numpy(t).cuda() for t in (x, g, b)), 1e-5).cpu().numpy()
    assert_close(got, oracle.layernorm_rows(x, g, b, 1e-5), 1e-5, 2e-5)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("shape,causal", [((5, 33), False), ((2, 3, 64, 64), True), ((3, 100, 1000), False), ((2, 2, 128, 256), True),
                                          ((1, 2, 1024, 1024), True), ((4, 2048), False), ((3, 5000), False), ((2, 300, 200), True)])
def test_softmax(shape, causal, dtype):
    rng = np.random.default_rng(32)
    x = rng.standard_normal(shape).astype(dtype)
    want = oracle.softmax_rows(x.astype(np.float32), causal)  # fp32 math on the fp16-rounded input
    got = K.softmax_rows(torch.from_numpy(x).cuda(), causal).cpu().numpy()
    assert got.dtype == dtype
    if dtype == np.float16:
        assert_close(got.astype(np.float32), want, 2e-2, 1e-4)
    else:
        assert_close(got, want, 1e-5, 1e-7)
    if causal:
        T, C = shape[-2], shape[-1]
        masked = np.triu(np.ones((T, C), bool), 1)
        assert (got[..., masked] == 0).all()  # excluded entries are exactly 0
    assert_close(got.astype(np.float64).sum(-1), np.ones(shape[:-1]), 2e-3 if dtype == np.float16 else 1e-5)


def test_softmax_configured_shape_slices_and_errors():
    # the configured tensor, fp16 [32,12,1024,1024]; the oracle on (batch, head) slices spread over it
    g = torch.Generator(device="cuda").manual_seed(4)
    s = torch.randn((32, 12, 1024, 1024), generator=g, device="cuda").half()
    y = K.softmax_rows(s, causal=True)
    for b, h in ((0, 0), (1, 3), (15, 7), (31, 11)):
        want = oracle.softmax_rows(s[b, h].float().cpu().numpy()[None], causal=True)[0]
        assert_close(y[b, h].float().cpu().numpy(), want, 2e-2, 1e-4, f"slice ({b},{h})")
    # size-independent properties over the whole output: nothing above the diagonal, rows sum to one
    mask = torch.triu(torch.ones(1024, 1024, dtype=torch.bool, device="cuda"), 1)
    assert not y[:, :, mask].any()
    sums = y.float().sum(-1)
    assert float((sums - 1).abs().max()) < 2e-3
    del y, sums
    with pytest.raises(RuntimeError):
        K.softmax_rows(s.permute(0, 1, 3, 2))  # non-contiguous rows are refused, not silently copied
    with pytest.raises(RuntimeError):
        K.softmax_rows(torch.zeros(4, 4, dtype=torch.int32, device="cuda"))


def test_rows_workload_on_two_streams_gives_the_kernels_bits():
    # the benchmark runs the LayerNorm on a stream that forks from and joins the timed one, under the softmax
    from pequegrad_b200 import workloads as W
    wl = W.Rows()
    wl.SM_SHAPE, wl.LN_SHAPE = (2, 12, 1024, 1024), (4096, 768)
    wl.setup(torch.device("cuda:0"), 0, 1)
    for _ in range(3):
        wl.step()
    torch.cuda.synchronize()
    assert torch.equal(wl.sm_out, K.softmax_rows(wl.S, causal=True))
    assert torch.equal(wl.ln_out, K.layernorm_rows(wl.X, wl.gamma, wl.beta, 1e-5))
