"""GPU parity of the tensor-core GEMMs through the C ABI.

int8 quantized linear: int32 accumulators bit-exact against the oracle; the
dequant + bias + ReLU epilogue and the dynamic activation quantiser bit-exact
too (same fp32 operations in the same order). f16 / bf16 matmul: fp32
accumulation, compared with an fp32 reference at 2e-2 (the bound north_star
states for half precision)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close
from pequegrad_b200 import _lib as L
from pequegrad_b200 import kernels as K

pytestmark = pytest.mark.gpu


def cu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("M,N,K_", [(128, 128, 128), (200, 10, 1024), (513, 1024, 784), (1024, 1024, 1024), (1, 16, 16), (130, 257, 48)])
def test_int8_accumulators_bit_exact(M, N, K_):
    rng = np.random.default_rng(41)
    a = rng.integers(-127, 128, (M, K_)).astype(np.int8)
    w = rng.integers(-127, 128, (N, K_)).astype(np.int8)
    ws = (rng.random(N) * 0.01 + 1e-3).astype(np.float32)
    b = (rng.standard_normal(N) * 0.05).astype(np.float32)
    want_acc = oracle.gemm_i8(a, w)
    for relu in (False, True):
        out, acc = K.qlinear_i8(cu(a), cu(w), cu(ws), a_scale=0.0123, bias=cu(b), relu=relu, want_acc=True)
        assert K.device_error() == 0
        assert np.array_equal(acc.cpu().numpy(), want_acc)
        want = oracle.dequant_bias_act(want_acc, ws, np.float32(0.0123), b, relu)
        assert np.array_equal(out.cpu().numpy(), want)  # same fp32 ops, same order
    out16, _ = K.qlinear_i8(cu(a), cu(w), cu(ws), a_scale=0.0123, bias=cu(b), relu=True, out_dtype=torch.float16)
    assert np.array_equal(out16.cpu().numpy(), want.astype(np.float16))
    _, acc = K.qlinear_i8(cu(a), cu(w), cu(ws), a_scale=1.0, want_acc=True, want_out=False)
    assert np.array_equal(acc.cpu().numpy(), want_acc)


def test_dynamic_activation_quantiser_bit_exact():
    rng = np.random.default_rng(42)
    for shape in [(7, 13), (1000, 784), (33, 4099)]:
        x = (rng.standard_normal(shape) * 3).astype(np.float32)
        am = K.absmax(cu(x))
        assert float(am.cpu()) == oracle.absmax(x)
        q = K.quantize_i8(cu(x), absmax_dev=am)
        s = oracle.quant_scale(oracle.absmax(x))
        assert np.array_equal(q.cpu().numpy(), oracle.quantize_i8(x, s))
        q2 = K.quantize_i8(cu(x), scale=float(s))
        assert np.array_equal(q2.cpu().numpy(), oracle.quantize_i8(x, s))
    z = np.zeros((5, 5), np.float32)  # the 1e-6 floor of examples/quantized_mlp.py:30
    assert (K.quantize_i8(cu(z), absmax_dev=K.absmax(cu(z))).cpu().numpy() == 0).all()


def _mlp_oracle(X, Ws, bs):
    """784 -> 1024 -> 1024 -> 10 with ReLU, per-channel int8 weights, dynamic per-tensor int8 activations."""
    h, per_layer = X, []
    for i, (W, b) in enumerate(zip(Ws, bs)):
        wq, wsc = oracle.quantize_weight_per_channel(W)
        sx = oracle.quant_scale(oracle.absmax(h))
        xq = oracle.quantize_i8(h, sx)
        acc = oracle.gemm_i8(xq, wq)
        h = oracle.dequant_bias_act(acc, wsc, sx, b, relu=i < len(Ws) - 1)
        per_layer.append((xq, wq, wsc, sx, acc, h))
    return per_layer


def test_quantized_mlp_layers_and_pipeline():
    rng = np.random.default_rng(3)
    dims = [784, 1024, 1024, 10]
    Ws = [(rng.standard_normal((dims[i], dims[i + 1])) * 0.05).astype(np.float32) for i in range(3)]
    bs = [(rng.standard_normal(dims[i + 1]) * 0.05).astype(np.float32) for i in range(3)]
    X = rng.random((2048, 784), dtype=np.float32)
    layers = _mlp_oracle(X, Ws, bs)
    # (1) per layer: the oracle's int8 inputs through the GPU GEMM -> bit-exact accumulators and outputs
    for i, (xq, wq, wsc, sx, acc, h) in enumerate(layers):
        out, gacc = K.qlinear_i8(cu(xq), cu(wq), cu(wsc), a_scale=float(sx), bias=cu(bs[i]), relu=i < 2, want_acc=True)
        assert np.array_equal(gacc.cpu().numpy(), acc), f"layer {i} accumulators"
        assert np.array_equal(out.cpu().numpy(), h), f"layer {i} outputs"
    # (2) whole pipeline on the device, scales never leave the GPU
    hd = cu(X)
    am = K.absmax(hd)
    for i in range(3):
        wq, wsc = layers[i][1], layers[i][2]
        xq = K.quantize_i8(hd, absmax_dev=am)
        assert np.array_equal(xq.cpu().numpy(), layers[i][0]), f"layer {i} quantised activations"
        nxt = torch.zeros(1, device="cuda")
        hd, _ = K.qlinear_i8(xq, cu(wq), cu(wsc), a_absmax=am, bias=cu(bs[i]), relu=i < 2, out_absmax=nxt)
        am = nxt
    assert K.device_error() == 0
    assert_close(hd.cpu().numpy(), layers[2][5], 1e-5)
    # and the quantised network tracks the fp32 one
    ref = X
    for i in range(3):
        ref = ref @ Ws[i] + bs[i]
        if i < 2:
            ref = np.maximum(ref, 0)
    assert np.abs(hd.cpu().numpy() - ref).mean() < 0.05 * np.abs(ref).mean()


def test_reference_fake_quant_numerics_through_the_fused_kernels():
    # examples/quantized_mlp.py:28-34 expanded to primitives: abs = (x**2)**0.5, round = trunc(x + 0.5),
    # clip = where chains; everything fp32, per tensor. Run as fused reduce + fused elementwise kernels.
    from pequegrad_b200 import _lib as L
    rng = np.random.default_rng(9)
    w = (rng.standard_normal((784, 1024)) * 0.05).astype(np.float32)
    wd = cu(w)
    absprog = [("LOAD", 0), ("IMM", 0, 0, 0, 2.0), ("POW", 0, 1), ("IMM", 0, 0, 0, 0.5), ("POW", 2, 3)]
    wmax = K.fused_reduce([wd], L.MAX, [0, 1], True, absprog, [("ACC",), ("IMM", 0, 0, 0, 1e-6), ("MAX", 0, 1)])
    scale = wmax.expand(784, 1024)
    q = [("LOAD", 0), ("LOAD", 1), ("DIV", 0, 1), ("IMM", 0, 0, 0, 127.0), ("MUL", 2, 3), ("IMM", 0, 0, 0, 0.5), ("ADD", 4, 5), ("CAST_I32", 6),
         ("IMM", 0, 0, 0, -128.0), ("IMM", 0, 0, 0, 127.0), ("GT", 7, 9), ("WHERE", 10, 9, 7), ("LT", 7, 8), ("WHERE", 12, 8, 11),
         ("DIV", 13, 3), ("MUL", 14, 1)]
    (wq,) = K.fused_elementwise([wd, scale], q)
    ws = np.float32(max(np.sqrt(np.float32(w) ** 2).max(), 1e-6))
    r = (w / ws * np.float32(127) + np.float32(0.5)).astype(np.int32).astype(np.float32)
    want = np.clip(r, -128, 127) / np.float32(127) * ws
    assert_close(float(wmax.cpu()), float(ws), 1e-6)
    got = wq.cpu().numpy()
    assert_close(got, want, 1e-5, 1e-6)
    # trunc(x + 0.5) rounds negatives toward zero-ish (-1.7 -> -1): up to one and a half steps off
    assert np.abs(got - w).max() <= ws / 127 * 1.51


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,N,K_", [(128, 128, 64), (300, 200, 520), (1024, 768, 768), (77, 50264, 64)])
def test_half_matmul_fp32_accumulate(M, N, K_, dt):
    g = torch.Generator(device="cuda").manual_seed(5)
    a = (torch.randn((M, K_), generator=g, device="cuda") * 0.5).to(dt)
    wt = (torch.randn((N, K_), generator=g, device="cuda") * 0.5).to(dt)
    out = K.matmul(a, wt.T, out_dtype=torch.float32)
    assert K.device_error() == 0
    ref = a.float() @ wt.float().T
    assert_close(out.cpu().numpy(), ref.cpu().numpy(), 1e-4, 1e-4 * float(ref.abs().max()))  # fp32 accumulation: far inside 2e-2
    out_h = K.matmul(a, wt.T)
    assert out_h.dtype == dt
    assert_close(out_h.float().cpu().numpy(), ref.cpu().numpy(), 2e-2, 2e-2 * float(ref.abs().max()))


def test_linear_epilogues_and_batched_attention_shapes():
    g = torch.Generator(device="cuda").manual_seed(6)
    x = (torch.randn((4, 96, 768), generator=g, device="cuda") * 0.5).half()
    wt = (torch.randn((3072, 768), generator=g, device="cuda") * 0.02).half()
    b = (torch.randn(3072, generator=g, device="cuda") * 0.02).half()
    y = K.matmul(x, wt.T, bias=b, act=2)  # Linear + GELU(tanh), batch folded into M
    z = (x.float() @ wt.float().T + b.float())
    ref = 0.5 * z * (1 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
    assert_close(y.float().cpu().numpy(), ref.cpu().numpy(), 2e-2, 2e-3)
    wt2 = (torch.randn((768, 3072), generator=g, device="cuda") * 0.02).half()
    res = (torch.randn((4, 96, 768), generator=g, device="cuda")).half()
    y2 = K.matmul(y, wt2.T, residual=res)  # projection + residual add
    ref2 = y.float() @ wt2.float().T + res.float()
    assert_close(y2.float().cpu().numpy(), ref2.cpu().numpy(), 2e-2, 2e-3)
    y3 = K.matmul(x, wt.T, act=1, out_dtype=torch.float32)
    assert_close(y3.cpu().numpy(), torch.relu(x.float() @ wt.float().T).cpu().numpy(), 1e-4, 1e-4)
    # scores = q @ k^T per (batch, head): both operands batched, k^T is a transposed view
    q = (torch.randn((2, 12, 256, 64), generator=g, device="cuda")).half()
    k = (torch.randn((2, 12, 256, 64), generator=g, device="cuda")).half()
    s = K.matmul(q, k.transpose(-2, -1), out_dtype=torch.float32)
    assert_close(s.cpu().numpy(), (q.float() @ k.float().transpose(-2, -1)).cpu().numpy(), 1e-4, 1e-3)
    assert K.device_error() == 0


def test_matmul_errors_follow_the_reference():
    a = torch.zeros((8, 16), device="cuda", dtype=torch.int32)
    with pytest.raises(RuntimeError, match="matmul_cuda not implemented for int32"):
        K.matmul(a, a.T)
    h = torch.zeros((16, 16), device="cuda", dtype=torch.float16)
    with pytest.raises(ValueError):
        K.matmul(h, torch.zeros((24, 8), device="cuda", dtype=torch.float16).T)


@pytest.mark.parametrize("M,N,K_", [(513, 1024, 784), (1000, 144, 256), (128, 4112, 64), (65, 272, 1040)])
def test_int8_layer_without_fp32_output(M, N, K_):
    """The TMA-store epilogues of the i8 kind: fp32 output, absmax-only pass, int8 requantising pass. All bit-exact:
    the int8 activations must equal what absmax -> quantise of the fp32 output gives."""
    rng = np.random.default_rng(43)
    a = rng.integers(-127, 128, (M, K_)).astype(np.int8)
    w = rng.integers(-127, 128, (N, K_)).astype(np.int8)
    ws = (rng.random(N) * 0.01 + 1e-3).astype(np.float32)
    b = (rng.standard_normal(N) * 0.05).astype(np.float32)
    a_scale = np.float32(0.0123)
    want = oracle.dequant_bias_act(oracle.gemm_i8(a, w), ws, a_scale, b, True)
    amax_want = oracle.absmax(want)
    q_want = oracle.quantize_i8(want, oracle.quant_scale(amax_want))
    A, W, WS, B = cu(a), cu(w), cu(ws), cu(b)
    amax = torch.zeros(1, device="cuda")
    out, _ = K.qlinear_i8(A, W, WS, a_scale=float(a_scale), bias=B, relu=True, out_absmax=amax)
    assert np.array_equal(out.cpu().numpy(), want)
    assert amax.item() == amax_want
    amax2 = torch.zeros(1, device="cuda")
    K.qlinear_i8(A, W, WS, a_scale=float(a_scale), bias=B, relu=True, want_out=False, out_absmax=amax2)
    assert amax2.item() == amax_want
    q = torch.full((M, N), 99, dtype=torch.int8, device="cuda")
    K.qlinear_i8(A, W, WS, a_scale=float(a_scale), bias=B, relu=True, out=q, out_absmax=amax2)
    assert np.array_equal(q.cpu().numpy(), q_want)
    assert K.device_error() == 0
    # and the stand-alone quantiser on a ReLU output (half zeros) and on values that sit on rounding boundaries
    assert np.array_equal(K.quantize_i8(out, absmax_dev=amax).cpu().numpy(), q_want)
    s = np.float32(0.37)
    ties = (np.arange(-130, 131, dtype=np.float32) + np.float32(0.5)) * s
    x = np.concatenate([ties, np.nextafter(ties, np.float32(np.inf)), np.nextafter(ties, np.float32(-np.inf)), np.zeros(7, np.float32)])
    x = np.resize(x, 4096).astype(np.float32)
    assert np.array_equal(K.quantize_i8(cu(x), scale=float(s)).cpu().numpy(), oracle.quantize_i8(x, s))


def test_int8_output_needs_wide_aligned_rows():
    a = torch.zeros((64, 64), dtype=torch.int8, device="cuda")
    w = torch.zeros((64, 64), dtype=torch.int8, device="cuda")
    ws = torch.ones(64, device="cuda")
    q = torch.zeros((64, 64), dtype=torch.int8, device="cuda")
    with pytest.raises(RuntimeError, match="more than 128 output channels"):
        K.qlinear_i8(a, w, ws, a_scale=1.0, out=q, out_absmax=torch.ones(1, device="cuda"))
    with pytest.raises(ValueError, match="device absmax"):
        K.qlinear_i8(a, w, ws, a_scale=1.0, out=q)


@pytest.mark.parametrize("shape_a,shape_b", [((3, 4), (4, 5)), ((5, 7), (7, 3)), ((2, 3, 4), (2, 4, 5)),   # tests/test_ops.py:257-274
                                             ((513, 300), (300, 1000)), ((4, 3, 130, 70), (4, 3, 70, 257)), ((6, 200, 64), (64, 96))])
def test_fp32_matmul_matches_the_cpu_path(shape_a, shape_b):
    """fp32 matmul (three tf32 products on the tensor cores) against the reference CPU matmul, at the reference tests' 1e-5."""
    rng = np.random.default_rng(44)
    a = rng.uniform(0.5, 0.9, shape_a).astype(np.float32)
    b = rng.uniform(0.5, 0.9, shape_b).astype(np.float32)
    want = np.matmul(a.astype(np.float64), b.astype(np.float64))
    got = K.matmul(cu(a), cu(b)).cpu().numpy()
    assert_close(got, want, 1e-5, 1e-5)
    if a.ndim == 2:
        assert_close(got, oracle.matmul_f32(a, b), 1e-5, 1e-5)
    # N(0,1) operands (sums that cancel), a transposed-view a, a column-major b and a bias + ReLU epilogue
    a2 = rng.standard_normal(shape_a[:-2] + (shape_a[-1], shape_a[-2])).astype(np.float32)
    b2 = rng.standard_normal(shape_b[:-2] + (shape_b[-1], shape_b[-2])).astype(np.float32)
    bias = rng.standard_normal(shape_b[-1]).astype(np.float32)
    A2, B2 = cu(a2).transpose(-2, -1), cu(b2).transpose(-2, -1)
    got2 = K.matmul(A2, B2, bias=cu(bias), act=1).cpu().numpy()
    at, bt = np.swapaxes(a2, -2, -1).astype(np.float64), np.swapaxes(b2, -2, -1).astype(np.float64)
    ref2 = np.maximum(np.matmul(at, bt) + bias, 0)
    # componentwise bound relative to sum_k |a_ik b_kj|: the tensor core truncates when it accumulates, so the error is
    # a few 1e-6 of that sum rather than fp32's sqrt(K) * 6e-8; 1e-5 is the classical fp32 bound for K = 170
    bound = 1e-5 * np.matmul(np.abs(at), np.abs(bt)) + 1e-6
    assert (np.abs(got2 - ref2) <= bound).all(), float((np.abs(got2 - ref2) / bound).max())
    assert K.device_error() == 0


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_half_matmul_accepts_any_view(dt):
    """Plain row-major [K, N] b, a transposed a, a contraction length that is not a multiple of 8, sliced bases: the
    operands that the tensor-map loads cannot read in place are re-laid-out first (the reference contiguises them)."""
    g = torch.Generator(device="cuda").manual_seed(9)
    r = lambda *s_: (torch.randn(s_, generator=g, device="cuda") * 0.5).to(dt)  # noqa: E731
    cases = [
        (r(200, 300), r(300, 130)),                                  # row-major b
        (r(77, 61), r(61, 45)),                                      # K = 61: pitches of 122 bytes
        (r(96, 40).T, r(96, 72)),                                    # a is a transposed view
        (r(3, 50, 64), r(3, 64, 33)),                                # batched, row-major b
        (r(2, 3, 40, 24)[..., 1:], r(2, 3, 24, 16)[..., 1:, :]),     # sliced: unaligned bases, K = 23
        (r(4, 30, 48), r(48, 20)),                                   # shared row-major weight
    ]
    for a, b in cases:
        got = K.matmul(a, b).float()
        want = a.float() @ b.float()
        tol = 2e-2 * max(1.0, want.abs().max().item())
        assert got.shape == want.shape and (got - want).abs().max().item() <= tol, (tuple(a.shape), tuple(b.shape))
    assert K.device_error() == 0


@pytest.mark.parametrize("shape_a,shape_b", [((3, 4), (4, 5)), ((5, 7), (7, 3)), ((2, 3, 4), (2, 4, 5)), ((130, 70), (70, 257)),
                                             ((2, 3, 65, 33), (2, 3, 33, 70)), ((4, 50, 16), (16, 9))])
def test_fp64_matmul(shape_a, shape_b):
    """tests/test_ops.py:257-274 runs matmul in float64 too: the fp64-unit kernel, compared at the reference tests' 1e-5 (it is
    accurate to rounding) on plain, transposed-view and batched operands, with a bias + ReLU + residual epilogue."""
    rng = np.random.default_rng(45)
    a = rng.uniform(0.5, 0.9, shape_a)
    b = rng.uniform(0.5, 0.9, shape_b)
    got = K.matmul(cu(a), cu(b)).cpu().numpy()
    np.testing.assert_allclose(got, np.matmul(a, b), rtol=1e-12, atol=1e-12)
    a2 = rng.standard_normal(shape_a[:-2] + (shape_a[-1], shape_a[-2]))
    bias = rng.standard_normal(shape_b[-1])
    res = rng.standard_normal(np.matmul(a, b).shape)
    got2 = K.matmul(cu(a2).transpose(-2, -1), cu(b), bias=cu(bias), act=1, residual=cu(res), alpha=0.5).cpu().numpy()
    want2 = np.maximum(np.matmul(np.swapaxes(a2, -2, -1), b) * 0.5 + bias, 0) + res
    np.testing.assert_allclose(got2, want2, rtol=1e-11, atol=1e-11)


class one_cta_kernel:
    """Keeps the GEMMs inside the block on the one-CTA kernel (pgb_gemm_pair_mode)."""

    def __enter__(self):
        self.old = K.gemm_pair_mode(0)

    def __exit__(self, *exc):
        K.gemm_pair_mode(self.old)


def both_kernels(fn, pair_mode=1):
    """fn() through the CTA-pair kernel and through the one-CTA kernel: same MMAs in the same order, same epilogue,
    so the results must be the same bits. pair_mode 3 sends int8 layers to the pair kernel too (they default to the
    one-CTA kernel, which measured faster for them)."""
    old = K.gemm_pair_mode(pair_mode)
    try:
        got = fn()
    finally:
        K.gemm_pair_mode(old)
    assert K.device_error() == 0
    with one_cta_kernel():
        want = fn()
    assert K.device_error() == 0
    got = got if isinstance(got, (tuple, list)) else (got,)
    want = want if isinstance(want, (tuple, list)) else (want,)
    for g_, w_ in zip(got, want):
        assert torch.equal(g_, w_)
    return got


@pytest.mark.parametrize("M,N,K_", [(256, 256, 128), (512, 2576, 1040), (4096, 1024, 784), (256 * 75, 768, 256)])
def test_int8_layers_same_bits_with_and_without_the_pair_switch(M, N, K_):
    g = torch.Generator(device="cuda").manual_seed(31)
    a = torch.randint(-127, 128, (M, K_), generator=g, device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (N, K_), generator=g, device="cuda", dtype=torch.int8)
    ws = torch.rand(N, generator=g, device="cuda") * 0.01 + 0.001
    b = torch.randn(N, generator=g, device="cuda")
    out, = both_kernels(lambda: K.qlinear_i8(a, w, ws, a_scale=0.02, bias=b, relu=True)[0], pair_mode=3)
    acc = a[:300].cpu().numpy().astype(np.int32) @ w.cpu().numpy().astype(np.int32).T  # int32 accumulators on the CPU
    want = np.maximum(acc.astype(np.float32) * (np.float32(0.02) * ws.cpu().numpy())[None, :] + b.cpu().numpy()[None, :], 0)
    assert np.array_equal(out[:300].cpu().numpy(), want)
    # absmax-only pass, then the int8-requantising pass
    def two_pass():
        am = torch.zeros(1, device="cuda")
        K.qlinear_i8(a, w, ws, a_scale=0.02, bias=b, relu=True, want_out=False, out_absmax=am)
        q = torch.empty((M, N), dtype=torch.int8, device="cuda")
        K.qlinear_i8(a, w, ws, a_scale=0.02, bias=b, relu=True, out=q, out_absmax=am)
        return am, q
    am, q = both_kernels(two_pass, pair_mode=3)
    assert float(am) == float(out.max())


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_cta_pair_kernel_16bit_matches_the_one_cta_kernel(dt):
    g = torch.Generator(device="cuda").manual_seed(32)
    x = (torch.randn((2, 1024, 768), generator=g, device="cuda") * 0.5).to(dt)
    wt = (torch.randn((3072, 768), generator=g, device="cuda") * 0.02).to(dt)
    b = (torch.randn(3072, generator=g, device="cuda") * 0.02).to(dt)
    y, = both_kernels(lambda: K.matmul(x, wt.T, bias=b, act=2))
    z = x.float() @ wt.float().T + b.float()
    ref = 0.5 * z * (1 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
    assert_close(y.float().cpu().numpy(), ref.cpu().numpy(), 2e-2, 2e-3)
    wt2 = (torch.randn((768, 3072), generator=g, device="cuda") * 0.02).to(dt)
    res = torch.randn((2, 1024, 768), generator=g, device="cuda").to(dt)
    both_kernels(lambda: K.matmul(y, wt2.T, residual=res))
    both_kernels(lambda: K.matmul(x, wt.T, out_dtype=torch.float32))
    # ragged right edge: the peer CTA's half of the last tile lies wholly beyond N
    wv = (torch.randn((2568, 768), generator=g, device="cuda") * 0.02).to(dt)
    lg, = both_kernels(lambda: K.matmul(x, wv.T))
    assert_close(lg.float().cpu().numpy(), (x.float() @ wv.float().T).cpu().numpy(), 2e-2, 2e-3)
    # batched operands (scores of 2 x 12 heads read in place from packed buffers)
    q = torch.randn((2, 12, 512, 64), generator=g, device="cuda").to(dt)
    k = torch.randn((2, 12, 512, 64), generator=g, device="cuda").to(dt)
    both_kernels(lambda: K.matmul(q, k.transpose(-2, -1), out_dtype=torch.float32))


def test_cta_pair_kernel_fp32_split_matmul():
    g = torch.Generator(device="cuda").manual_seed(33)
    a = torch.randn((1024, 520), generator=g, device="cuda")
    b = torch.randn((520, 384), generator=g, device="cuda")
    c, = both_kernels(lambda: K.matmul(a, b))
    bound = 1e-5 * (a.abs().double() @ b.abs().double())
    assert bool(((c.double() - a.double() @ b.double()).abs() <= bound).all())


def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable():
    """Failure detection without a fault: the next GEMM's producer is told to load nothing and every wait to give up
    after 1024 polls. The kernel must record who gave up, free its tensor memory and return; while the error word is
    set further launches do nothing; once the host has read and cleared it the same GEMM is bit-exact again."""
    g = torch.Generator(device="cuda").manual_seed(41)
    a = torch.randint(-127, 128, (128, 256), generator=g, device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (128, 256), generator=g, device="cuda", dtype=torch.int8)
    ws = torch.rand(128, generator=g, device="cuda") * 0.01 + 0.001
    want = a.cpu().numpy().astype(np.int32) @ w.cpu().numpy().astype(np.int32).T
    _, acc = K.qlinear_i8(a, w, ws, a_scale=0.02, want_acc=True, want_out=False)
    assert np.array_equal(acc.cpu().numpy(), want) and K.device_error() == 0
    K.gemm_wait_drill(1024, skip_loads=True)
    _, acc = K.qlinear_i8(a, w, ws, a_scale=0.02, want_acc=True, want_out=False)  # one 128 x 128 tile, block 0
    torch.cuda.synchronize()  # returns: nothing hangs
    code = C.c_int(0)
    st = L.lib().pgb_device_error(C.byref(code), 0)
    assert st == L.ERR_TIMEOUT and "wait ran out" in L.lib().pgb_last_error().decode()
    assert (code.value >> 16) in (2, 3) and (code.value & 0xffff) == 0  # the MMA issuer (or the epilogue behind it) of block 0
    # the word is still set: the next launch returns at once and leaves its output alone
    sentinel = torch.full((128, 128), 7.0, device="cuda")
    K.qlinear_i8(a, w, ws, a_scale=0.02, out=sentinel)
    torch.cuda.synchronize()
    assert (sentinel == 7).all()
    assert K.device_error(reset=True) == code.value
    assert K.device_error() == 0
    # the drill applied to one launch only, and the device is as good as before
    _, acc = K.qlinear_i8(a, w, ws, a_scale=0.02, want_acc=True, want_out=False)
    assert np.array_equal(acc.cpu().numpy(), want) and K.device_error() == 0
    x = torch.randn((256, 512), generator=g, device="cuda").half()
    y = torch.randn((384, 512), generator=g, device="cuda").half()
    assert_close(K.matmul(x, y.T).float().cpu().numpy(), (x.float() @ y.float().T).cpu().numpy(), 2e-2, 2e-2)
