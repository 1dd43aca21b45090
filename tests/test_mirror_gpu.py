"""The host-side mirror (lazy Tensor, jit) against torch CPU, in the form of the reference's
own tests: `_compare_fn_with_torch` with seed 1337 and uniform[0.5,0.9) inputs
(tests/test_ops.py:20-80), jit-vs-eager (tests/test_compile.py:26-57), composites
(tests/test_high_level_ops.py:100-121, 354-367, 529-544)."""
import numpy as np
import pytest
import torch

from helpers import assert_close, ref_test_inputs
from pequegrad_b200 import _lib as L
from pequegrad_b200 import fuser
from pequegrad_b200 import tensor as pg

pytestmark = pytest.mark.gpu


def _compare_fn_with_torch(shapes, pg_fn, torch_fn=None, tol=1e-5, dtype=np.float32, jit=False):
    torch_fn = torch_fn or pg_fn
    arrs = ref_test_inputs(shapes, dtype)
    want = torch_fn(*[torch.from_numpy(a) for a in arrs])
    fn = fuser.jit(pg_fn) if jit else pg_fn
    got = fn(*[pg.Tensor(a) for a in arrs])
    assert list(got.shape) == list(want.shape)
    assert_close(got.numpy(), want.numpy().astype(got.numpy().dtype), tol, tol)


def launches(fn):
    before = L.lib().pgb_launch_count()
    fn()
    return L.lib().pgb_launch_count() - before


@pytest.mark.parametrize("jit", [False, True])
@pytest.mark.parametrize("shape", [(2, 3), (3, 4), (4, 5)])
def test_binary_unary_and_reducers_like_the_reference_tests(shape, jit):
    ops = [(lambda x, y: x + y, None), (lambda x, y: x * y, None), (lambda x, y: x - y, None), (lambda x, y: x / y, None),
           (lambda x, y: x ** y, None), (lambda x, y: pg.max(x, y) if isinstance(x, pg.Tensor) else torch.max(x, y), None)]
    for f, _ in ops:
        _compare_fn_with_torch([shape, shape], f, jit=jit)
    # comparisons return 0/1 in the operand dtype (csrc/cuda/binary.cu:24-41)
    _compare_fn_with_torch([shape, shape], lambda x, y: x > y, lambda x, y: (x > y).float(), jit=jit)
    _compare_fn_with_torch([shape, shape, shape], lambda a, b, c: (a * b + c) * b, jit=jit)  # tests/test_ops.py:96-104
    _compare_fn_with_torch([shape], lambda x: x.exp() if isinstance(x, pg.Tensor) else torch.exp(x), jit=jit)
    _compare_fn_with_torch([shape], lambda x: x.log() if isinstance(x, pg.Tensor) else torch.log(x), jit=jit)
    for axes in [(0, 1), (1, 0), (0,), (1,), -1, (-1, -2), None]:
        for kd in (True, False):
            tdim = list(range(len(shape))) if axes is None else axes
            _compare_fn_with_torch([shape], lambda x: x.sum(axes, kd), lambda x: torch.sum(x, dim=tdim, keepdim=kd), jit=jit)
            _compare_fn_with_torch([shape], lambda x: x.mean(axes, kd), lambda x: torch.mean(x, dim=tdim, keepdim=kd), jit=jit)
            _compare_fn_with_torch([shape], lambda x: x.max_reduce(axes, kd), lambda x: torch.amax(x, dim=tdim, keepdim=kd), jit=jit)


def test_permute_broadcast_where_astype():
    _compare_fn_with_torch([(2, 3, 4)], lambda x: pg.permute(x, (2, 0, 1)) * 2.0 if isinstance(x, pg.Tensor) else x.permute(2, 0, 1) * 2.0)
    _compare_fn_with_torch([(4, 3, 2), (2,)], lambda x, y: x * y + 5.0, jit=True)  # tests/test_compile.py broadcast case
    _compare_fn_with_torch([(3, 4), (3, 4), (3, 4)], lambda c, a, b: pg.where(c > 0.7, a, b) if isinstance(c, pg.Tensor) else torch.where(c > 0.7, a, b))
    x = ref_test_inputs([(5, 6)], np.float32)[0] * 10
    assert np.array_equal(pg.Tensor(x).astype(pg.int32).numpy(), x.astype(np.int32))
    assert pg.Tensor(x).reshape(6, 5).permute(1, 0).reshape(30).numpy().tolist() == x.reshape(6, 5).T.reshape(30).tolist()
    with pytest.raises(ValueError):
        pg.Tensor(x) + pg.Tensor(x.astype(np.float64))


def test_readme_fusion_is_one_kernel_and_matches_eager():
    # README.md:59-63; eager = fill, fill, add, add, sum, mul kernels; jit = one fused reduce kernel
    rng = np.random.default_rng(1)
    x = pg.Tensor(rng.random((1000, 20, 100), dtype=np.float32))
    y = pg.Tensor(rng.random((1000, 100, 20), dtype=np.float32))

    def f(x, y):
        return ((pg.permute(x, (0, 2, 1)) + 2) + y).sum(2) * 3
    out = {}
    n_eager = launches(lambda: out.setdefault("e", f(x, y).numpy()))
    n_jit = launches(lambda: out.setdefault("j", fuser.jit(f)(x, y).numpy()))
    assert n_jit == 1 and n_eager >= 4
    want = ((x.numpy().transpose(0, 2, 1).astype(np.float64) + 2 + y.numpy()).sum(2) * 3)
    assert_close(out["j"], want, 1e-5)
    assert_close(out["e"], out["j"], 1e-6)


def test_long_reduce_with_prologue_and_epilogue_fuses():
    # the reference refuses to fuse reduces of >= 1024 elements (csrc/compiler/scheduler.cpp:55-61)
    rng = np.random.default_rng(2)
    a = rng.standard_normal((256, 4096)).astype(np.float32)
    x = pg.Tensor(a)
    for ax in (0, 1):
        f = lambda t: ((t * 1.5 + 0.25).mean(ax)).exp()  # noqa: E731
        got = {}
        assert launches(lambda: got.setdefault("v", fuser.jit(f)(x).numpy())) <= 2  # the kernel (+ finish kernel if split)
        assert_close(got["v"], np.exp((a.astype(np.float64) * 1.5 + 0.25).mean(ax)), 1e-5)
    assert np.array_equal(pg.argmax(x, 1).numpy(), a.argmax(1))


def test_composites_eager_and_jit():
    # layer_norm shapes and tolerance of tests/test_high_level_ops.py:100-121
    for shape, ns in [((2, 3, 4), (4,)), ((2, 3, 4), (3, 4)), ((5, 10), (10,)), ((64, 768), (768,))]:
        (x,) = ref_test_inputs([shape], np.float32)
        want = torch.nn.functional.layer_norm(torch.from_numpy(x), ns, eps=1e-5).numpy()
        assert_close(pg.layer_norm(pg.Tensor(x), ns).numpy(), want, 1e-4)
        assert_close(fuser.jit(lambda t: pg.layer_norm(t, ns))(pg.Tensor(x)).numpy(), want, 1e-4)
    (x,) = ref_test_inputs([(8, 1024)], np.float32)
    want = torch.softmax(torch.from_numpy(x), -1).numpy()
    assert_close(pg.softmax(pg.Tensor(x)).numpy(), want, 1e-5)
    n = launches(lambda: assert_close(fuser.jit(pg.softmax)(pg.Tensor(x)).numpy(), want, 1e-5))
    assert n == 1
    (x,) = ref_test_inputs([(2, 3)], np.float32)
    want = torch.nn.functional.gelu(torch.from_numpy(x), approximate="tanh").numpy()
    assert_close(pg.gelu(pg.Tensor(x)).numpy(), want, 1e-5)
    assert_close(fuser.jit(pg.gelu)(pg.Tensor(x)).numpy(), want, 1e-5)


def test_matmul_half_float_double_and_reference_error_for_int32():
    rng = np.random.default_rng(3)
    a = rng.standard_normal((5, 64, 128)).astype(np.float16)
    w = rng.standard_normal((128, 96)).astype(np.float16)
    got = (pg.Tensor(a) @ pg.Tensor(w)).numpy().astype(np.float32)
    want = a.astype(np.float32) @ w.astype(np.float32)
    assert_close(got, want, 2e-2, 2e-2 * float(np.abs(want).max()))
    b = rng.standard_normal((5, 128, 32)).astype(np.float16)
    got = (pg.Tensor(a) @ pg.Tensor(b)).numpy().astype(np.float32)
    want = a.astype(np.float32) @ b.astype(np.float32)
    assert_close(got, want, 2e-2, 2e-2 * float(np.abs(want).max()))
    # fp32 runs on the tensor cores as three tf32 products per term
    a32, w32 = a.astype(np.float32), w.astype(np.float32)
    got = (pg.Tensor(a32) @ pg.Tensor(w32)).numpy()
    want = a32.astype(np.float64) @ w32.astype(np.float64)
    assert np.abs(got - want).max() <= 1e-5 * float((np.abs(a32) @ np.abs(w32)).max())
    a64, w64 = a.astype(np.float64), w.astype(np.float64)
    np.testing.assert_allclose((pg.Tensor(a64) @ pg.Tensor(w64)).numpy(), a64 @ w64, rtol=1e-12, atol=1e-12)
    with pytest.raises(RuntimeError, match="matmul_cuda not implemented for int32"):
        (pg.Tensor(a.astype(np.int32)) @ pg.Tensor(w.astype(np.int32))).eval()


def test_fused_linear_pattern_is_one_gemm():
    """`recursive_fused_linear` (FusedLinearBiasAct, csrc/cuda/other.cu:19-166): under jit, act(x @ w + b) is ONE
    GEMM launch with the bias and the activation in its epilogue; eager runs matmul, add and max as separate kernels."""
    rng = np.random.default_rng(11)
    x = (rng.standard_normal((256, 128)) * 0.5).astype(np.float16)
    wt = (rng.standard_normal((192, 128)) * 0.1).astype(np.float16)  # the weight as [N, K]: its transposed view is read in place
    b = rng.standard_normal(192).astype(np.float16)
    pre = x.astype(np.float32) @ wt.astype(np.float32).T + b.astype(np.float32)
    wt_d = pg.Tensor(wt)
    for f, want in [(lambda t, w, c: (t @ w + c).relu(), np.maximum(pre, 0)),
                    (lambda t, w, c: pg.gelu(t @ w + c), torch.nn.functional.gelu(torch.from_numpy(pre), approximate="tanh").numpy()),
                    (lambda t, w, c: t @ w + c, pre)]:
        eager = f(pg.Tensor(x), wt_d.transpose(0, 1), pg.Tensor(b)).numpy().astype(np.float32)
        out = {}
        n = launches(lambda: out.setdefault("v", fuser.jit(f)(pg.Tensor(x), wt_d.transpose(0, 1), pg.Tensor(b)).numpy()))
        assert n == 1
        assert_close(out["v"].astype(np.float32), want, 2e-2, 2e-2 * float(np.abs(want).max()))
        assert_close(eager, want, 2e-2, 2e-2 * float(np.abs(want).max()))
    # inside a larger region the bias and the activation still ride in the GEMM: GEMM + one elementwise kernel
    g = lambda t, w, c: (t @ w + c).relu() * 2.0 + 1.0  # noqa: E731
    n = launches(lambda: out.setdefault("g", fuser.jit(g)(pg.Tensor(x), wt_d.transpose(0, 1), pg.Tensor(b)).numpy()))
    assert n == 2
    assert_close(out["g"].astype(np.float32), np.maximum(pre, 0) * 2 + 1, 2e-2, 2e-2 * float(np.abs(pre).max()))
    # fp32: bias + ReLU go into the tf32-split GEMM's epilogue too (the exact-chain GELU stays a kernel of its own)
    x32, w32, b32 = x.astype(np.float32), wt.astype(np.float32).T.copy(), b.astype(np.float32)
    got = fuser.jit(lambda t, w, c: (t @ w + c).relu())(pg.Tensor(x32), pg.Tensor(w32), pg.Tensor(b32)).numpy()
    assert_close(got, np.maximum(x32.astype(np.float64) @ w32 + b32, 0), 1e-5, 1e-5 * float(np.abs(pre).max()))
    got = fuser.jit(lambda t, w, c: pg.gelu(t @ w + c))(pg.Tensor(x32), pg.Tensor(w32), pg.Tensor(b32)).numpy()
    assert_close(got, torch.nn.functional.gelu(torch.from_numpy(x32 @ w32 + b32), approximate="tanh").numpy(), 1e-5, 1e-5)


def test_amp_runs_fp32_matmuls_as_fp16_gemms_with_fp32_results():
    """pequegrad/transforms/automatic_mixed_precision.py:37-146 (`matmul_amp`, `bias_relu_add_amp`, the astype pairs);
    the reference has no test of its own for amp (examples/amp_fc.py only times it), so the fp32 function is the
    yardstick, at the 16-bit tolerance."""
    rng = np.random.default_rng(12)
    x = (rng.standard_normal((4, 128, 256)) * 0.5).astype(np.float32)
    w1 = (rng.standard_normal((256, 512)) * 0.05).astype(np.float32)
    b1 = rng.standard_normal(512).astype(np.float32)
    w2 = (rng.standard_normal((512, 64)) * 0.05).astype(np.float32)

    def mlp(t, a, c, d):
        return (t @ a + c).relu() @ d

    want = np.maximum(x @ w1 + b1, 0) @ w2
    out = {}
    got = fuser.amp(mlp)(*(pg.Tensor(t) for t in (x, w1, b1, w2)))
    assert got.dtype == pg.float32  # results come back as fp32
    n = launches(lambda: got.numpy())
    assert n == 6  # two casts + GEMM (bias and ReLU in its epilogue), twice
    assert_close(got.numpy(), want, 2e-2, 2e-2 * float(np.abs(want).max()))
    # exactly the fp16-rounded operands with an fp32 accumulator: far tighter than fp16 accumulation would allow
    h16 = np.maximum(x.astype(np.float16).astype(np.float64) @ w1.astype(np.float16).astype(np.float64) + b1, 0).astype(np.float32)
    want16 = h16.astype(np.float16).astype(np.float64) @ w2.astype(np.float16).astype(np.float64)
    assert_close(got.numpy(), want16, 1e-4, 1e-4 * float(np.abs(want16).max()))
    # astype pairs vanish under amp (the value keeps its original precision): no kernel at all
    t16 = pg.Tensor(x.astype(np.float16))
    back = fuser.amp(lambda t: t.astype(pg.float32).astype(pg.float16))(t16)
    assert launches(lambda: back.eval()) == 0 and np.array_equal(back.numpy(), x.astype(np.float16))
    # non-fp32 matmuls are left alone
    assert fuser.amp(lambda a, c: a @ c)(t16, pg.Tensor(w1.astype(np.float16))).dtype == pg.float16


def test_sdpa_composite_and_its_fused_form():
    """pequegrad/ops.py:792-818 and tests/test_high_level_ops.py:623-639 (sdpa with a tril mask): eager = the composite
    (matmul, where, softmax, matmul), under jit without a mask tensor = the one-kernel attention."""
    rng = np.random.default_rng(8)
    q, k, v = (rng.standard_normal((2, 3, 96, 64)).astype(np.float16) for _ in range(3))
    tril = np.tril(np.ones((96, 96), dtype=bool))
    s = (q.astype(np.float32) @ k.astype(np.float32).transpose(0, 1, 3, 2)) / 8.0

    def ref(masked):
        z = np.where(tril, s, -1e9) if masked else s
        e = np.exp(z - z.max(-1, keepdims=True))
        return (e / e.sum(-1, keepdims=True)) @ v.astype(np.float32)

    mask = pg.Tensor(np.broadcast_to(tril, (2, 3, 96, 96)).astype(np.float16)) > 0.5
    eager = pg.scaled_dot_product_attention(pg.Tensor(q), pg.Tensor(k), pg.Tensor(v), mask=mask).numpy().astype(np.float32)
    assert_close(eager, ref(True), 2e-2, 2e-2)
    before = L.lib().pgb_launch_count()
    fused = fuser.jit(lambda a, b, c: pg.scaled_dot_product_attention(a, b, c, is_causal=True))(pg.Tensor(q), pg.Tensor(k), pg.Tensor(v))
    got = fused.numpy().astype(np.float32)
    assert L.lib().pgb_launch_count() - before == 1  # one kernel
    assert_close(got, ref(True), 2e-2, 2e-2)
    full = fuser.jit(lambda a, b, c: pg.scaled_dot_product_attention(a, b, c))(pg.Tensor(q), pg.Tensor(k), pg.Tensor(v)).numpy().astype(np.float32)
    assert_close(full, ref(False), 2e-2, 2e-2)
    with pytest.raises(NotImplementedError, match="use a mask"):
        pg.scaled_dot_product_attention(pg.Tensor(q), pg.Tensor(k), pg.Tensor(v), is_causal=True)


def test_multi_reduce_chains_written_from_primitives_are_one_kernel():
    """The reference's scheduler allows one reduce per fused kernel (csrc/compiler/scheduler.cpp:62-66), so a softmax or
    a LayerNorm written out by hand costs a kernel per reduce there. Here the fuser recognises both chains in the graph:
    one launch each, same numbers as eager."""
    (x,) = ref_test_inputs([(64, 1024)], np.float32)
    x = (x - 0.7) * 10

    def my_softmax(t):
        m = t.max_reduce(-1, True)
        e = (t - m).exp()
        return e / e.sum(-1, True)

    want = torch.softmax(torch.from_numpy(x), -1).numpy()
    out = {}
    assert launches(lambda: out.setdefault("j", fuser.jit(my_softmax)(pg.Tensor(x)).numpy())) == 1
    assert launches(lambda: out.setdefault("e", my_softmax(pg.Tensor(x)).numpy())) >= 5
    assert_close(out["j"], want, 1e-5)
    assert_close(out["e"], want, 1e-5)
    # through a permuted view: the rows are made contiguous by one copy kernel, then the row kernel
    xt = np.ascontiguousarray(x.T)
    n = launches(lambda: out.setdefault("p", fuser.jit(lambda t: my_softmax(t.permute(1, 0)))(pg.Tensor(xt)).numpy()))
    assert n == 2
    assert_close(out["p"], want, 1e-5)

    w, b = ref_test_inputs([(1024,), (1024,)], np.float32)

    def my_layernorm(t, g, c):
        mu = t.mean(-1, True)
        var = ((t - mu) ** 2.0).sum(-1, True) / 1024.0
        return (t - mu) / (var + 1e-5) ** 0.5 * g + c

    want = torch.nn.functional.layer_norm(torch.from_numpy(x), (1024,), torch.from_numpy(w), torch.from_numpy(b), 1e-5).numpy()
    assert launches(lambda: out.setdefault("lj", fuser.jit(my_layernorm)(pg.Tensor(x), pg.Tensor(w), pg.Tensor(b)).numpy())) == 1
    assert launches(lambda: out.setdefault("le", my_layernorm(pg.Tensor(x), pg.Tensor(w), pg.Tensor(b)).numpy())) >= 8
    assert_close(out["lj"], want, 1e-4)
    assert_close(out["le"], want, 1e-4)
    # not LayerNorm's variance (divided by n - 1): stays a sequence of fused regions, and still agrees with eager
    def other(t):
        mu = t.mean(-1, True)
        return (t - mu) / (((t - mu) ** 2.0).sum(-1, True) / 1023.0 + 1e-5) ** 0.5
    assert_close(fuser.jit(other)(pg.Tensor(x)).numpy(), other(pg.Tensor(x)).numpy(), 1e-5)


def test_regions_larger_than_the_kernel_limits_are_split_not_refused():
    """A fused kernel takes at most 6 operands and 32 instructions. Larger expressions are cut into several regions;
    jit must agree with eager on them."""
    arrs = ref_test_inputs([(33, 40)] * 10, np.float32)

    def ten_sum(*ts):
        acc = ts[0]
        for t in ts[1:]:
            acc = acc + t * 0.5
        return acc

    got = {}
    n = launches(lambda: got.setdefault("v", fuser.jit(ten_sum)(*[pg.Tensor(a) for a in arrs]).numpy()))
    assert 2 <= n <= 6  # 10 operands and 37 instructions: at least two regions; eager would be 27 kernels
    assert_close(got["v"], ten_sum(*[pg.Tensor(a) for a in arrs]).numpy(), 1e-6)
    assert_close(got["v"], arrs[0] + 0.5 * np.sum(arrs[1:], axis=0), 1e-5)

    def long_chain(t):
        for i in range(40):
            t = (t * 0.9 + 0.1) if i % 3 else (t + 1.0).log()
        return t

    n = launches(lambda: got.setdefault("c", fuser.jit(long_chain)(pg.Tensor(arrs[0])).numpy()))
    assert 6 <= n <= 12  # about 146 instructions in regions of at most 28; eager would be 120 kernels
    assert_close(got["c"], long_chain(pg.Tensor(arrs[0])).numpy(), 1e-5)
    # the same with a reduce on top: prologue and epilogue each cut where needed
    def reduced(*ts):
        return (ten_sum(*ts).sum(1) * 2.0).exp()
    assert_close(fuser.jit(reduced)(*[pg.Tensor(a * 0.01) for a in arrs]).numpy(), reduced(*[pg.Tensor(a * 0.01) for a in arrs]).numpy(), 1e-5)


def test_outputs_of_one_call_share_a_kernel():
    """Sibling outputs of a fused region (csrc/compiler/scheduler.cpp:229-256, csrc/compiler/ir.cpp:667-675): the
    elementwise results of one traced call come out of ONE multi-output kernel, common subexpressions computed once."""
    a, b, c = ref_test_inputs([(17, 130)] * 3, np.float32)

    def f(x, y, z):
        t = x * y + z
        return t, t * 2.0 - x, (y > z), (x - y).astype(pg.float16)

    outs = fuser.jit(f)(pg.Tensor(a), pg.Tensor(b), pg.Tensor(c))
    n = launches(lambda: [o.eval() for o in outs])
    assert n == 1
    t = a * b + c
    assert_close(outs[0].numpy(), t, 1e-6)
    assert_close(outs[1].numpy(), t * 2 - a, 1e-6)
    assert np.array_equal(outs[2].numpy(), (b > c).astype(np.float32))
    assert outs[3].numpy().dtype == np.float16 and np.array_equal(outs[3].numpy(), (a - b).astype(np.float16))
    # an output with a reduce, or of another shape, is a kernel of its own
    def g(x, y):
        return x + y, (x * y).sum(1), x.permute(1, 0) * 2.0
    outs = fuser.jit(g)(pg.Tensor(a), pg.Tensor(b))
    assert launches(lambda: [o.eval() for o in outs]) == 3
    assert_close(outs[1].numpy(), (a * b).sum(1), 1e-5)
    assert_close(outs[2].numpy(), a.T * 2, 1e-6)
