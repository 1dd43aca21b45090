"""The two model-level workloads of the path, through the kernels: the int8 quantized MLP
(examples/quantized_mlp.py) and the GPT-2 forward (examples/gpt2.py), against CPU restatements."""
import numpy as np
import pytest
import torch

import oracle
from helpers import assert_close
from pequegrad_b200 import gpt2 as G
from pequegrad_b200 import kernels as K
from pequegrad_b200.qmlp import QuantizedMLP, quantize_weight

pytestmark = pytest.mark.gpu


def test_quantized_mlp_class_matches_the_oracle_pipeline():
    rng = np.random.default_rng(3)
    dims = [784, 1024, 1024, 10]
    Ws = [(rng.standard_normal((dims[i], dims[i + 1])) * 0.05).astype(np.float32) for i in range(3)]
    bs = [(rng.standard_normal(dims[i + 1]) * 0.05).astype(np.float32) for i in range(3)]
    X = rng.random((1500, 784), dtype=np.float32)
    for W in Ws:  # the device-side weight preparation is the oracle's
        q, s = quantize_weight(W)
        q2, s2 = oracle.quantize_weight_per_channel(W)
        assert np.array_equal(q, q2) and np.array_equal(s, s2)
    mlp = QuantizedMLP(Ws, bs)
    out, kept = mlp.forward(torch.from_numpy(X).cuda(), keep=True)
    out = out.clone()  # the model reuses its buffers
    h = X
    for i in range(3):
        wq, wsc = oracle.quantize_weight_per_channel(Ws[i])
        sx = oracle.quant_scale(oracle.absmax(h))
        xq = oracle.quantize_i8(h, sx)
        assert np.array_equal(kept[i][0].cpu().numpy(), xq), f"layer {i} int8 activations"
        h = oracle.dequant_bias_act(oracle.gemm_i8(xq, wq), wsc, sx, bs[i], relu=i < 2)
        assert_close(kept[i][1].cpu().numpy(), h, 1e-5, 1e-6, f"layer {i} output")
    assert K.device_error() == 0
    # the same batch, rows reversed, through the route that never writes the hidden fp32 activations (absmax-only GEMM pass,
    # then a GEMM pass that stores int8): same accumulators, same arithmetic, so the logits are the same bits
    out2 = mlp.forward(torch.from_numpy(X[::-1].copy()).cuda())
    assert torch.equal(out2.flip(0), out)
    assert K.device_error() == 0


def test_quantized_mlp_at_the_configured_batch_of_65536_rows():
    """The benchmark's batch: 65536 x 784 uniform[0,1). Rows are independent given the per-tensor scales, so slabs of
    the full-size run (first, middle, last 256 rows) are compared with the oracle pipeline fed the run's own
    absmax values; the absmax values themselves are checked against the whole tensors."""
    from pequegrad_b200.workloads import mlp_weights
    Ws, bs = mlp_weights()
    g = torch.Generator(device="cuda").manual_seed(3)
    X = torch.rand((65536, 784), generator=g, device="cuda")
    mlp = QuantizedMLP(Ws, bs)
    out, kept = mlp.forward(X, keep=True)
    out = out.clone()
    amax = mlp._buffers(65536, X.device)["amax"].cpu().numpy()
    assert amax[0] == float(X.abs().max())
    for i in range(2):  # max |relu output| of the whole batch, folded in by the GEMM epilogues
        assert amax[i + 1] == float(kept[i][1].abs().max()), f"absmax of layer {i}'s output"
    prep = [oracle.quantize_weight_per_channel(W) for W in Ws]
    for lo in (0, 32768 - 128, 65536 - 256):
        h = X[lo:lo + 256].cpu().numpy()
        for i in range(3):
            sx = oracle.quant_scale(amax[i])
            xq = oracle.quantize_i8(h, sx)
            assert np.array_equal(kept[i][0][lo:lo + 256].cpu().numpy(), xq), f"rows {lo}: layer {i} int8 activations"
            h = oracle.dequant_bias_act(oracle.gemm_i8(xq, prep[i][0]), prep[i][1], sx, bs[i], relu=i < 2)
            assert_close(kept[i][1][lo:lo + 256].cpu().numpy(), h, 1e-5, 1e-6, f"rows {lo}: layer {i} output")
    # the route the benchmark runs (hidden fp32 activations never written) gives the same logits, bit for bit
    assert torch.equal(mlp.forward(X), out)
    # and so does any split of the rows, because the absmax is combined over the shards
    for parts in (2, 8):
        outs = mlp.forward_sharded(list(X.chunk(parts, 0)))
        assert torch.equal(torch.cat(outs, 0), out), f"{parts} row shards"
    assert K.device_error() == 0


@pytest.mark.parametrize("cfg,B,T", [(G.GPT2Config(n_layer=2, n_head=2, n_embd=128, vocab_size=1000, block_size=64), 3, 64),
                                     (G.GPT2Config(n_layer=3, n_head=4, n_embd=256, vocab_size=517, block_size=128), 2, 100),
                                     (G.GPT2Config(n_layer=2, n_head=4, n_embd=128, vocab_size=300, block_size=64), 2, 48)])
def test_gpt2_small_configs_match_fp32_reference(cfg, B, T):
    w = G.init_weights(cfg, seed=5)
    # non-trivial LayerNorm parameters and biases so that every epilogue operand matters
    rng = np.random.default_rng(6)
    for i in range(cfg.n_layer):
        for k, v in w[f"h{i}"].items():
            if k.endswith("_b"):
                w[f"h{i}"][k] = (rng.standard_normal(v.shape) * 0.02).astype(np.float32)
            if k.endswith("_g"):
                w[f"h{i}"][k] = (1 + rng.standard_normal(v.shape) * 0.02).astype(np.float32)
    idx = rng.integers(0, cfg.vocab_size, (B, T)).astype(np.int32)
    want = G.reference_forward(cfg, w, idx)
    # head dim 64 runs the fused attention kernel; every config also runs attention as four kernels
    for fused in ([True, False] if T % 8 == 0 else [True]):
        model = G.GPT2(cfg, w, fused_attention=fused)
        logits = model.forward(torch.from_numpy(idx).cuda())
        assert K.device_error() == 0
        got = logits.float().cpu().numpy()
        assert got.shape == want.shape
        assert_close(got, want, 2e-2, 2e-2 * float(np.abs(want).max()), f"logits (fused attention: {model.fused_attention})")


def test_gpt2_small_full_architecture_two_sequences():
    # the configured model (12 layers, 768, 12 heads, vocab 50257, context 1024) on a 2 x 1024 slice of the batch;
    # the CPU reference at fp32 takes some seconds
    cfg = G.GPT2Config()
    w = G.init_weights(cfg, seed=5)
    rng = np.random.default_rng(5)
    idx = rng.integers(0, cfg.vocab_size, (2, 1024)).astype(np.int32)
    model = G.GPT2(cfg, w)
    got = model.forward(torch.from_numpy(idx).cuda()).float().cpu().numpy()
    assert K.device_error() == 0
    want = G.reference_forward(cfg, w, idx)
    assert_close(got, want, 2e-2, 2e-2 * float(np.abs(want).max()), "logits")
    # and the argmax token agrees almost everywhere (ties aside)
    assert (got.argmax(-1) == want.argmax(-1)).mean() > 0.98


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_embedding_rows_is_an_exact_gather(dtype):
    """out[r] = wte[ids[r]] + wpe[r % T] (pequegrad/modules.py:329-337 over csrc/cuda/select.cuh:27-79): index work, so
    the gathered rows are compared bit for bit; the positional row wraps at T; an id outside the table gives a zero row."""
    g = torch.Generator(device="cuda").manual_seed(9)
    V, C, T = 1000, 96, 7
    wte = torch.randn((V, C), generator=g, device="cuda").to(dtype)
    wpe = torch.randn((T, C), generator=g, device="cuda").to(dtype)
    ids = torch.randint(0, V, (5, T), generator=g, device="cuda", dtype=torch.int32)
    # without positions: a pure gather
    got = K.embedding_rows(ids, wte, None, T)
    assert got.shape == (5, T, C) and torch.equal(got, wte[ids.long()])
    # with positions: one add per element, in the table's dtype arithmetic (fp32 add, rounded once for fp16)
    got = K.embedding_rows(ids, wte, wpe, T)
    want = (wte[ids.long()].float() + wpe[None].float()).to(dtype)
    assert torch.equal(got, want)
    # a flat id list longer than T: row r uses position r % T
    flat = ids.reshape(-1)
    got = K.embedding_rows(flat, wte, wpe, T)
    pos = torch.arange(flat.numel(), device="cuda") % T
    assert torch.equal(got, (wte[flat.long()].float() + wpe[pos].float()).to(dtype))
    # ids outside [0, V) read nothing: the whole output row is zero, with or without positions
    bad = ids.clone()
    bad[0, 0], bad[2, 3] = V, -1
    got = K.embedding_rows(bad, wte, wpe, T)
    assert (got[0, 0] == 0).all() and (got[2, 3] == 0).all()
    got = K.embedding_rows(bad, wte, None, T)
    assert (got[0, 0] == 0).all() and (got[2, 3] == 0).all()
    ok = torch.ones((5, T), dtype=torch.bool, device="cuda")
    ok[0, 0] = ok[2, 3] = False
    assert torch.equal(got[ok], wte[bad.long().clamp(0, V - 1)][ok])
