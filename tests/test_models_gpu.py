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


def test_gpt2_small_full_architecture_one_sequence():
    # the configured model (12 layers, 768, 12 heads, vocab 50257, context 1024) on one sequence; the CPU
    # reference at fp32 takes a few seconds
    cfg = G.GPT2Config()
    w = G.init_weights(cfg, seed=5)
    rng = np.random.default_rng(5)
    idx = rng.integers(0, cfg.vocab_size, (1, 1024)).astype(np.int32)
    model = G.GPT2(cfg, w)
    got = model.forward(torch.from_numpy(idx).cuda()).float().cpu().numpy()
    assert K.device_error() == 0
    want = G.reference_forward(cfg, w, idx)
    assert_close(got, want, 2e-2, 2e-2 * float(np.abs(want).max()), "logits")
    # and the argmax token agrees almost everywhere (ties aside)
    assert (got.argmax(-1) == want.argmax(-1)).mean() > 0.98
