"""Benchmark workloads beyond the reduction sweep, in the shape `bench.py` drives:

    setup(dev, rank); step(); units_per_step; e2e_setup(); e2e_step() with h2d / d2h byte counts;
    roofline(pk, reps) -> dict for the dominant kernel; cpu_sample(budget_s, threads).

All inputs are seeded synthetic tensors of the configured shapes and distributions.
"""
from __future__ import annotations

import statistics
import time

import numpy as np

MLP_DIMS = [784, 1024, 1024, 10]
MLP_ROWS = 65536
GPT2_BATCH, GPT2_T = 32, 1024


def _event_us(fn, reps, flush=None):
    """Median device time of fn() in microseconds, CUDA events on the current stream."""
    import torch
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    runway = getattr(torch.cuda, "_sleep", None)  # a spin kernel; without it the timings below are upper bounds
    for a, b in evs:
        if flush is not None:
            flush()
        # The device first spins for ~0.2 ms without touching memory, so that the launch below is already queued when
        # the first event is reached: without this runway the interval also holds the host's time to issue the call
        # (tens of microseconds for a ctypes call), which swamps kernels of 10-60 us.
        if runway is not None:
            runway(400_000)
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    return statistics.median(a.elapsed_time(b) for a, b in evs) * 1e3


def mlp_weights(seed=3):
    rng = np.random.default_rng(seed)
    Ws = [(rng.standard_normal((MLP_DIMS[i], MLP_DIMS[i + 1])) * 0.05).astype(np.float32) for i in range(3)]
    bs = [(rng.standard_normal(MLP_DIMS[i + 1]) * 0.05).astype(np.float32) for i in range(3)]
    return Ws, bs


class Mlp:
    """int8 quantized MLP 784 -> 1024 -> 1024 -> 10, `rows` activations rows per GPU."""
    name, metric, unit, dtype = "mlp", "int8-MLP rows/s", "rows/s", "i8"

    def __init__(self, rows=MLP_ROWS):
        self.rows = rows
        self.desc = (f"quantized MLP inference 784->1024->1024->10 with ReLU, {rows} rows per GPU; weights N(0,0.05) int8 per output "
                     "channel, activations uniform[0,1) fp32 quantized per tensor on the device; int32 accumulate, fused dequant+bias+ReLU")

    def setup(self, dev, rank):
        import torch
        from .qmlp import QuantizedMLP
        Ws, bs = mlp_weights()
        self.mlp = QuantizedMLP(Ws, bs, device=dev)
        g = torch.Generator(device=dev).manual_seed(2 + rank)
        self.X = torch.rand((self.rows, MLP_DIMS[0]), generator=g, device=dev)
        self.units_per_step = self.rows
        self.ops_per_row = 2 * sum(MLP_DIMS[i] * MLP_DIMS[i + 1] for i in range(3))
        self.config = {"rows_per_gpu": self.rows, "int8_ops_per_step": self.ops_per_row * self.rows,
                       "l2": "activations per layer (51 to 268 MB) are larger than or comparable to the 126 MB L2; each layer "
                             "reads what the one before wrote, as the pipeline does in use"}

    def step(self):
        self.out = self.mlp.forward(self.X)

    def e2e_setup(self):
        import torch
        self.host_x = torch.empty(self.X.shape, dtype=torch.float32).pin_memory()
        self.host_x.copy_(self.X)
        self.step()
        self.host_out = torch.empty(self.out.shape, dtype=torch.float32).pin_memory()
        self.h2d = self.host_x.numel() * 4
        self.d2h = self.host_out.numel() * 4

    def e2e_step(self):
        self.X.copy_(self.host_x, non_blocking=True)
        self.step()
        self.host_out.copy_(self.out, non_blocking=True)

    def roofline(self, pk, reps):
        """The 1024 -> 1024 hidden layer's GEMM as the pipeline runs it: the absmax-only pass and the pass that stores
        requantised int8 (the slower of the two is the reported kernel), plus the fp32-output variant for comparison."""
        from . import kernels as K
        wq, ws, bias = self.mlp.layers[1]
        b = self.mlp._buffers(self.rows, self.X.device)
        xq, amax = b["q"][1], b["amax"]
        flush = lambda: b["h"][0].zero_()  # noqa: E731  268 MB: nothing of the operands stays in L2
        t_abs = _event_us(lambda: K.qlinear_i8(xq, wq, ws, a_absmax=amax[1:2], bias=bias, relu=True, want_out=False, out_absmax=amax[2:3]), reps, flush)
        t_q = _event_us(lambda: K.qlinear_i8(xq, wq, ws, a_absmax=amax[1:2], bias=bias, relu=True, out=b["q"][2], out_absmax=amax[2:3]), reps, flush)
        t_f = _event_us(lambda: K.qlinear_i8(xq, wq, ws, a_absmax=amax[1:2], bias=bias, relu=True, out=b["h"][1]), reps, flush)
        ops = 2.0 * self.rows * 1024 * 1024
        peak = 2 * pk["f16"]
        us = max(t_abs, t_q)
        ach = ops / (us * 1e-6) / 1e12
        tops = lambda t: round(ops / (t * 1e-6) / 1e12, 1)  # noqa: E731
        other = {"absmax_f32_us": round(_event_us(lambda: K.absmax(self.X, out=amax[0:1]), reps), 1),
                 "quantize_input_us": round(_event_us(lambda: K.quantize_i8(self.X, absmax_dev=amax[0:1], out=b["q"][0]), reps), 1),
                 "quantize_hidden_us (materialising route only)": round(_event_us(lambda: K.quantize_i8(b["h"][1], absmax_dev=amax[2:3], out=b["q"][2]), reps), 1)}
        return {"bound": "tensor", "kernel": "gemm_tc_kernel<i8> %dx1024x1024, %s epilogue" % (self.rows, "int8-requantising" if t_q >= t_abs else "absmax-only"),
                "achieved": round(ach, 1), "peak": peak, "unit": "TOP/s", "frac": round(ach / peak, 4),
                "peak_source": pk["source"] + " bf16 GEMM rate x 2 (int8 issues at twice the 16-bit rate on the same pipe)",
                "traffic": None, "us": round(us, 1), "algorithmic_ops_per_launch": ops,
                "variants": {"absmax_only": {"us": round(t_abs, 1), "tops": tops(t_abs), "frac": round(tops(t_abs) / peak, 4)},
                             "int8_out": {"us": round(t_q, 1), "tops": tops(t_q), "frac": round(tops(t_q) / peak, 4)},
                             "fp32_out (268 MB written)": {"us": round(t_f, 1), "tops": tops(t_f), "frac": round(tops(t_f) / peak, 4)}},
                "other_kernels": other}

    def cpu_sample(self, budget_s, threads):
        """The int8 pipeline of the CPU restatement on blocks of 2048 rows until the budget is spent."""
        import oracle
        Ws, bs = mlp_weights()
        prep = [oracle.quantize_weight_per_channel(W) for W in Ws]
        rng = np.random.default_rng(2)
        rows, t_total = 0, 0.0
        while t_total < budget_s:
            h = rng.random((2048, MLP_DIMS[0]), dtype=np.float32)
            t0 = time.perf_counter()
            for i in range(3):
                sx = oracle.quant_scale(oracle.absmax(h))
                h = oracle.dequant_bias_act(oracle.gemm_i8(oracle.quantize_i8(h, sx), prep[i][0]), prep[i][1], sx, bs[i], relu=i < 2)
            t_total += time.perf_counter() - t0
            rows += 2048
        return rows, t_total, f"{rows} rows in blocks of 2048 through the 3-layer int8 pipeline, {t_total:.1f} s of CPU work, {threads} threads", "port"


class Gpt2:
    """GPT-2 small forward (12 layers, 768, 12 heads, vocab 50257), `batch` sequences of `T` tokens per GPU."""
    name, metric, unit, dtype = "gpt2", "GPT-2 tok/s", "tok/s", "f16"

    def __init__(self, batch=GPT2_BATCH, T=GPT2_T):
        self.B, self.T = batch, T
        self.desc = (f"GPT-2 small forward inference from random init N(0,0.02): 12 layers, d_model 768, 12 heads, d_ff 3072, vocab 50257, "
                     f"{batch} x {T} token ids uniform in [0,50257) per GPU; fp16 activations and weights, fp32 accumulate")

    def setup(self, dev, rank):
        import torch
        from . import gpt2 as G
        self.cfg = G.GPT2Config()
        self.weights = G.init_weights(self.cfg, seed=5)
        self.model = G.GPT2(self.cfg, self.weights, device=dev)
        g = torch.Generator(device=dev).manual_seed(2 + rank)
        self.idx = torch.randint(0, self.cfg.vocab_size, (self.B, self.T), generator=g, device=dev, dtype=torch.int32)
        self.logits_buf = torch.empty((self.B, self.T, self.model.vocab_ld), dtype=torch.float16, device=dev)
        self.units_per_step = self.B * self.T
        C, L_, V, T = self.cfg.n_embd, self.cfg.n_layer, self.cfg.vocab_size, self.T
        # multiply-adds x 2 per token: the four Linear layers of a block, the lm_head, and both attention GEMMs over the
        # causal half of the [T, T] square (the average query row sees (T + 1) / 2 keys)
        self.flops_per_token = 2.0 * (L_ * (C * 3 * C + C * C + 2 * C * 4 * C) + C * V) + 2.0 * 2.0 * ((T + 1) / 2.0) * C * L_
        self.config = {"batch_per_gpu": self.B, "seq_len": T, "flops_per_token": self.flops_per_token,
                       "l2": "activations of a layer (50 to 805 MB) and the 3.3 GB of logits are larger than the 126 MB L2"}

    def step(self):
        self.logits = self.model.forward(self.idx, logits_out=self.logits_buf)

    def e2e_setup(self):
        import torch
        from . import _lib as L
        from . import kernels as K
        self.host_idx = torch.empty(self.idx.shape, dtype=torch.int32).pin_memory()
        self.host_idx.copy_(self.idx)
        self.step()
        # the result a caller reads back: the greedy next-token id at every position (argmax over the vocabulary,
        # one fused reduce launch over the fp16 logits view)
        self.next_ids = K.PreparedReduce([self.logits], L.ARGMAX, [-1], False)
        self.host_ids = torch.empty(self.next_ids.out.shape, dtype=torch.int32).pin_memory()
        self.h2d = self.host_idx.numel() * 4
        self.d2h = self.host_ids.numel() * 4

    def e2e_step(self):
        self.idx.copy_(self.host_idx, non_blocking=True)
        self.step()
        self.host_ids.copy_(self.next_ids(), non_blocking=True)

    def roofline(self, pk, reps):
        """The MLP up-projection GEMM (32768 x 3072 x 768, + bias + tanh GELU, fp16 out) timed alone, and per-kernel shares of a layer."""
        import torch
        from . import kernels as K
        dev = self.idx.device
        M, C = self.B * self.T, self.cfg.n_embd
        blk = self.model.blocks[0]
        g = torch.Generator(device=dev).manual_seed(7)
        h = (torch.randn((M, C), generator=g, device=dev) * 0.5).half()
        out = torch.empty((M, 4 * C), dtype=torch.float16, device=dev)
        us = _event_us(lambda: K.matmul(h, blk["fc_wt"].T, bias=blk["fc_b"], act=2, out=out), reps)
        flops = 2.0 * M * C * 4 * C
        ach = flops / (us * 1e-6) / 1e12
        parts = {}
        x3 = h.view(self.B, self.T, C)
        qkv = K.matmul(x3, blk["attn_wt"].T, bias=blk["attn_b"])
        H, D = self.cfg.n_head, C // self.cfg.n_head
        q, k, v = (qkv[:, :, i * C:(i + 1) * C].view(self.B, self.T, H, D).permute(0, 2, 1, 3) for i in range(3))
        att = K.matmul(q, k.transpose(-2, -1), alpha=0.125)
        (vt,) = K.fused_elementwise([v.transpose(-2, -1)], [("LOAD", 0)])
        y = torch.empty((self.B, self.T, C), dtype=torch.float16, device=dev)
        parts["layernorm"] = _event_us(lambda: K.layernorm_rows(x3, blk["ln1_g"], blk["ln1_b"], 1e-5), reps)
        parts["qkv_gemm"] = _event_us(lambda: K.matmul(x3, blk["attn_wt"].T, bias=blk["attn_b"], out=qkv), reps)
        y_heads = y.view(self.B, self.T, H, D).permute(0, 2, 1, 3)
        parts["fused_attention"] = _event_us(lambda: K.attention(q, k, v, scale=0.125, causal=True, out=y_heads), reps)
        # the same attention as four kernels (what GPT2(fused_attention=False) runs), for comparison
        parts["unfused_scores_gemm"] = _event_us(lambda: K.matmul(q, k.transpose(-2, -1), alpha=0.125, out=att), reps)
        parts["unfused_causal_softmax"] = _event_us(lambda: K.softmax_rows(att, causal=True), reps)
        parts["unfused_v_transpose"] = _event_us(lambda: K.fused_elementwise([v.transpose(-2, -1)], [("LOAD", 0)]), reps)
        parts["unfused_pv_gemm"] = _event_us(lambda: K.matmul(att, vt.transpose(-2, -1), out=y_heads), reps)
        parts["proj_gemm"] = _event_us(lambda: K.matmul(y, blk["proj_wt"].T, bias=blk["proj_b"], residual=x3, out=y), reps)
        parts["fc_gemm_gelu"] = us
        parts["fc2_gemm"] = _event_us(lambda: K.matmul(out.view(self.B, self.T, 4 * C), blk["fc2_wt"].T, bias=blk["fc2_b"], residual=x3, out=y), reps)
        parts["lm_head_gemm"] = _event_us(lambda: K.matmul(x3, self.model.lm_head_t.T, out=self.logits_buf[:, :, : self.cfg.vocab_size]), max(3, reps // 2))
        return {"bound": "tensor", "kernel": "gemm_tc_kernel<f16> 32768x3072x768 + bias + GELU epilogue", "achieved": round(ach, 1),
                "peak": pk["f16_sustained"], "unit": "TFLOP/s", "frac": round(ach / pk["f16_sustained"], 4),
                "peak_source": pk["source"] + " (sustained bf16 cuBLAS rate: the kernel runs inside a long step)", "traffic": None,
                "us": round(us, 1), "algorithmic_flops_per_launch": flops, "kernel_us": {k_: round(v_, 1) for k_, v_ in parts.items()}}

    def cpu_sample(self, budget_s, threads):
        """The fp32 CPU restatement of the model on sequences of 256 tokens until the budget is spent."""
        import torch
        from . import gpt2 as G
        torch.set_num_threads(threads)
        if not hasattr(self, "cfg"):
            self.cfg = G.GPT2Config()
            self.weights = G.init_weights(self.cfg, seed=5)
        rounded = G.round_weights_fp16(self.weights)
        rng = np.random.default_rng(2)
        toks, t_total = 0, 0.0
        while t_total < budget_s:
            idx = rng.integers(0, self.cfg.vocab_size, (1, 256)).astype(np.int32)
            t0 = time.perf_counter()
            G.reference_forward(self.cfg, self.weights, idx, rounded)
            t_total += time.perf_counter() - t0
            toks += 256
        return toks, t_total, f"{toks} tokens as sequences of 256 through the fp32 CPU restatement of the model, {t_total:.1f} s, {threads} threads", "port"


class Rows:
    """Causal row softmax over fp16 scores [32,12,1024,1024] and LayerNorm over fp32 [16384,768], one kernel each."""
    name, metric, unit, dtype = "rows", "softmax+LayerNorm HBM GB/s", "GB/s", "f16/f32"
    SM_SHAPE, LN_SHAPE = (32, 12, 1024, 1024), (16384, 768)

    def __init__(self):
        self.desc = ("row softmax over fp16 scores [32,12,1024,1024] N(0,1) with causal mask; LayerNorm over fp32 [16384,768] N(0,1), "
                     "gamma=1+N(0,0.02), beta=N(0,0.02), eps=1e-5; a single kernel each")

    def setup(self, dev, rank):
        import torch
        g = torch.Generator(device=dev).manual_seed(2 + rank)
        self.S = torch.randn(self.SM_SHAPE, generator=g, device=dev).half()
        self.X = torch.randn(self.LN_SHAPE, generator=g, device=dev)
        self.gamma = 1 + 0.02 * torch.randn(768, generator=g, device=dev)
        self.beta = 0.02 * torch.randn(768, generator=g, device=dev)
        # the causal kernel reads the lower triangle only and writes every element
        T = self.SM_SHAPE[-1]
        n_rows = self.S.numel() // T
        self.sm_bytes = n_rows * (T + 1) // 2 * 2 + self.S.numel() * 2
        self.ln_bytes = self.X.numel() * 8 + 768 * 8
        self.units_per_step = (self.sm_bytes + self.ln_bytes) / 1e9
        self.config = {"softmax_bytes": self.sm_bytes, "layernorm_bytes": self.ln_bytes,
                       "l2": "the 805 MB of scores are larger than the 126 MB L2; the 50 MB LayerNorm input is flushed by the softmax between launches"}

    def step(self):
        from . import kernels as K
        self.sm_out = K.softmax_rows(self.S, causal=True)
        self.ln_out = K.layernorm_rows(self.X, self.gamma, self.beta, 1e-5)

    def e2e_setup(self):
        import torch
        self.host_x = torch.empty(self.LN_SHAPE, dtype=torch.float32).pin_memory()
        self.host_x.copy_(self.X)
        self.host_y = torch.empty(self.LN_SHAPE, dtype=torch.float32).pin_memory()
        self.h2d = self.host_x.numel() * 4
        self.d2h = self.host_y.numel() * 4

    def e2e_step(self):
        # the scores of an attention layer never leave the device in use; LayerNorm rows go both ways
        self.X.copy_(self.host_x, non_blocking=True)
        self.step()
        self.host_y.copy_(self.ln_out, non_blocking=True)

    def _flush_l2(self):
        # 201 MB written, then another 201 MB read: the L2 (126 MB) ends up holding clean lines of unrelated data, as
        # it would after the kernels that run between two LayerNorms in use. Writing alone leaves the L2 full of dirty
        # lines, and their write-back would be charged to the timed kernel's first misses.
        self.S[:8].zero_().add_(1)
        self._sink = self.S[8:16].amax()

    def roofline(self, pk, reps):
        from . import kernels as K
        sm_us = _event_us(lambda: K.softmax_rows(self.S, causal=True), reps)
        ln_us = _event_us(lambda: K.layernorm_rows(self.X, self.gamma, self.beta, 1e-5), reps, flush=self._flush_l2)
        ach = self.sm_bytes / (sm_us * 1e-6) / 1e9
        ln = self.ln_bytes / (ln_us * 1e-6) / 1e9
        return {"bound": "hbm", "kernel": "softmax_rows (causal, fp16, 1024 columns)", "achieved": round(ach, 1), "peak": pk["hbm"], "unit": "GB/s",
                "frac": round(ach / pk["hbm"], 4), "peak_source": pk["source"], "traffic": None, "us": round(sm_us, 1),
                "algorithmic_bytes_per_launch": self.sm_bytes,
                "layernorm": {"gbs": round(ln, 1), "frac": round(ln / pk["hbm"], 4), "us": round(ln_us, 1), "bytes": self.ln_bytes}}

    def cpu_sample(self, budget_s, threads):
        """The CPU restatement of both row kernels on slices of the same tensors until the budget is spent."""
        import oracle
        rng = np.random.default_rng(2)
        S = rng.standard_normal((2, 1024, 1024)).astype(np.float16)
        X = rng.standard_normal((4096, 768)).astype(np.float32)
        gm, bt = np.ones(768, np.float32), np.zeros(768, np.float32)
        done, t_total = 0.0, 0.0
        while t_total < budget_s:
            t0 = time.perf_counter()
            oracle.softmax_rows(S, causal=True)
            oracle.layernorm_rows(X, gm, bt, 1e-5)
            t_total += time.perf_counter() - t0
            done += (S.size * 3 + X.size * 8) / 1e9
        return done, t_total, f"softmax over [2,1024,1024] fp16 + LayerNorm over [4096,768] fp32, repeated for {t_total:.1f} s, {threads} threads", "port"
