"""GPT-2 forward inference on the kernels of this library.

The model is the one of the reference's examples/gpt2.py:149-204, 365-380
(pre-LN blocks, c_attn 768->2304, 12 heads of 64, causal softmax attention,
MLP 768->3072->768 with tanh GELU, final LayerNorm, untied lm_head without
bias), batched over sequences: fp16 weights and activations, fp32 accumulation
in every GEMM and in LayerNorm / softmax. Per layer the launches are:
  layernorm | qkv GEMM(+bias) | fused causal attention (scores, softmax and PV in
  one kernel, heads read from and written to the packed [B, T, C] buffers) |
  proj GEMM(+bias,+residual) | layernorm | fc GEMM(+bias,+GELU) | proj GEMM(+bias,+residual)
Weights of a Linear are kept transposed ([out, in], K-major for the GEMM).
`fused_attention=False` runs attention as the reference composes it (scores GEMM,
causal softmax kernel, V transpose, PV GEMM) for comparison.
"""
from __future__ import annotations

import numpy as np
import torch

from . import kernels as K


class GPT2Config:
    def __init__(self, n_layer=12, n_head=12, n_embd=768, vocab_size=50257, block_size=1024):
        self.n_layer, self.n_head, self.n_embd, self.vocab_size, self.block_size = n_layer, n_head, n_embd, vocab_size, block_size


def init_weights(cfg: GPT2Config, seed: int = 5) -> dict:
    """Random init as the benchmark configuration states: every weight N(0, 0.02), LayerNorm gamma 1 / beta 0, biases 0.
    numpy fp32, in the reference's layouts (Linear weight [in, out])."""
    rng = np.random.default_rng(seed)
    C, V = cfg.n_embd, cfg.vocab_size
    n = lambda *s: (rng.standard_normal(s) * 0.02).astype(np.float32)  # noqa: E731
    w = {"wte": n(V, C), "wpe": n(cfg.block_size, C), "lnf_g": np.ones(C, np.float32), "lnf_b": np.zeros(C, np.float32), "lm_head": n(C, V)}
    for i in range(cfg.n_layer):
        w[f"h{i}"] = dict(ln1_g=np.ones(C, np.float32), ln1_b=np.zeros(C, np.float32), attn_w=n(C, 3 * C), attn_b=np.zeros(3 * C, np.float32),
                          proj_w=n(C, C), proj_b=np.zeros(C, np.float32), ln2_g=np.ones(C, np.float32), ln2_b=np.zeros(C, np.float32),
                          fc_w=n(C, 4 * C), fc_b=np.zeros(4 * C, np.float32), fc2_w=n(4 * C, C), fc2_b=np.zeros(C, np.float32))
    return w


class GPT2:
    def __init__(self, cfg: GPT2Config, weights: dict, device="cuda", dtype=torch.float16, fused_attention: bool = True):
        self.cfg, self.dtype = cfg, dtype
        self.fused_attention = fused_attention and cfg.n_embd // cfg.n_head == 64
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device=device, dtype=dtype)  # noqa: E731
        lin = lambda w_: dev(np.ascontiguousarray(w_.T))  # noqa: E731  [in, out] -> [out, in]
        self.wte, self.wpe = dev(weights["wte"]), dev(weights["wpe"])
        self.lnf_g, self.lnf_b = dev(weights["lnf_g"]), dev(weights["lnf_b"])
        self.lm_head_t = lin(weights["lm_head"])
        self.blocks = []
        for i in range(cfg.n_layer):
            h = weights[f"h{i}"]
            self.blocks.append(dict(ln1_g=dev(h["ln1_g"]), ln1_b=dev(h["ln1_b"]), attn_wt=lin(h["attn_w"]), attn_b=dev(h["attn_b"]),
                                    proj_wt=lin(h["proj_w"]), proj_b=dev(h["proj_b"]), ln2_g=dev(h["ln2_g"]), ln2_b=dev(h["ln2_b"]),
                                    fc_wt=lin(h["fc_w"]), fc_b=dev(h["fc_b"]), fc2_wt=lin(h["fc2_w"]), fc2_b=dev(h["fc2_b"])))
        # logits rows are padded to a multiple of 8 halves so every row starts 16-byte aligned (50257 -> 50264)
        self.vocab_ld = (cfg.vocab_size + 7) // 8 * 8

    def forward(self, idx: torch.Tensor, logits_out: torch.Tensor | None = None) -> torch.Tensor:
        """idx: [B, T] int32 token ids on the device. Returns logits [B, T, vocab] (a view of a row-padded buffer)."""
        cfg = self.cfg
        B, T = idx.shape
        C, H = cfg.n_embd, cfg.n_head
        D = C // H
        if T > cfg.block_size:
            raise ValueError("GPT2.forward: the sequence is longer than block_size")
        if not self.fused_attention and T % 8:
            # the [T, T] score rows feed the tensor-map loads of the PV GEMM, whose row pitch must be a multiple of 16 bytes
            raise ValueError("GPT2.forward: the unfused attention path needs a sequence length that is a multiple of 8")
        x = K.embedding_rows(idx, self.wte, self.wpe, T)  # [B, T, C]
        for blk in self.blocks:
            h = K.layernorm_rows(x, blk["ln1_g"], blk["ln1_b"], 1e-5)
            qkv = K.matmul(h, blk["attn_wt"].T, bias=blk["attn_b"])  # [B, T, 3C]
            q, k, v = (qkv[:, :, i * C:(i + 1) * C].view(B, T, H, D).permute(0, 2, 1, 3) for i in range(3))  # [B, H, T, D] views
            y = torch.empty((B, T, C), dtype=self.dtype, device=x.device)
            y_heads = y.view(B, T, H, D).permute(0, 2, 1, 3)  # heads written straight into [B, T, C]
            if self.fused_attention:
                K.attention(q, k, v, scale=float(D) ** -0.5, causal=True, out=y_heads)
            else:
                att = K.matmul(q, k.transpose(-2, -1), alpha=1.0 / 8.0 if D == 64 else float(D) ** -0.5)  # [B, H, T, T]
                att = K.softmax_rows(att, causal=True)
                (vt,) = K.fused_elementwise([v.transpose(-2, -1)], [("LOAD", 0)])  # [B, H, D, T] contiguous: V with T as the contraction dim
                K.matmul(att, vt.transpose(-2, -1), out=y_heads)
            x = K.matmul(y, blk["proj_wt"].T, bias=blk["proj_b"], residual=x)
            h = K.layernorm_rows(x, blk["ln2_g"], blk["ln2_b"], 1e-5)
            h = K.matmul(h, blk["fc_wt"].T, bias=blk["fc_b"], act=2)
            x = K.matmul(h, blk["fc2_wt"].T, bias=blk["fc2_b"], residual=x)
        x = K.layernorm_rows(x, self.lnf_g, self.lnf_b, 1e-5)
        if logits_out is None:
            logits_out = torch.empty((B, T, self.vocab_ld), dtype=self.dtype, device=x.device)
        logits = logits_out[:, :, : cfg.vocab_size]
        K.matmul(x, self.lm_head_t.T, out=logits)
        return logits


def round_weights_fp16(weights: dict) -> dict:
    """The weights as fp32 torch-CPU tensors after a round trip through fp16 (what the device model stores)."""
    r = lambda a: torch.from_numpy(a.astype(np.float16).astype(np.float32))  # noqa: E731
    return {k: ({k2: r(v2) for k2, v2 in v.items()} if isinstance(v, dict) else r(v)) for k, v in weights.items()}


def reference_forward(cfg: GPT2Config, weights: dict, idx: np.ndarray, rounded: dict | None = None) -> np.ndarray:
    """fp32 torch-CPU restatement of examples/gpt2.py for parity tests (masked scores are -inf here where the
    example adds -1e9: after the softmax both give exactly 0 in fp32). Weights are first rounded to fp16 as
    the device model stores them (`rounded` = a cached `round_weights_fp16(weights)`)."""
    w = rounded if rounded is not None else round_weights_fp16(weights)
    B, T = idx.shape
    C, H = cfg.n_embd, cfg.n_head
    ids = torch.from_numpy(idx.astype(np.int64))
    x = w["wte"][ids] + w["wpe"][:T]
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    ln = lambda t, g, b: torch.nn.functional.layer_norm(t, (C,), g, b, 1e-5)  # noqa: E731
    for i in range(cfg.n_layer):
        h = w[f"h{i}"]
        a = ln(x, h["ln1_g"], h["ln1_b"]) @ h["attn_w"] + h["attn_b"]
        q, k, v = (t.view(B, T, H, C // H).transpose(1, 2) for t in a.split(C, dim=2))
        s = (q @ k.transpose(-2, -1)) / (C // H) ** 0.5
        s = torch.softmax(s.masked_fill(~mask, float("-inf")), -1)
        y = (s @ v).transpose(1, 2).reshape(B, T, C)
        x = x + y @ h["proj_w"] + h["proj_b"]
        m = ln(x, h["ln2_g"], h["ln2_b"]) @ h["fc_w"] + h["fc_b"]
        m = 0.5 * m * (1.0 + torch.tanh(0.7978845608028654 * (m + 0.044715 * m ** 3)))
        x = x + m @ h["fc2_w"] + h["fc2_b"]
    x = ln(x, w["lnf_g"], w["lnf_b"])
    return (x @ w["lm_head"]).numpy()
