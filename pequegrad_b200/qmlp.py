"""int8 quantized MLP inference (784 -> 1024 -> 1024 -> 10 with ReLU).

The workload of the reference's examples/quantized_mlp.py, with real int8 in
place of its fp32 fake quantisation (examples/quantized_mlp.py:28-48):
  weights      offline, per output channel: s_w[n] = max(max_k |W[k,n]|, 1e-6) / 127,
               Wq[n,k] = clip(rint(W[k,n] / s_w[n]), -127, 127), stored [N, K] (K-major)
  activations  on the device, per tensor and per layer: s_x = max(max|x|, 1e-6) / 127,
               xq = clip(rint(x / s_x), -127, 127); the absmax never leaves the GPU
  layer        acc = xq . Wq^T in int32 (tcgen05 kind::i8), then
               h = relu(acc * (s_x * s_w[n]) + b[n]) in fp32; the last layer has no ReLU
A hidden layer never writes its fp32 output: the GEMM runs twice on the same int8
operands, first with an epilogue that only folds max|h| into a device scalar, then
with one that quantises h for the next layer and stores int8 (a quarter of the fp32
bytes). The accumulators and the epilogue arithmetic are the same in both, so the
int8 activations equal those of the materialising route (`keep=True`: quantise
kernel, GEMM with fp32 output and fused absmax), which the parity tests check.
"""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from . import kernels as K


def quantize_weight(w: np.ndarray):
    """w: [K, N] fp32 as a Linear stores it (pequegrad/modules.py:221-225) -> (Wq [N, K] int8, s_w [N] fp32)."""
    wt = np.ascontiguousarray(w.T, np.float32)
    amax = np.maximum(np.abs(wt).max(axis=1), np.float32(1e-6)).astype(np.float32)
    scale = (amax / np.float32(127)).astype(np.float32)
    q = np.clip(np.rint(wt / scale[:, None]), -127, 127).astype(np.int8)
    return q, scale


class QuantizedMLP:
    def __init__(self, weights: Sequence[np.ndarray], biases: Sequence[np.ndarray], device="cuda"):
        self.layers = []
        for w, b in zip(weights, biases):
            q, s = quantize_weight(w)
            self.layers.append((torch.from_numpy(q).to(device), torch.from_numpy(s).to(device),
                                torch.from_numpy(np.ascontiguousarray(b, np.float32)).to(device)))
        self._bufs = {}

    def _buffers(self, rows: int, device, slot: int = 0):
        key = (rows, str(device), slot)
        if key not in self._bufs:
            dims = [self.layers[0][0].shape[1]] + [l[0].shape[0] for l in self.layers]
            self._bufs[key] = dict(
                q=[torch.empty((rows, d), dtype=torch.int8, device=device) for d in dims[:-1]],
                h=[torch.empty((rows, d), dtype=torch.float32, device=device) for d in dims[1:]],
                amax=torch.zeros(len(self.layers) + 1, dtype=torch.float32, device=device),
            )
        return self._bufs[key]

    def forward(self, x: torch.Tensor, keep: bool = False):
        """x: [rows, 784] fp32 on the device. Returns logits [rows, 10] fp32 (and, with keep, the per-layer tensors)."""
        out = self.forward_sharded([x], keep)[0]
        return out

    def forward_sharded(self, xs, keep: bool = False, peers=None):
        """The same forward over row shards of ONE batch: `xs` is this process's list of shards (or a
        `distrib.ShardedTensor` split along dim 0). "Per tensor" keeps meaning the whole batch: after every
        absmax the shards' maxima are combined (`distrib.all_reduce(.., "max")`: one float per layer, across the
        shards held here and across processes), so the int8 activations and the outputs have the same bits
        however the rows are split. With `peers` (a `distrib.PeerGroup`, one shard per process) the maxima are
        exchanged by the peer-memory kernel, one small launch, instead of a library collective. Returns one output
        per local shard."""
        from . import distrib as D
        xs = xs.shards if isinstance(xs, D.ShardedTensor) else list(xs)
        S = len(xs)
        lone = S == 1 and D.rank_world()[1] == 1
        bufs = [self._buffers(x.shape[0], x.device, j) for j, x in enumerate(xs)]
        for b in bufs:
            b["amax"][1:].zero_()  # slot i holds max|input of layer i|; the GEMM epilogues fold into slots 1..

        def combine(i):
            if lone:
                return
            if peers is not None and S == 1:
                peers.allreduce_max(bufs[0]["amax"][i:i + 1])
            else:
                D.all_reduce([b["amax"][i:i + 1] for b in bufs], "max")

        for x, b in zip(xs, bufs):
            K.absmax(x, out=b["amax"][0:1])
        combine(0)
        xq = [K.quantize_i8(x, absmax_dev=b["amax"][0:1], out=b["q"][0]) for x, b in zip(xs, bufs)]
        kept = [[] for _ in xs]
        hs = [None] * S
        n = len(self.layers)
        for i, (wq, ws, bias) in enumerate(self.layers):
            last = i == n - 1
            fused = not keep and not last and wq.shape[0] > 128 and wq.shape[0] % 16 == 0
            if fused:
                for j, b in enumerate(bufs):
                    K.qlinear_i8(xq[j], wq, ws, a_absmax=b["amax"][i:i + 1], bias=bias, relu=True, want_out=False, out_absmax=b["amax"][i + 1:i + 2])
                combine(i + 1)
                for j, b in enumerate(bufs):
                    # with an int8 output the absmax slot is an input: the scale the epilogue quantises with
                    xq[j], _ = K.qlinear_i8(xq[j], wq, ws, a_absmax=b["amax"][i:i + 1], bias=bias, relu=True, out=b["q"][i + 1],
                                            out_absmax=b["amax"][i + 1:i + 2])
                continue
            for j, b in enumerate(bufs):
                hs[j], _ = K.qlinear_i8(xq[j], wq, ws, a_absmax=b["amax"][i:i + 1], bias=bias, relu=not last, out=b["h"][i],
                                        out_absmax=b["amax"][i + 1:i + 2] if not last else None)
                if keep:
                    kept[j].append((xq[j], hs[j]))
            if not last:
                combine(i + 1)
                for j, b in enumerate(bufs):
                    xq[j] = K.quantize_i8(hs[j], absmax_dev=b["amax"][i + 1:i + 2], out=b["q"][i + 1])
        return [(h, k) for h, k in zip(hs, kept)] if keep else hs
