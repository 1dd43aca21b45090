"""Evaluation of lazy `Tensor` graphs: eager (one kernel per primitive) and fused.

The fused path mirrors the reference fuser: starting from an output it grows a
region of elementwise primitives around at most ONE reduce
(csrc/compiler/scheduler.cpp:53-97), everything else (views, matmuls, other
reduces, inputs) is a leaf passed with its strides, `Fill` constants become
immediates (csrc/compiler/ir.cpp:235-255), and the region is lowered to the
linear program the kernels take (the counterpart of `graph_to_ir`,
csrc/compiler/ir.cpp:839-1286). Unlike the reference there is no
"fewer than 1024 reduced elements" refusal and shapes are runtime data, so one
compiled kernel serves every shape.

Two graph rewrites of the reference run here as well:
  * the fused-linear pattern (`recursive_fused_linear`, csrc/compiler/compile.hpp;
    FusedLinearBiasAct, csrc/cuda/other.cu:19-166): `act(x @ w + bias)` becomes ONE
    tensor-core GEMM whose epilogue adds the bias and applies ReLU / tanh-GELU;
  * `amp(f)` (pequegrad/transforms/automatic_mixed_precision.py:37-146): matmuls of
    fp32 operands run as fp16-in / fp32-accumulate GEMMs with an fp32 result, the
    `(xw + b).relu()` pattern rides in that GEMM's epilogue, and fp32 -> fp16 -> fp32
    cast pairs (and the reverse) are dropped.
"""
from __future__ import annotations

import contextlib

import torch

from . import _lib as L
from . import kernels as K
from . import tensor as T

MAX_REGION_INSTRS = 28
_ELEMENTWISE = set(T.BINARY) | set(T.UNARY) | {"where", "astype", "fill"}
_REDUCES = {"sum", "mean", "max_reduce", "argmax"}
_CAST = {torch.float16: "CAST_F16", torch.float32: "CAST_F32", torch.int32: "CAST_I32", torch.bfloat16: "CAST_BF16"}
_fuse_composites = False
EAGER, JIT, AMP = 0, 1, 2  # evaluation modes handed down the graph walk


@contextlib.contextmanager
def fusing_composites():
    global _fuse_composites
    old, _fuse_composites = _fuse_composites, True
    try:
        yield
    finally:
        _fuse_composites = old


def _view(node: T.Tensor, buf: torch.Tensor) -> torch.Tensor:
    if node.op == "permute":
        return buf.permute(node.attrs["dims"])
    if node.op == "broadcast_to":
        return buf.expand(node.attrs["shape"])
    shape = node.attrs["shape"]
    try:
        return buf.view(shape)
    except RuntimeError:
        # a reshape that needs a copy: materialise through the elementwise kernel (as_contiguous, csrc/cuda/view_helpers.cu:11-95)
        (c,) = K.fused_elementwise([buf], [("LOAD", 0)])
        return c.view(shape)


def _matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    # any view goes: the library reads K-major operands in place and re-lays-out the others itself
    if b.dim() > 2 and b.shape[:-2] != a.shape[:-2]:
        batch = torch.broadcast_shapes(a.shape[:-2], b.shape[:-2])
        a, b = a.expand(batch + a.shape[-2:]), b.expand(batch + b.shape[-2:])
    return K.matmul(a, b)


def _strip_broadcast(node):
    while node.op == "broadcast_to" and node._buf is None:
        node = node.args[0]
    return node


def _is_zero(node) -> bool:
    node = _strip_broadcast(node)
    return node.op == "fill" and node.attrs["value"] == 0.0


def _match_linear(node, mode):
    """(matmul node, bias node or None, act) when `node` is `act(x @ w + bias)` with a bias over the last dim and
    act in {none, ReLU as max(., 0), the tanh-GELU composite}; None when there is nothing to fold into the GEMM."""
    act, n = 0, node
    if "gelu_of" in n.attrs and (mode == AMP or n.dtype in (torch.float16, torch.bfloat16)):
        # the epilogue's GELU uses the hardware tanh approximation: good to ~1e-3, so fp32 results keep the exact chain
        act, n = 2, n.attrs["gelu_of"]
    elif n.op == "max" and n._buf is None and len(n.args) == 2:
        a, b = n.args
        if _is_zero(b):
            act, n = 1, a
        elif _is_zero(a):
            act, n = 1, b
    bias = None
    if n.op == "add" and n._buf is None:
        for mm, bb in (n.args, n.args[::-1]):
            base = _strip_broadcast(bb)
            if (mm.op == "matmul" and mm._buf is None and base.op != "fill" and base.ndim >= 1 and base.shape[-1] == mm.shape[-1]
                    and all(d == 1 for d in base.shape[:-1])):
                bias, n = base, mm
                break
        else:
            return None
    if n.op != "matmul" or n._buf is not None or (bias is None and act == 0):
        return None
    return n, bias, act


def _half_operands(a: torch.Tensor, b: torch.Tensor):
    """fp32 matmul operands as fp16, each cast in one pass: `a` row-major, `b` straight into the [.., N, K]
    array whose transposed view the GEMM reads in place (no second re-layout of the weight)."""
    (a16,) = K.fused_elementwise([a], [("LOAD", 0)], out_dtypes=[torch.float16])
    (bt16,) = K.fused_elementwise([b.transpose(-2, -1)], [("LOAD", 0)], out_dtypes=[torch.float16])
    return a16, bt16.transpose(-2, -1)


def _linear(mm, bias, act, mode, out_dtype):
    a, b = (_emit_leaf(t, mode) for t in mm.args)
    bias_buf = None if bias is None else _emit_leaf(bias, mode).reshape(-1)
    if mode == AMP and a.dtype == torch.float32 and b.dtype == torch.float32:
        a, b = _half_operands(a, b)
        if bias_buf is not None and bias_buf.dtype != torch.float32:
            (bias_buf,) = K.fused_elementwise([bias_buf], [("LOAD", 0)], out_dtypes=[torch.float32])
    if b.dim() > 2 and b.shape[:-2] != a.shape[:-2]:
        batch = torch.broadcast_shapes(a.shape[:-2], b.shape[:-2])
        a, b = a.expand(batch + a.shape[-2:]), b.expand(batch + b.shape[-2:])
    return K.matmul(a, b, bias=bias_buf, act=act, out_dtype=out_dtype)


def _emit_leaf(node: T.Tensor, fuse: bool) -> torch.Tensor:
    evaluate(node, fuse)
    return node._buf


class _Region:
    """Collects the program and the leaf tensors of one fused region."""

    def __init__(self, shape, fuse):
        self.shape, self.fuse = tuple(shape), fuse
        self.prog, self.inputs, self.memo, self.leaf_ix = [], [], {}, {}

    def leaf(self, node):
        buf = _emit_leaf(node, self.fuse)
        key = (buf.data_ptr(), tuple(buf.shape), tuple(buf.stride()), buf.dtype)
        if key not in self.leaf_ix:  # duplicates are dropped from the argument list (csrc/compiler/ir.cpp:950-965)
            self.leaf_ix[key] = len(self.inputs)
            self.inputs.append(buf)
        self.prog.append(("LOAD", self.leaf_ix[key]))
        return len(self.prog) - 1

    def emit(self, node, stop=None):
        """Value index of `node`; `stop` is the reduce node whose result reads as ACC."""
        if id(node) in self.memo:
            return self.memo[id(node)]
        if node is stop:
            self.prog.append(("ACC",))
            ix = len(self.prog) - 1
        elif node.op == "fill":
            self.prog.append(("IMM", 0, 0, 0, node.attrs["value"]))
            ix = len(self.prog) - 1
        elif node.op == "broadcast_to" and node.args[0].op == "fill":
            ix = self.emit(node.args[0], stop)  # a constant seen through a broadcast is still an immediate
        elif _match_linear(node, self.fuse) is not None:
            return self._as_leaf(node)  # act(x @ w + bias) inside a larger region: bias and activation stay in the GEMM
        elif (node.op in _ELEMENTWISE and node._buf is None and node.shape == self.shape and len(self.prog) < MAX_REGION_INSTRS
              and (len(self.inputs) < L.MAX_INPUTS - 1)):
            if node.op in T.BINARY:
                a, b = self.emit(node.args[0], stop), self.emit(node.args[1], stop)
                self.prog.append((T.BINARY[node.op], a, b))
            elif node.op in T.UNARY:
                self.prog.append((T.UNARY[node.op], self.emit(node.args[0], stop)))
            elif node.op == "where":
                c, a, b = (self.emit(t, stop) for t in node.args)
                self.prog.append(("WHERE", c, a, b))
            else:  # astype
                if node.attrs["dtype"] not in _CAST:
                    return self._as_leaf(node)
                a = self.emit(node.args[0], stop)
                self.prog.append((_CAST[node.attrs["dtype"]], a))
            ix = len(self.prog) - 1
        else:
            return self._as_leaf(node)
        self.memo[id(node)] = ix
        return ix

    def _as_leaf(self, node):
        ix = self.leaf(node)
        self.memo[id(node)] = ix
        return ix


def _find_reduce(node, shape, seen=None):
    """First fusable reduce reachable from `node` through elementwise nodes of the output shape."""
    if node._buf is not None:
        return None
    if node.op in ("sum", "mean", "max_reduce") and node.shape == shape:
        return node
    if node.op in _ELEMENTWISE and node.shape == shape:
        for a in node.args:
            r = _find_reduce(a, shape)
            if r is not None:
                return r
    if node.op == "broadcast_to" and node.args[0].op == "fill":
        return None
    return None


def _eval_fused(node: T.Tensor, mode: int = JIT):
    red = node if node.op in _REDUCES else _find_reduce(node, node.shape)
    if red is None:
        reg = _Region(node.shape, mode)
        reg.emit(node)
        if not reg.inputs:  # constants only
            (out,) = K.fused_elementwise([], reg.prog, shape=node.shape, out_dtypes=[node.dtype])
        else:
            (out,) = K.fused_elementwise(reg.inputs, reg.prog, shape=node.shape, out_dtypes=[node.dtype])
        node._buf = out
        return
    x = red.args[0]
    pro = _Region(x.shape, mode)
    pro.emit(x)
    epi_prog, epi_inputs = [], []
    if red is not node:
        epi = _Region(node.shape, mode)
        epi.emit(node, stop=red)
        epi_prog = epi.prog
        keep = K.reduced_shape(x.shape, red.attrs["axes"], True)
        epi_inputs = [b.reshape(keep) if b.dim() != len(keep) else b for b in epi.inputs]
    out = K.fused_reduce(pro.inputs, T.REDUCE[red.op], red.attrs["axes"], red.attrs["keepdims"], pro.prog, epi_prog, epi_inputs,
                         out_dtype=node.dtype)
    node._buf = out.view(node.shape)


def _eval_eager(node: T.Tensor):
    args = [_emit_leaf(a, False) for a in node.args]
    if node.op in T.BINARY:
        (node._buf,) = K.fused_elementwise(args, [("LOAD", 0), ("LOAD", 1), (T.BINARY[node.op], 0, 1)])
    elif node.op in T.UNARY:
        (node._buf,) = K.fused_elementwise(args, [("LOAD", 0), (T.UNARY[node.op], 0)])
    elif node.op == "where":
        (node._buf,) = K.fused_elementwise(args, [("LOAD", 0), ("LOAD", 1), ("LOAD", 2), ("WHERE", 0, 1, 2)], out_dtypes=[node.dtype])
    elif node.op == "astype":
        (node._buf,) = K.fused_elementwise(args, [("LOAD", 0)], out_dtypes=[node.dtype])
    else:
        node._buf = K.fused_reduce(args, T.REDUCE[node.op], node.attrs["axes"], node.attrs["keepdims"])


def evaluate(node: T.Tensor, fuse: bool = False):
    """Materialise `node` (and what it needs) on the device."""
    if node._buf is not None:
        return
    fuse = max(int(fuse), int(getattr(node, "_jit", 0)))
    lin = _match_linear(node, fuse) if fuse else None
    if lin is not None:
        node._buf = _linear(*lin, fuse, node.dtype)
    elif (fuse == AMP and node.op == "astype" and node.args[0].op == "astype" and node.args[0]._buf is None
          and node.args[0].args[0].dtype == node.dtype and {node.dtype, node.args[0].dtype} == {torch.float16, torch.float32}):
        # astype_f32_f16_f32 / astype_f16_f32_f16 (automatic_mixed_precision.py:83-113): the pair is dropped
        node._buf = _emit_leaf(node.args[0].args[0], fuse)
    elif node.op in T.VIEW_OPS:
        node._buf = _view(node, _emit_leaf(node.args[0], fuse))
    elif node.op == "fill":
        (node._buf,) = K.fused_elementwise([], [("IMM", 0, 0, 0, node.attrs["value"])], shape=node.shape, out_dtypes=[node.dtype])
    elif node.op == "matmul":
        a, b = _emit_leaf(node.args[0], fuse), _emit_leaf(node.args[1], fuse)
        if fuse == AMP and a.dtype == torch.float32 and b.dtype == torch.float32:
            node._buf = _linear(node, None, 0, fuse, torch.float32)  # matmul_amp: fp16 operands, fp32 accumulator and result
        else:
            node._buf = _matmul(a, b)
    elif node.op == "attention":
        q, k, v = (_emit_leaf(a, fuse) for a in node.args)
        node._buf = K.attention(q, k, v, scale=node.attrs["scale"], causal=node.attrs["causal"])
    elif node.op == "softmax_rows":
        node._buf = K.softmax_rows(_emit_leaf(node.args[0], fuse).contiguous(), node.attrs.get("causal", False))
    elif node.op == "layernorm_rows":
        x, g, b = (None if a is None else _emit_leaf(a, fuse) for a in node.attrs["operands"])
        rows = x.reshape(-1, node.attrs["n"])
        node._buf = K.layernorm_rows(rows, g if g is None else g.reshape(-1), b if b is None else b.reshape(-1), node.attrs["eps"]).view(node.shape)
    elif fuse:
        _eval_fused(node, fuse)
    else:
        _eval_eager(node)
    node.args = ()  # evaluated nodes drop their graph, as the reference frees children after eval


def _traced(f, mode):
    def wrapped(*args, **kwargs):
        with fusing_composites():
            out = f(*args, **kwargs)
        outs = out if isinstance(out, (tuple, list)) else (out,)
        for o in outs:
            if isinstance(o, T.Tensor):
                o._jit = mode
        return out
    return wrapped


def jit(f):
    """`pg.jit`: the outputs of `f` are evaluated through the fuser (pequegrad/transforms/compile.py:84-236).
    Tracing is just running `f` on lazy tensors; there is no per-shape compilation to cache."""
    return _traced(f, JIT)


def amp(f):
    """`pg.amp`: automatic mixed precision (pequegrad/transforms/automatic_mixed_precision.py:145-146). Every
    matmul of fp32 operands runs as an fp16 GEMM and returns fp32; where the reference's `cublasHgemm` accumulates
    in fp16 (csrc/cuda/matmul.cu:140-155), the accumulator here is fp32 in tensor memory, and the bias + ReLU of
    `bias_relu_add_amp` are applied to that fp32 accumulator in the GEMM's epilogue instead of in fp16."""
    return _traced(f, AMP)
