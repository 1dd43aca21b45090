"""Evaluation of lazy `Tensor` graphs: eager (one kernel per primitive) and fused.

The fused path mirrors the reference fuser: starting from an output it grows a
region of elementwise primitives around at most ONE reduce
(csrc/compiler/scheduler.cpp:53-97), everything else (views, matmuls, other
reduces, inputs) is a leaf passed with its strides, `Fill` constants become
immediates (csrc/compiler/ir.cpp:235-255), and the region is lowered to the
linear program the kernels take (the counterpart of `graph_to_ir`,
csrc/compiler/ir.cpp:839-1286). Unlike the reference there is no
"fewer than 1024 reduced elements" refusal and shapes are runtime data, so one
compiled kernel serves every shape. The "one reduce per kernel" rule is lifted
for the two multi-reduce chains that matter on this path: a softmax or a
LayerNorm written from primitives is recognised in the graph and runs as ONE
row kernel. Outputs of one traced call that are elementwise results of the same
shape come out of one multi-output kernel (the reference's sibling outputs,
csrc/compiler/scheduler.cpp:229-256).

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

import builtins
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


def _const(node):
    """The value of a constant seen through broadcasts, else None."""
    node = _strip_broadcast(node)
    return node.attrs["value"] if node.op == "fill" else None


def _last_dims(axes, nd) -> bool:
    return len(axes) >= 1 and tuple(sorted(axes)) == tuple(range(nd - len(axes), nd))


def _match_softmax(node):
    """x when `node` is the softmax composite over the last axis written from primitives,
    exp(x - max(x)) / sum(exp(x - max(x))) (pequegrad/ops.py:259-267): two reduces and three elementwise passes that
    the reference's scheduler can only split (one reduce per kernel, csrc/compiler/scheduler.cpp:62-66) and that the
    row kernel computes in one read and one write of the tensor."""
    if node.op != "div" or node._buf is not None:
        return None
    e, den = node.args
    s = _strip_broadcast(den)
    if s.op != "sum" or s._buf is not None or s.args[0] is not e or not s.attrs["keepdims"] or tuple(s.attrs["axes"]) != (e.ndim - 1,):
        return None
    if e.op != "exp" or e._buf is not None or e.args[0].op != "sub" or e.args[0]._buf is not None:
        return None
    x, mb = e.args[0].args
    m = _strip_broadcast(mb)
    if m.op != "max_reduce" or m._buf is not None or m.args[0] is not x or not m.attrs["keepdims"] or tuple(m.attrs["axes"]) != (x.ndim - 1,):
        return None
    if x.dtype not in (torch.float32, torch.float16, torch.bfloat16) or x.ndim < 1:
        return None
    return x


def _match_centered(node):
    """(x, mean node) when `node` is x - mean(x, last dims, keepdim)."""
    if node.op != "sub" or node._buf is not None:
        return None
    x, mb = node.args
    mu = _strip_broadcast(mb)
    if mu.op != "mean" or mu._buf is not None or mu.args[0] is not x or not mu.attrs["keepdims"] or not _last_dims(mu.attrs["axes"], x.ndim):
        return None
    return x, mu


def _match_layernorm(node):
    """(x, weight, bias, eps, n) when `node` is the LayerNorm composite written from primitives,
    (x - mean) / (var + eps) ** 0.5 [* weight] [+ bias] with var = sum((x - mean) ** 2) / n over the last dims
    (pequegrad/ops.py:515-551, 480-501): three reduces in the reference's terms, one row kernel here."""
    weight = bias = None
    n0 = node
    if n0.op == "add" and n0._buf is None:
        for a, b in (n0.args, n0.args[::-1]):
            base = _strip_broadcast(b)
            if base.op not in _ELEMENTWISE and base.op not in _REDUCES and a.op in ("mul", "div") and a._buf is None:
                cand = (a, base)
                break
        else:
            return None
        n0, bias = cand
    if n0.op == "mul" and n0._buf is None:
        for a, b in (n0.args, n0.args[::-1]):
            base = _strip_broadcast(b)
            if base.op not in _ELEMENTWISE and base.op not in _REDUCES and a.op == "div" and a._buf is None:
                cand = (a, base)
                break
        else:
            return None
        n0, weight = cand
    if n0.op != "div" or n0._buf is not None:
        return None
    num, den = n0.args
    c = _match_centered(num)
    if c is None:
        return None
    x, mu = c
    sd = _strip_broadcast(den)
    if sd.op != "pow" or sd._buf is not None or _const(sd.args[1]) != 0.5:
        return None
    ve = sd.args[0]
    if ve.op != "add" or ve._buf is not None or _const(ve.args[1]) is None:
        return None
    eps, var = _const(ve.args[1]), ve.args[0]
    if var.op != "div" or var._buf is not None or _const(var.args[1]) is None:
        return None
    n, ss = _const(var.args[1]), var.args[0]
    if ss.op != "sum" or ss._buf is not None or not ss.attrs["keepdims"] or tuple(sorted(ss.attrs["axes"])) != tuple(sorted(mu.attrs["axes"])):
        return None
    sq = ss.args[0]
    if sq.op != "pow" or sq._buf is not None or _const(sq.args[1]) != 2.0:
        return None
    c2 = _match_centered(sq.args[0])
    if c2 is None or c2[0] is not x:
        return None
    k = len(mu.attrs["axes"])
    count = 1
    for d in x.shape[x.ndim - k:]:
        count *= d
    if float(n) != float(count) or x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        return None
    for t in (weight, bias):
        if t is not None and (tuple(t.shape[-k:]) != tuple(x.shape[-k:]) or any(d != 1 for d in t.shape[:-k]) or t.dtype != x.dtype):
            return None
    return x, weight, bias, float(eps), count


def _rows_of(buf: torch.Tensor, n: int) -> torch.Tensor:
    """`buf` as contiguous rows of n (a copy through the elementwise kernel only when the view is not contiguous)."""
    if not buf.is_contiguous():
        (buf,) = K.fused_elementwise([buf], [("LOAD", 0)])
    return buf.reshape(-1, n)


def _emit_leaf(node: T.Tensor, fuse: bool) -> torch.Tensor:
    evaluate(node, fuse)
    return node._buf


def _subtree_size(node, shape, memo=None) -> int:
    """Instructions the fusable subtree under `node` would add to a region (shared nodes counted once)."""
    memo = {} if memo is None else memo
    if id(node) in memo:
        return 0
    memo[id(node)] = True
    if node._buf is not None or node.op not in _ELEMENTWISE or node.shape != shape or node.op == "fill":
        return 1
    return 1 + builtins.sum(_subtree_size(a, shape, memo) for a in node.args)


class _Region:
    """Collects the program and the leaf tensors of one fused region. The C ABI takes at most `max_instrs`
    instructions and `max_inputs` operands per region: a node is fused only if, with everything under it, the
    region still fits; otherwise its largest operand subtrees are cut off into leaves of their own (which are
    evaluated as separate regions), largest first, until it does."""

    def __init__(self, shape, fuse, max_instrs=MAX_REGION_INSTRS, max_inputs=L.MAX_INPUTS):
        self.shape, self.fuse = tuple(shape), fuse
        self.max_instrs, self.max_inputs = max_instrs, max_inputs
        self.prog, self.inputs, self.memo, self.leaf_ix = [], [], {}, {}

    def _snapshot(self):
        return len(self.prog), len(self.inputs), dict(self.memo), dict(self.leaf_ix)

    def _restore(self, snap):
        n_prog, n_in, memo, leaf_ix = snap
        del self.prog[n_prog:]
        del self.inputs[n_in:]
        self.memo, self.leaf_ix = memo, leaf_ix

    def fits(self) -> bool:
        return len(self.prog) <= self.max_instrs and len(self.inputs) <= self.max_inputs

    def leaf(self, node):
        buf = _emit_leaf(node, self.fuse)
        key = (buf.data_ptr(), tuple(buf.shape), tuple(buf.stride()), buf.dtype)
        if key not in self.leaf_ix:  # duplicates are dropped from the argument list (csrc/compiler/ir.cpp:950-965)
            self.leaf_ix[key] = len(self.inputs)
            self.inputs.append(buf)
        self.prog.append(("LOAD", self.leaf_ix[key]))
        return len(self.prog) - 1

    def _fusable(self, node) -> bool:
        if node._buf is not None or node.op not in _ELEMENTWISE or node.shape != self.shape:
            return False
        return node.op != "astype" or node.attrs["dtype"] in _CAST

    def emit(self, node, stop=None, forced_leaves=frozenset()):
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
        elif id(node) in forced_leaves or not self._fusable(node) or _match_linear(node, self.fuse) is not None:
            # (act(x @ w + bias) inside a larger region: bias and activation stay in the GEMM)
            return self._as_leaf(node)
        else:
            return self._emit_op(node, stop)
        self.memo[id(node)] = ix
        return ix

    def _emit_op(self, node, stop):
        forced = set()
        while True:
            snap = self._snapshot()
            ops = [self.emit(a, stop, frozenset(forced)) for a in node.args]
            if node.op in T.BINARY:
                self.prog.append((T.BINARY[node.op], ops[0], ops[1]))
            elif node.op in T.UNARY:
                self.prog.append((T.UNARY[node.op], ops[0]))
            elif node.op == "where":
                self.prog.append(("WHERE", ops[0], ops[1], ops[2]))
            else:  # astype
                self.prog.append((_CAST[node.attrs["dtype"]], ops[0]))
            if self.fits():
                ix = len(self.prog) - 1
                self.memo[id(node)] = ix
                return ix
            # too large: cut the biggest operand subtree that is still fused off into a leaf and try again
            self._restore(snap)
            cands = [a for a in node.args if id(a) not in forced and a is not stop and self._fusable(a)]
            if not cands:
                if snap[0] == 0:
                    raise RuntimeError("fuser: a single operation does not fit the region limits")  # cannot happen: <= 4 instructions
                return self._as_leaf(node)  # the region was already nearly full: this node starts a region of its own
            forced.add(id(builtins.max(cands, key=lambda a: _subtree_size(a, self.shape))))

    def _as_leaf(self, node):
        ix = self.leaf(node)
        self.memo[id(node)] = ix
        return ix


def _find_reduce(node, shape, seen=None):
    """First fusable reduce reachable from `node` through elementwise nodes of the output shape."""
    seen = set() if seen is None else seen
    if id(node) in seen or node._buf is not None:
        return None
    seen.add(id(node))
    if node.op in ("sum", "mean", "max_reduce") and node.shape == shape:
        return node
    if node.op in _ELEMENTWISE and node.shape == shape:
        for a in node.args:
            r = _find_reduce(a, shape, seen)
            if r is not None:
                return r
    return None


def _eval_elementwise(nodes, mode):
    """One fused elementwise kernel for `nodes` (same shape; more than one = the sibling outputs of a region,
    csrc/compiler/scheduler.cpp:229-256). Returns the nodes that did not fit and must be evaluated on their own."""
    reg = _Region(nodes[0].shape, mode)
    outs, left = [], []
    for n in nodes:
        snap = reg._snapshot()
        try:
            ix = reg.emit(n)
        except RuntimeError:
            ix = None
        if ix is None or not reg.fits() or len(outs) >= 4:
            reg._restore(snap)
            left.append(n)
            continue
        outs.append((n, ix))
    if not outs:
        return left
    bufs = K.fused_elementwise(reg.inputs, reg.prog, shape=nodes[0].shape, out_dtypes=[n.dtype for n, _ in outs], out_vals=[ix for _, ix in outs])
    for (n, _), b in zip(outs, bufs):
        n._buf = b
    return left


def _siblings(node):
    """Other outputs of the same traced call that can share a kernel with `node`: unevaluated elementwise results of
    the same shape with no reduce of their own."""
    sib = [s for s in getattr(node, "_siblings", ()) if s is not node and s._buf is None and s.shape == node.shape
           and s.op in _ELEMENTWISE and s.op != "fill" and _find_reduce(s, s.shape) is None and _match_linear(s, JIT) is None]
    return sib[:3]


def _eval_fused(node: T.Tensor, mode: int = JIT):
    red = node if node.op in _REDUCES else _find_reduce(node, node.shape)
    if red is not None:
        x = red.args[0]
        pro = _Region(x.shape, mode)
        pro.emit(x)
        epi_prog, epi_inputs = [], []
        fused_epilogue = True
        if red is not node:
            epi = _Region(node.shape, mode)
            epi.emit(node, stop=red)
            # the reduce may have been cut out of the epilogue by the region limits: then it is a plain leaf of `node`
            fused_epilogue = any(i[0] == "ACC" for i in epi.prog)
            epi_prog = epi.prog
            keep = K.reduced_shape(x.shape, red.attrs["axes"], True)
            epi_inputs = [b.reshape(keep) if b.dim() != len(keep) else b for b in epi.inputs]
        if fused_epilogue and red._buf is None:
            out = K.fused_reduce(pro.inputs, T.REDUCE[red.op], red.attrs["axes"], red.attrs["keepdims"], pro.prog, epi_prog, epi_inputs,
                                 out_dtype=node.dtype)
            node._buf = out.view(node.shape)
            return
    left = _eval_elementwise([node] + _siblings(node), mode)
    for n in left:
        if n is node:
            raise RuntimeError("fuser: could not place the output in a region")
    # siblings that did not fit are evaluated when they are asked for


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
    elif fuse and _match_softmax(node) is not None:
        # a softmax written from primitives: one row kernel instead of a region per reduce
        x = _emit_leaf(_match_softmax(node), fuse)
        node._buf = K.softmax_rows(_rows_of(x, x.shape[-1])).view(node.shape)
    elif fuse and _match_layernorm(node) is not None:
        xn, w, b, eps, n = _match_layernorm(node)
        x, g, be = (None if a is None else _emit_leaf(a, fuse) for a in (xn, w, b))
        node._buf = K.layernorm_rows(_rows_of(x, n), g if g is None else g.reshape(-1).contiguous(), be if be is None else be.reshape(-1).contiguous(),
                                     eps).view(node.shape)
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
        tens = [o for o in outs if isinstance(o, T.Tensor)]
        for o in tens:
            o._jit = mode
            o._siblings = tens  # outputs of one call may come out of one kernel (multi-output regions)
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
