"""Calls into the C ABI with torch CUDA tensors as device memory.

torch is plumbing here: it owns allocations and the current stream. Every
function below builds `pgb_tensor` descriptors (pointer, shape, BYTE strides —
the reference's `View`, csrc/tensor.hpp:263-273) and enqueues exactly the
kernels of `libpgb200.so`; nothing is computed by torch.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from . import _lib as L

_TORCH2PGB = {
    torch.int32: L.I32, torch.float16: L.F16, torch.float32: L.F32,
    torch.float64: L.F64, torch.int8: L.I8, torch.bfloat16: L.BF16,
}


def pgb_dtype(dt: torch.dtype) -> int:
    try:
        return _TORCH2PGB[dt]
    except KeyError:
        raise RuntimeError(f"dtype {dt} is not supported by pgb200") from None


def desc(t: torch.Tensor) -> L.PgbTensor:
    """Descriptor of a (possibly permuted / expanded / sliced) CUDA tensor view."""
    if not t.is_cuda:
        raise RuntimeError("pgb200 kernels need CUDA tensors: there is no CPU path")
    es = t.element_size()
    return L.make_tensor(t.data_ptr(), pgb_dtype(t.dtype), t.shape, [s * es for s in t.stride()])


def _arr(descs: Sequence[L.PgbTensor]):
    a = (L.PgbTensor * max(len(descs), 1))()
    for i, d in enumerate(descs):
        a[i] = d
    return a


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def reduced_shape(shape, axes, keepdims):
    nd = len(shape)
    ax = sorted({a + nd if a < 0 else a for a in axes})
    if keepdims:
        return tuple(1 if i in ax else s for i, s in enumerate(shape))
    return tuple(s for i, s in enumerate(shape) if i not in ax)


def fused_reduce(inputs: Sequence[torch.Tensor], op: int, axes: Sequence[int], keepdims: bool = False,
                 prologue=(), epilogue=(), epi_inputs: Sequence[torch.Tensor] = (), out_dtype=None,
                 out: torch.Tensor | None = None, workspace: torch.Tensor | None = None) -> torch.Tensor:
    """prologue / epilogue: lists of (opname, a, b, c, imm); see include/pgb200.h."""
    x0 = inputs[0]
    axes = list(axes)
    if out is None:
        if out_dtype is None:
            out_dtype = torch.int32 if op == L.ARGMAX else x0.dtype
        out = torch.empty(reduced_shape(x0.shape, axes, keepdims), dtype=out_dtype, device=x0.device)
    ins = _arr([desc(t) for t in inputs])
    eins = _arr([desc(t) for t in epi_inputs])
    pro, npro = L.make_program(list(prologue))
    epi, nepi = L.make_program(list(epilogue))
    ax = (C.c_int32 * max(len(axes), 1))(*axes)
    od = desc(out)
    ws_ptr, ws_bytes = (None, 0) if workspace is None else (workspace.data_ptr(), workspace.numel() * workspace.element_size())
    with torch.cuda.device(x0.device):
        st = L.lib().pgb_fused_reduce(ins, len(inputs), C.byref(od), op, ax, len(axes), pro, npro, eins, len(epi_inputs), epi, nepi,
                                      ws_ptr, ws_bytes, _stream())
    L.check(st)
    return out


def fused_reduce_noalloc(inputs: Sequence[torch.Tensor], op: int, axes: Sequence[int], out: torch.Tensor, prologue=(), epilogue=(),
                         epi_inputs: Sequence[torch.Tensor] = ()) -> torch.Tensor:
    """`fused_reduce` through the entry point that allocates nothing on the device: the caller
    passes the output, split reductions use the library's built-in scratch array. For callers
    that own all device memory themselves or may not call an allocator on their hot path."""
    axes = list(axes)
    ins = _arr([desc(t) for t in inputs])
    eins = _arr([desc(t) for t in epi_inputs])
    pro, npro = L.make_program(list(prologue))
    epi, nepi = L.make_program(list(epilogue))
    ax = (C.c_int32 * max(len(axes), 1))(*axes)
    od = desc(out)
    with torch.cuda.device(inputs[0].device):
        st = L.lib().pgb_fused_reduce_noalloc(ins, len(inputs), C.byref(od), op, ax, len(axes), pro, npro, eins, len(epi_inputs), epi, nepi,
                                              _stream())
    L.check(st)
    return out


def reduce_workspace_bytes(x_desc_or_tensor, out_shape, op: int, axes: Sequence[int], out_dtype=torch.float32) -> int:
    d = x_desc_or_tensor if isinstance(x_desc_or_tensor, L.PgbTensor) else desc(x_desc_or_tensor)
    es = torch.empty((), dtype=out_dtype).element_size()
    strides, acc = [], es
    for s in reversed(out_shape):
        strides.append(acc)
        acc *= s
    od = L.make_tensor(256, pgb_dtype(out_dtype), out_shape, list(reversed(strides)))
    ax = (C.c_int32 * max(len(axes), 1))(*axes)
    n = C.c_size_t(0)
    L.check(L.lib().pgb_fused_reduce_workspace(_arr([d]), 1, C.byref(od), op, ax, len(axes), C.byref(n)))
    return int(n.value)


def describe_reduce(in_descs: Sequence[L.PgbTensor], out_desc: L.PgbTensor, op: int, axes: Sequence[int], prologue=()) -> str:
    """The planner's choice for these arguments; needs no GPU."""
    pro, npro = L.make_program(list(prologue))
    ax = (C.c_int32 * max(len(axes), 1))(*axes)
    buf = C.create_string_buffer(512)
    L.check(L.lib().pgb_fused_reduce_describe(_arr(list(in_descs)), len(in_descs), C.byref(out_desc), op, ax, len(axes), pro, npro, buf, 512))
    return buf.value.decode()


def fused_elementwise(inputs: Sequence[torch.Tensor], prog, shape=None, out_dtypes=None, out_vals=None, outs=None) -> list:
    """Evaluate `prog` per element; inputs must already be views of `shape`. `outs`: caller-allocated outputs."""
    if shape is None:
        shape = tuple(outs[0].shape) if outs else tuple(inputs[0].shape)
    n = len(prog)
    if out_vals is None:
        out_vals = [n - 1]
    dev = inputs[0].device if inputs else torch.device("cuda")
    if outs is None:
        if out_dtypes is None:
            out_dtypes = [inputs[0].dtype] * len(out_vals)
        outs = [torch.empty(shape, dtype=dt, device=dev) for dt in out_dtypes]
    p, n = L.make_program(list(prog))
    ov = (C.c_int16 * len(out_vals))(*out_vals)
    with torch.cuda.device(dev):
        st = L.lib().pgb_fused_elementwise(_arr([desc(t) for t in inputs]), len(inputs), _arr([desc(o) for o in outs]), len(outs), p, n, ov,
                                           _stream())
    L.check(st)
    return outs


def softmax_rows(x: torch.Tensor, causal: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
    y = torch.empty_like(x, memory_format=torch.contiguous_format) if out is None else out
    xd, yd = desc(x), desc(y)
    with torch.cuda.device(x.device):
        st = L.lib().pgb_softmax_rows(C.byref(xd), C.byref(yd), 1 if causal else 0, _stream())
    L.check(st)
    return y


def layernorm_rows(x: torch.Tensor, gamma: torch.Tensor | None, beta: torch.Tensor | None, eps: float = 1e-5,
                   out: torch.Tensor | None = None) -> torch.Tensor:
    y = torch.empty_like(x, memory_format=torch.contiguous_format) if out is None else out
    xd, yd = desc(x), desc(y)
    gd = desc(gamma) if gamma is not None else None
    bd = desc(beta) if beta is not None else None
    with torch.cuda.device(x.device):
        st = L.lib().pgb_layernorm_rows(C.byref(xd), C.byref(gd) if gd else None, C.byref(bd) if bd else None, eps, C.byref(yd), _stream())
    L.check(st)
    return y


def embedding_rows(ids: torch.Tensor, wte: torch.Tensor, wpe: torch.Tensor | None, T: int) -> torch.Tensor:
    """out[r] = wte[ids[r]] + wpe[r % T]; ids int32 of any shape, result ids.shape + (C,)."""
    out = torch.empty(tuple(ids.shape) + (wte.shape[1],), dtype=wte.dtype, device=wte.device)
    idd, td, od = desc(ids), desc(wte), desc(out)
    pd = desc(wpe) if wpe is not None else None
    with torch.cuda.device(wte.device):
        st = L.lib().pgb_embedding_rows(C.byref(idd), C.byref(td), C.byref(pd) if pd else None, T, C.byref(od), _stream())
    L.check(st)
    return out


def _ref(t):
    if t is None:
        return None
    d = desc(t)
    return C.byref(d), d  # keep the descriptor alive alongside the reference


def matmul(a: torch.Tensor, b: torch.Tensor, bias: torch.Tensor | None = None, act: int = 0, residual: torch.Tensor | None = None,
           out: torch.Tensor | None = None, out_dtype=None, alpha: float = 1.0) -> torch.Tensor:
    """out = act(a @ b + bias) + residual on the tensor cores. `b` is the [.., K, N] operand as a
    view whose K dim is contiguous (e.g. `w_t.T` for a weight stored as [N, K])."""
    if out is None:
        shape = tuple(a.shape[:-1]) + (b.shape[-1],)
        out = torch.empty(shape, dtype=out_dtype or a.dtype, device=a.device)
    ad, bd, od = desc(a), desc(b), desc(out)
    bi, rs = _ref(bias), _ref(residual)
    with torch.cuda.device(a.device):
        st = L.lib().pgb_matmul(C.byref(ad), C.byref(bd), bi[0] if bi else None, act, alpha, rs[0] if rs else None, C.byref(od), _stream())
    L.check(st)
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None = None, causal: bool = False,
              out: torch.Tensor | None = None) -> torch.Tensor:
    """softmax(scale * q @ k^T [+ causal mask]) @ v in one kernel. q [.., T, 64], k / v [.., Tk, 64] (views with a
    contiguous last dim); `out` may be a view too (e.g. heads written straight into a [B, T, H*64] buffer)."""
    if scale is None:
        scale = float(q.shape[-1]) ** -0.5
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    qd, kd, vd, od = desc(q), desc(k), desc(v), desc(out)
    with torch.cuda.device(q.device):
        st = L.lib().pgb_attention(C.byref(qd), C.byref(kd), C.byref(vd), scale, 1 if causal else 0, C.byref(od), _stream())
    L.check(st)
    return out


def absmax(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    if out is None:
        out = torch.empty(1, dtype=torch.float32, device=x.device)
    xd = desc(x)
    with torch.cuda.device(x.device):
        st = L.lib().pgb_absmax_f32(C.byref(xd), out.data_ptr(), _stream())
    L.check(st)
    return out


def quantize_i8(x: torch.Tensor, absmax_dev: torch.Tensor | None = None, scale: float = 0.0, out: torch.Tensor | None = None) -> torch.Tensor:
    if out is None:
        out = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    xd, qd = desc(x), desc(out)
    with torch.cuda.device(x.device):
        st = L.lib().pgb_quantize_i8(C.byref(xd), absmax_dev.data_ptr() if absmax_dev is not None else None, scale, C.byref(qd), _stream())
    L.check(st)
    return out


def qlinear_i8(a: torch.Tensor, w: torch.Tensor, w_scale: torch.Tensor, a_scale: float = 0.0, a_absmax: torch.Tensor | None = None,
               bias: torch.Tensor | None = None, relu: bool = False, out: torch.Tensor | None = None, out_dtype=torch.float32,
               want_acc: bool = False, out_absmax: torch.Tensor | None = None, want_out: bool = True):
    """Returns (out, acc_i32 or None). a [M,K] int8, w [N,K] int8, w_scale [N] f32 on the device."""
    M, N = a.shape[0], w.shape[0]
    if out is None and want_out:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    acc = torch.empty((M, N), dtype=torch.int32, device=a.device) if want_acc else None
    ad, wd = desc(a), desc(w)
    bi, oo, ac = _ref(bias), _ref(out), _ref(acc)
    with torch.cuda.device(a.device):
        st = L.lib().pgb_qlinear_i8(C.byref(ad), C.byref(wd), w_scale.data_ptr(), a_scale, a_absmax.data_ptr() if a_absmax is not None else None,
                                    bi[0] if bi else None, 1 if relu else 0, oo[0] if oo else None, ac[0] if ac else None,
                                    out_absmax.data_ptr() if out_absmax is not None else None, _stream())
    L.check(st)
    return out, acc


def device_error(reset: bool = True) -> int:
    """The error word of the kernels' bounded waits: 0, or (role << 16) | block of the first wait that ran out."""
    code = C.c_int(0)
    st = L.lib().pgb_device_error(C.byref(code), 1 if reset else 0)
    if st not in (L.OK, L.ERR_TIMEOUT):
        L.check(st)
    return code.value


def gemm_pair_mode(mode: int) -> int:
    """0: every GEMM on the one-CTA kernel; 1: CTA pairs where they measured faster (the default). Returns the previous mode."""
    return L.lib().pgb_gemm_pair_mode(mode)


def gemm_wait_drill(polls: int, skip_loads: bool = True) -> None:
    """The next tensor-core GEMM of this thread polls each wait at most `polls` times; with `skip_loads` its producer
    loads nothing, so a wait runs out and the kernel reports it through `device_error` (nothing faults or hangs)."""
    L.check(L.lib().pgb_gemm_wait_drill(polls, 1 if skip_loads else 0))


class PreparedReduce:
    """A fused reduce with its descriptors and programs built once, so that a
    call is one C-ABI invocation (what the reference's `Compiled` primitive
    does by baking shapes into the kernel, csrc/compiler/ir.cpp:975-985)."""

    def __init__(self, inputs: Sequence[torch.Tensor], op: int, axes: Sequence[int], keepdims: bool = False, prologue=(),
                 epilogue=(), out: torch.Tensor | None = None, out_dtype=None, workspace: torch.Tensor | None = None):
        x0 = inputs[0]
        self.inputs = list(inputs)
        self.device = x0.device
        axes = list(axes)
        if out is None:
            if out_dtype is None:
                out_dtype = torch.int32 if op == L.ARGMAX else x0.dtype
            out = torch.empty(reduced_shape(x0.shape, axes, keepdims), dtype=out_dtype, device=x0.device)
        self.out = out
        self._ins = _arr([desc(t) for t in inputs])
        self._n_in = len(inputs)
        self._od = desc(out)
        self._op = op
        self._ax = (C.c_int32 * max(len(axes), 1))(*axes)
        self._n_ax = len(axes)
        self._pro, self._npro = L.make_program(list(prologue))
        self._epi, self._nepi = L.make_program(list(epilogue))
        self._none = _arr([])
        n = C.c_size_t(0)
        L.check(L.lib().pgb_fused_reduce_workspace(self._ins, self._n_in, C.byref(self._od), op, self._ax, self._n_ax, C.byref(n)))
        self.workspace_bytes = int(n.value)
        if workspace is None and self.workspace_bytes:
            workspace = torch.empty(self.workspace_bytes, dtype=torch.uint8, device=x0.device)
        self.workspace = workspace
        self._fn = L.lib().pgb_fused_reduce
        self.plan = describe_reduce([desc(t) for t in inputs], self._od, op, axes, prologue)

    def __call__(self, stream: int | None = None) -> torch.Tensor:
        ws = self.workspace
        st = self._fn(self._ins, self._n_in, C.byref(self._od), self._op, self._ax, self._n_ax, self._pro, self._npro, self._none, 0,
                      self._epi, self._nepi, ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
                      _stream() if stream is None else stream)
        if st != L.OK:
            L.check(st)
        return self.out
