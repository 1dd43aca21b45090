"""ctypes binding of `libpgb200.so` (the C ABI in `include/pgb200.h`).

There is no fallback: if the library is missing, or a call fails, an exception
is raised. Errors map the way the reference's pybind layer maps them
(csrc/utils.hpp:10-25): invalid arguments -> ValueError, everything else ->
RuntimeError.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

MAX_DIMS = 8
MAX_INPUTS = 6
MAX_INSTRS = 32

# pgb_dtype
I32, F16, F32, F64, I8, BF16 = 0, 1, 2, 3, 4, 5
# pgb_status
OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT, ERR_WORKSPACE = 0, -1, -2, -3, -4, -5
# pgb_reduce_op
SUM, MAX, MEAN, ARGMAX = 0, 1, 2, 3

OPS = dict(
    LOAD=0, IMM=1, ACC=2,
    LOG=8, EXP=9, SIN=10, COS=11, CAST_F16=12, CAST_F32=13, CAST_I32=14, CAST_BF16=15,
    ADD=16, MUL=17, MAX=18, SUB=19, DIV=20, GT=21, LT=22, MOD=23, EQ=24, POW=25, LTE=26, NEQ=27, GTE=28,
    WHERE=32,
)


class PgbTensor(C.Structure):
    _fields_ = [
        ("data", C.c_void_p),
        ("dtype", C.c_int32),
        ("ndim", C.c_int32),
        ("shape", C.c_int64 * MAX_DIMS),
        ("stride_bytes", C.c_int64 * MAX_DIMS),
    ]


class PgbInstr(C.Structure):
    _fields_ = [
        ("op", C.c_uint8),
        ("reserved", C.c_uint8),
        ("a", C.c_int16),
        ("b", C.c_int16),
        ("c", C.c_int16),
        ("imm", C.c_double),
    ]


LIB_PATH = Path(__file__).resolve().parent / "lib" / "libpgb200.so"

# every symbol include/pgb200.h declares
EXPORTS = [
    "pgb_status_string", "pgb_last_error", "pgb_version", "pgb_launch_count",
    "pgb_fused_elementwise", "pgb_fused_reduce", "pgb_fused_reduce_workspace", "pgb_fused_reduce_describe",
    "pgb_softmax_rows", "pgb_layernorm_rows", "pgb_fused_reduce_noalloc",
    "pgb_embedding_rows", "pgb_matmul", "pgb_attention", "pgb_qlinear_i8", "pgb_absmax_f32", "pgb_quantize_i8", "pgb_device_error",
    "pgb_gemm_pair_mode", "pgb_gemm_wait_drill",
    "pgb_peer_ctrl_bytes", "pgb_peer_poll_limit", "pgb_peer_alloc", "pgb_peer_free", "pgb_peer_export", "pgb_peer_open", "pgb_peer_close",
    "pgb_peer_allreduce_max_f32", "pgb_peer_allgather",
]
NOALLOC_SCRATCH_BYTES = 4 << 20  # PGB_NOALLOC_SCRATCH_BYTES

_lib = None


def lib() -> C.CDLL:
    """Load the native library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m pequegrad_b200.build` "
            "(there is no CPU or PyTorch fallback for these kernels)"
        )
    L = C.CDLL(str(LIB_PATH))
    TP, IP = C.POINTER(PgbTensor), C.POINTER(PgbInstr)
    L.pgb_status_string.restype = C.c_char_p
    L.pgb_status_string.argtypes = [C.c_int]
    L.pgb_last_error.restype = C.c_char_p
    L.pgb_version.restype = C.c_char_p
    L.pgb_launch_count.restype = C.c_uint64
    L.pgb_fused_elementwise.argtypes = [TP, C.c_int, TP, C.c_int, IP, C.c_int, C.POINTER(C.c_int16), C.c_void_p]
    L.pgb_fused_reduce.argtypes = [TP, C.c_int, TP, C.c_int, C.POINTER(C.c_int32), C.c_int, IP, C.c_int, TP, C.c_int, IP, C.c_int,
                                   C.c_void_p, C.c_size_t, C.c_void_p]
    L.pgb_fused_reduce_workspace.argtypes = [TP, C.c_int, TP, C.c_int, C.POINTER(C.c_int32), C.c_int, C.POINTER(C.c_size_t)]
    L.pgb_fused_reduce_describe.argtypes = [TP, C.c_int, TP, C.c_int, C.POINTER(C.c_int32), C.c_int, IP, C.c_int, C.c_char_p, C.c_size_t]
    L.pgb_fused_reduce_noalloc.argtypes = [TP, C.c_int, TP, C.c_int, C.POINTER(C.c_int32), C.c_int, IP, C.c_int, TP, C.c_int, IP, C.c_int,
                                           C.c_void_p]
    L.pgb_embedding_rows.argtypes = [TP, TP, TP, C.c_int64, TP, C.c_void_p]
    L.pgb_matmul.argtypes = [TP, TP, TP, C.c_int, C.c_float, TP, TP, C.c_void_p]
    L.pgb_attention.argtypes = [TP, TP, TP, C.c_float, C.c_int, TP, C.c_void_p]
    L.pgb_qlinear_i8.argtypes = [TP, TP, C.c_void_p, C.c_float, C.c_void_p, TP, C.c_int, TP, TP, C.c_void_p, C.c_void_p]
    L.pgb_absmax_f32.argtypes = [TP, C.c_void_p, C.c_void_p]
    L.pgb_quantize_i8.argtypes = [TP, C.c_void_p, C.c_float, TP, C.c_void_p]
    L.pgb_device_error.argtypes = [C.POINTER(C.c_int), C.c_int]
    L.pgb_gemm_pair_mode.argtypes = [C.c_int]
    L.pgb_gemm_wait_drill.argtypes = [C.c_uint, C.c_int]
    L.pgb_peer_ctrl_bytes.restype = C.c_size_t
    L.pgb_peer_poll_limit.restype = C.c_uint
    L.pgb_peer_poll_limit.argtypes = [C.c_uint]
    L.pgb_peer_alloc.argtypes = [C.c_size_t, C.POINTER(C.c_void_p)]
    L.pgb_peer_free.argtypes = [C.c_void_p]
    L.pgb_peer_export.argtypes = [C.c_void_p, C.c_char_p]
    L.pgb_peer_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    L.pgb_peer_close.argtypes = [C.c_void_p]
    L.pgb_peer_allreduce_max_f32.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_void_p]
    L.pgb_peer_allgather.argtypes = [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_void_p]
    L.pgb_softmax_rows.argtypes = [TP, TP, C.c_int, C.c_void_p]
    L.pgb_layernorm_rows.argtypes = [TP, TP, TP, C.c_float, TP, C.c_void_p]
    for name in EXPORTS:
        getattr(L, name)
    _lib = L
    return L


def check(status: int) -> None:
    if status == OK:
        return
    L = lib()
    msg = L.pgb_last_error().decode() or L.pgb_status_string(status).decode()
    if status == ERR_INVALID_ARG:
        raise ValueError(msg)
    raise RuntimeError(msg)


def make_tensor(ptr: int, dtype: int, shape, stride_bytes) -> PgbTensor:
    t = PgbTensor()
    t.data = ptr
    t.dtype = dtype
    t.ndim = len(shape)
    if len(shape) > MAX_DIMS:
        raise ValueError("at most 8 dims are supported")
    for i, (s, st) in enumerate(zip(shape, stride_bytes)):
        t.shape[i] = int(s)
        t.stride_bytes[i] = int(st)
    return t


def make_program(instrs) -> tuple:
    """instrs: list of (opname, a, b, c, imm) tuples (trailing fields optional)."""
    n = len(instrs)
    arr = (PgbInstr * max(n, 1))()
    for i, ins in enumerate(instrs):
        ins = tuple(ins) + (0,) * (5 - len(ins))
        arr[i].op = OPS[ins[0]] if isinstance(ins[0], str) else int(ins[0])
        arr[i].a, arr[i].b, arr[i].c = int(ins[1]), int(ins[2]), int(ins[3])
        arr[i].imm = float(ins[4])
    return arr, n
