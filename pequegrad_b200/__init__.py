"""pequegrad_b200 — B200 (sm_100a) kernels for pequegrad's data-parallel hot path.

Only what that path needs lives here: the CUDA sources and C ABI (`csrc/`,
`include/pgb200.h`), the ctypes binding (`_lib`), torch-pointer wrappers
(`kernels`), and a host-side mirror of the reference's operator interface
(`tensor`, `fuser`, `distrib`): lazy tensors, `jit`, `shard_tensor` / `pmap`.
"""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
