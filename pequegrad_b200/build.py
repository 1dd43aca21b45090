"""Builds the in-tree native libraries with nvcc / gcc.

`libpgb200.so` holds every CUDA kernel and the C ABI declared in
`include/pgb200.h`; it is compiled for sm_100a only. Object files are cached
under `pequegrad_b200/lib/obj` and rebuilt when a source or header is newer.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
OBJDIR = LIBDIR / "obj"
LIB = LIBDIR / "libpgb200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
    "-I", str(ROOT / "include"),
]
# + - * / must round as the reference's separate kernels do: no contraction
EXACT_FLAGS = ["-fmad=false"]
# files whose arithmetic is not compared bit-for-bit (tensor-core GEMMs)
FMAD_OK = {"gemm_kind_i8.cu", "gemm_kind_f16.cu", "gemm_kind_bf16.cu", "gemm_kind_tf32.cu"}


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")


def _newest_header() -> float:
    hs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.hpp")) + list((ROOT / "include").glob("*.h"))
    return max(h.stat().st_mtime for h in hs)


def _compile(src: Path, verbose: bool) -> Path:
    obj = OBJDIR / (src.stem + ".o")
    cmd = [_nvcc(), *NVCC_FLAGS]
    if src.name not in FMAD_OK:
        cmd += EXACT_FLAGS
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        (OBJDIR / (src.stem + ".ptxas.txt")).write_text(r.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu under csrc/ and link libpgb200.so. Returns its path."""
    OBJDIR.mkdir(parents=True, exist_ok=True)
    srcs = sorted(CSRC.glob("*.cu"))
    hdr = _newest_header()
    todo = []
    for s in srcs:
        o = OBJDIR / (s.stem + ".o")
        if force or not o.exists() or o.stat().st_mtime < max(s.stat().st_mtime, hdr):
            todo.append(s)
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            list(ex.map(lambda s: _compile(s, verbose), todo))
    objs = [OBJDIR / (s.stem + ".o") for s in srcs]
    if todo or not LIB.exists():
        cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC", "-lnvrtc" if False else "-lcudart_static", "-lpthread", "-ldl", "-lrt"]
        cmd = [c for c in cmd if c]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(p)
