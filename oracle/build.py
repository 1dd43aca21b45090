"""TEST INFRASTRUCTURE — builds the CPU oracle libraries.

  oracle/libpgoracle.so      the C restatement (pgoracle.c), always built
  oracle/_ref/libpgref.so    the reference's own CPU templates behind the same
                             C entry points (ref_shim.cpp), built only where a
                             reference checkout is present; the prebuilt file
                             travels with the repository snapshot otherwise.
  oracle/_ref_cuda/libpgrefcuda.so
                             the reference's own CUDA kernels (reduce, binary,
                             exp, where, and the generated kernel its README
                             prints) behind C entry points (ref_cuda_shim.cu),
                             cross-compiled by nvcc under the same condition.

No reference source is copied: the compilers are pointed at the checkout
(`build(reference=...)`, the PGB_REFERENCE variable, or a `reference`
directory beside this repository).
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
PORT = HERE / "libpgoracle.so"
REF_DIR = HERE / "_ref"
REF = REF_DIR / "libpgref.so"
REF_CUDA_DIR = HERE / "_ref_cuda"
REF_CUDA = REF_CUDA_DIR / "libpgrefcuda.so"


def reference_root(reference: str | os.PathLike | None = None) -> Path | None:
    cands = [reference, os.environ.get("PGB_REFERENCE"), HERE.parent.parent / "reference"]
    for cand in cands:
        if cand and (Path(cand) / "csrc" / "cpu" / "reduce.hpp").exists():
            return Path(cand)
    return None


def _readme_kernel(root: Path) -> str:
    """The generated CUDA kernel the reference's README prints for its fusion example, cut out of the README."""
    lines = (root / "README.md").read_text().splitlines()
    start = next(i for i, l in enumerate(lines) if l.startswith("__global__ void") and "reduce_kernel" in l)
    end = next(i for i in range(start, len(lines)) if lines[i].rstrip() == "}")
    return "\n".join(lines[start:end + 1]) + "\n"


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("oracle build failed: " + " ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)


def build(force: bool = False, reference: str | os.PathLike | None = None) -> dict:
    out = {}
    src = HERE / "pgoracle.c"
    if force or not PORT.exists() or PORT.stat().st_mtime < src.stat().st_mtime:
        _run(["gcc", "-O2", "-std=gnu11", "-fopenmp", "-ffp-contract=off", "-fPIC", "-shared", "-fvisibility=hidden",
              str(src), "-o", str(PORT), "-lm"])
    out["port"] = PORT
    root = reference_root(reference)
    shim = HERE / "ref_shim.cpp"
    if root is not None and (force or not REF.exists() or REF.stat().st_mtime < shim.stat().st_mtime):
        REF_DIR.mkdir(exist_ok=True)
        # -fpermissive: the reference headers use MSVC-only constructs; no -mavx*: its AVX
        # path needs SVML intrinsics gcc lacks (csrc/cpu/unary.hpp:55-62)
        _run(["g++", "-O2", "-std=c++17", "-fopenmp", "-ffp-contract=off", "-fPIC", "-shared", "-fpermissive", "-w",
              "-fvisibility=hidden", "-I", str(HERE / "shim"), "-I", str(root / "csrc"), "-I", "/usr/local/cuda/include",
              str(shim), "-o", str(REF)])
    out["ref"] = REF if REF.exists() else None
    cshim = HERE / "ref_cuda_shim.cu"
    if root is not None and (force or not REF_CUDA.exists() or REF_CUDA.stat().st_mtime < cshim.stat().st_mtime):
        REF_CUDA_DIR.mkdir(exist_ok=True)
        (REF_CUDA_DIR / "readme_kernel.inc").write_text(_readme_kernel(root))
        nvcc = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
        _run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fpermissive", "-Xcompiler", "-fvisibility=hidden", "-w", "-I", str(REF_CUDA_DIR), "-I", str(HERE / "shim"),
              "-I", str(root / "csrc"), str(cshim), "-o", str(REF_CUDA), "-lcudart_static", "-lpthread", "-ldl", "-lrt"])
    out["ref_cuda"] = REF_CUDA if REF_CUDA.exists() else None
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
