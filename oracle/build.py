"""TEST INFRASTRUCTURE — builds the CPU oracle libraries.

  oracle/libpgoracle.so      the C restatement (pgoracle.c), always built
  oracle/_ref/libpgref.so    the reference's own CPU templates behind the same
                             C entry points (ref_shim.cpp), built only where a
                             reference checkout is present; the prebuilt file
                             travels with the repository snapshot otherwise.

No reference source is copied: the compiler is pointed at the checkout.
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


def reference_root() -> Path | None:
    cand = Path(os.environ.get("PGB_REFERENCE", "/root/reference"))
    return cand if (cand / "csrc" / "cpu" / "reduce.hpp").exists() else None


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("oracle build failed: " + " ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)


def build(force: bool = False) -> dict:
    out = {}
    src = HERE / "pgoracle.c"
    if force or not PORT.exists() or PORT.stat().st_mtime < src.stat().st_mtime:
        _run(["gcc", "-O2", "-std=gnu11", "-fopenmp", "-ffp-contract=off", "-fPIC", "-shared", "-fvisibility=hidden",
              str(src), "-o", str(PORT), "-lm"])
    out["port"] = PORT
    root = reference_root()
    shim = HERE / "ref_shim.cpp"
    if root is not None and (force or not REF.exists() or REF.stat().st_mtime < shim.stat().st_mtime):
        REF_DIR.mkdir(exist_ok=True)
        # -fpermissive: the reference headers use MSVC-only constructs; no -mavx*: its AVX
        # path needs SVML intrinsics gcc lacks (csrc/cpu/unary.hpp:55-62)
        _run(["g++", "-O2", "-std=c++17", "-fopenmp", "-ffp-contract=off", "-fPIC", "-shared", "-fpermissive", "-w",
              "-fvisibility=hidden", "-I", str(HERE / "shim"), "-I", str(root / "csrc"), "-I", "/usr/local/cuda/include",
              str(shim), "-o", str(REF)])
    out["ref"] = REF if REF.exists() else None
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
