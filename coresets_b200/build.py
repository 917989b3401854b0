"""Build the C-ABI shared library ``libcoresets_b200.so`` next to this file with nvcc.

    python -m coresets_b200.build [--force] [--verbose]

sm_100a only.  ``-ftz=true`` because the reference kernels are built with ``--use_fast_math``
(flush-to-zero is part of the bit-level contract); ``-fmad=false`` because every fused
multiply-add on the arithmetic path is written out explicitly in the source.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
LIB = Path(os.environ["CORESETS_B200_LIB"]) if os.environ.get("CORESETS_B200_LIB") else PKG / "libcoresets_b200.so"
SOURCES = [PKG / "csrc" / "fps_kernels.cu"]          # one translation unit; the kernels live in csrc/*.cuh
HEADERS = [ROOT / "include" / "coresets_b200.h", *sorted((PKG / "csrc").glob("*.cuh"))]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-ftz=true", "-fmad=false", "-prec-div=true", "-prec-sqrt=true",
    "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-cudart", "static",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isfile(cand):
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def needs_build() -> bool:
    if not LIB.is_file():
        return True
    t = LIB.stat().st_mtime
    return any(p.stat().st_mtime > t for p in SOURCES + HEADERS + [Path(__file__)])


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(ROOT / "include"), *os.environ.get("CORESETS_B200_NVCC_DEFS", "").split()]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(LIB), *map(str, SOURCES)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed ({res.returncode}): {' '.join(cmd)}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
