"""Build the reference's own CUDA extension, from its sources where they lie, into oracle/_ref/.

Test infrastructure only: the product never loads what this script builds.  The resulting
module is the bit-exact GPU oracle used by tests/golden/make_golden_gpu.py to produce the
committed golden vectors.  The reference sources are compiled in place (nothing is copied
into this repository) with the reference's own flags, `-O3 --use_fast_math`
(src/coresets/cuda/extension.py:60-67), for compute capability 10.0.

Usage:  python oracle/build_ref.py [--reference /path/to/reference]
"""
from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"

KERNEL_FILES = ("warp.cu", "argmax.cu", "commit.cu", "simulate.cu", "multi.cu", "bindings.cu")


def build(reference_root: str) -> Path:
    kernels_dir = Path(reference_root) / "src" / "coresets" / "cuda" / "kernels"
    sources = [str(kernels_dir / n) for n in KERNEL_FILES]
    missing = [s for s in sources if not os.path.isfile(s)]
    if missing:
        raise FileNotFoundError(f"reference kernel sources missing: {missing}")

    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MAX_JOBS", "6")
    build_dir = OUT / "build"
    build_dir.mkdir(parents=True, exist_ok=True)

    from torch.utils.cpp_extension import load

    try:
        load(
            name="coreset_kernels",
            sources=sources,
            extra_cuda_cflags=["-O3", "--use_fast_math"],
            extra_cflags=["-O3"],
            extra_include_paths=[str(kernels_dir)],
            build_directory=str(build_dir),
            verbose=True,
        )
    except ImportError as e:  # built but not importable on a GPU-less host: fine
        print(f"note: built, import skipped: {e}")
    so = build_dir / "coreset_kernels.so"
    if not so.is_file():
        raise RuntimeError(f"build did not produce {so}")
    return so


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("CORESETS_REFERENCE_ROOT"),
                    required=not os.environ.get("CORESETS_REFERENCE_ROOT"), help="the reference checkout (or set CORESETS_REFERENCE_ROOT)")
    a = ap.parse_args()
    print(build(a.reference))
