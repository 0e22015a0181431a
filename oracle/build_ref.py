#!/usr/bin/env python3
"""Recipe for the oracle's compiled helper: the reference's own number-format conversions.

TEST INFRASTRUCTURE ONLY.  Compiles `oracle/ref_formats.cpp` against headers that stay where they
are in a checkout of the reference (its vendored CUTLASS and its `blackwell/csrc` directory) and
writes `oracle/_ref/libref_formats.so`.  Nothing from the reference is copied into this tree; the
output directory is ignored by git.  When no checkout of the reference is found the recipe does
nothing and leaves a previously built library in place.

The checkout is looked up in `$RK_REFERENCE_ROOT`, then in a directory named `reference` beside
this repository.
"""

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
OUT = OUT_DIR / "libref_formats.so"


def reference_root():
    candidates = []
    if os.environ.get("RK_REFERENCE_ROOT"):
        candidates.append(Path(os.environ["RK_REFERENCE_ROOT"]))
    candidates.append(HERE.parent.parent / "reference")
    for c in candidates:
        if (c / "src" / "robotics_kernels" / "blackwell" / "csrc" / "mxfp8_common.cuh").exists():
            return c
    return None


def build(verbose=False):
    """Returns the path of the built library, or None when the reference checkout is absent."""
    root = reference_root()
    if root is None:
        return OUT if OUT.exists() else None
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    kernels = root / "src" / "robotics_kernels"
    includes = [kernels / "ampere_ada" / "third_party" / "cutlass" / "include", kernels / "blackwell" / "csrc"]
    src = HERE / "ref_formats.cpp"
    if OUT.exists() and OUT.stat().st_mtime >= src.stat().st_mtime:
        return OUT
    OUT_DIR.mkdir(exist_ok=True)
    cmd = [nvcc, "-x", "cu", "-std=c++17", "-O2", "-shared", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
           "-gencode", "arch=compute_100a,code=sm_100a", "-w"]
    for inc in includes:
        cmd += ["-I", str(inc)]
    cmd += [str(src), "-o", str(OUT)]
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
