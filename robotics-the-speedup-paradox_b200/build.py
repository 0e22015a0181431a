#!/usr/bin/env python3
"""Build the B200 quantized-linear kernel library (``librk_b200.so``) with nvcc.

Counterpart of the reference's ``tools/build_blackwell.py`` (one ``.so`` per Blackwell
backend built through torch's extension loader against CUTLASS): here every backend
(``integer``, ``w4a16``, ``fp8``, ``mxfp8``, ``fp4``) lives in ONE shared library with a flat
C ABI (``include/rk_b200.h``), built straight from ``csrc/*.cu`` for ``sm_100a`` with no
CUTLASS include path and no torch headers.  ``--backend`` is accepted for command-line
compatibility and only checked for validity.

The library is written next to the Python wrappers (``rk_b200/librk_b200.so``) so that an
in-tree checkout is self-contained.
"""

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
INCLUDE = ROOT.parent / "include"
DEFAULT_OUTPUT = ROOT / "rk_b200" / "librk_b200.so"
BACKENDS = ("all", "integer", "w4a16", "fp8", "mxfp8", "fp4")
SOURCES = ("rk_api.cu", "rk_quant.cu", "rk_rope.cu", "rk_gemm.cu")


def _arch_flags(arch):
    # "10.0a" -> compute_100a / sm_100a
    digits = arch.replace(".", "")
    return ["-gencode", f"arch=compute_{digits},code=sm_{digits}"]


def _nvcc():
    candidate = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(candidate).exists():
        raise RuntimeError("nvcc not found; the kernels cannot be built")
    return candidate


def _digest(paths, flags):
    h = hashlib.sha256(" ".join(flags).encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def build(arch="10.0a", build_dir=None, output=DEFAULT_OUTPUT, verbose=False, force=False):
    """Compile every translation unit and link the shared library.  Returns the library path."""
    nvcc = _nvcc()
    build_dir = Path(build_dir) if build_dir else ROOT / "build"
    build_dir.mkdir(parents=True, exist_ok=True)
    output = Path(output)
    sources = [CSRC / s for s in SOURCES if (CSRC / s).exists()]
    deps = sorted(CSRC.glob("*.cu*")) + sorted(CSRC.glob("*.h")) + sorted(INCLUDE.glob("*.h"))
    flags = _arch_flags(arch) + ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]
    stamp = build_dir / "librk_b200.sha256"
    digest = _digest(deps, flags)
    if not force and output.exists() and stamp.exists() and stamp.read_text() == digest:
        return output

    def compile_one(src):
        obj = build_dir / (src.stem + ".o")
        cmd = [nvcc, *flags, "-c", str(src), "-o", str(obj)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        (build_dir / (src.stem + ".log")).write_text(proc.stdout + proc.stderr)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stderr[-4000:]}")
        if verbose:
            print(proc.stderr, file=sys.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=int(os.environ.get("MAX_JOBS", "4"))) as pool:
        objects = list(pool.map(compile_one, sources))
    output.parent.mkdir(parents=True, exist_ok=True)
    link = [nvcc, "-shared", *_arch_flags(arch), "-o", str(output), *map(str, objects)]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed:\n{proc.stderr[-4000:]}")
    stamp.write_text(digest)
    return output


def main():
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--backend", choices=BACKENDS, default="all")
    parser.add_argument("--arch", default="10.0a", help="CUDA target; only 10.0a is supported")
    parser.add_argument("--build-dir", type=Path)
    parser.add_argument("--output", type=Path, default=DEFAULT_OUTPUT)
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    args = parser.parse_args()
    if args.arch != "10.0a":
        parser.error("these kernels use tcgen05 / TMEM and build for 10.0a only")
    print(build(args.arch, args.build_dir, args.output, args.verbose, args.force))


if __name__ == "__main__":
    main()
