#!/usr/bin/env python3
"""Recipe for the reference's own Blackwell extensions (quantizers, packers and CUTLASS GEMMs).

TEST / BASELINE INFRASTRUCTURE ONLY.  Each extension is one `.cu` file of the reference
(`src/robotics_kernels/blackwell/csrc/`) that registers `torch.ops.<namespace>.*`.  This recipe
compiles the file WHERE IT LIES in a checkout of the reference with plain `nvcc` (the flags of the
reference's `tools/build_blackwell.py`: `-O3 -std=c++17 --use_fast_math --expt-relaxed-constexpr
-lineinfo`, target 10.0a) against torch's headers and the CUTLASS tree vendored in the reference,
and writes `oracle/_ref/libref_<backend>.so`.  Nothing from the reference is copied into this
tree; the output directory is ignored by git.  nvcc cross-compiles without a GPU; the libraries
are loaded with `torch.ops.load_library` on a machine that has a B200.

Their large-tile GEMM specialisations use thread-block clusters with multicast copies, so the
libraries are kept out of multi-GPU runs and are only ever loaded by single-GPU processes
(`oracle/ref_kernels.py`).

Usage: python oracle/build_ref_kernels.py [backend ...]     (default: all of BACKENDS)
"""

import os
import shutil
import subprocess
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"

# backend -> (source file, torch.ops namespace)
BACKENDS = {
    "mxfp8": ("mxfp8_cutlass_linear.cu", "robotics_mxfp8"),
    "fp8": ("fp8_cutlass_linear.cu", "robotics_cutlass_fp8"),
    "fp4": ("fp4_cutlass_linear.cu", "robotics_cutlass_fp4"),
    "fp4_mixed": ("fp4_mixed_cutlass_linear.cu", "robotics_cutlass_fp4_mixed"),
    "fp4_mx": ("fp4_mx_cutlass_linear.cu", "robotics_cutlass_fp4_mx"),
    "mxfp8_swiglu": ("mxfp8_swiglu.cu", "robotics_mxfp8_swiglu"),
}


# Extra nvcc flags per backend.  fp4_mx_cutlass_linear.cu calls __nv_cvt_float2_to_fp4x2 without
# including <cuda_fp4.h> (it does not compile as it stands); the header is force-included, the source
# stays untouched.
EXTRA_FLAGS = {"fp4_mx": ["-include", "cuda_fp4.h"]}


def reference_root():
    candidates = []
    if os.environ.get("RK_REFERENCE_ROOT"):
        candidates.append(Path(os.environ["RK_REFERENCE_ROOT"]))
    candidates.append(HERE.parent.parent / "reference")
    for c in candidates:
        if (c / "src" / "robotics_kernels" / "blackwell" / "csrc" / "mxfp8_common.cuh").exists():
            return c
    return None


def library_path(backend):
    return OUT_DIR / f"libref_{backend}.so"


def build_one(backend, verbose=False, force=False):
    """Returns (path or None, log text).  None when the checkout is absent or the compile failed."""
    root = reference_root()
    out = library_path(backend)
    if root is None:
        return (out if out.exists() else None), "no reference checkout"
    source, _ = BACKENDS[backend]
    src = root / "src" / "robotics_kernels" / "blackwell" / "csrc" / source
    if out.exists() and not force and out.stat().st_mtime >= src.stat().st_mtime:
        return out, "up to date"
    import torch  # noqa: F401  (headers and libraries come from the installed wheel)
    from torch.utils import cpp_extension as ext

    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cutlass = root / "src" / "robotics_kernels" / "ampere_ada" / "third_party" / "cutlass"
    OUT_DIR.mkdir(exist_ok=True)
    cmd = [nvcc, "-O3", "-std=c++17", "--use_fast_math", "--expt-relaxed-constexpr", "-lineinfo",
           "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC", "-w",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1",
           "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
           "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__"]
    for inc in [cutlass / "include", cutlass / "tools" / "util" / "include", *ext.include_paths("cuda")]:
        cmd += ["-isystem" if "torch" in str(inc) else "-I", str(inc)]
    for lib in ext.library_paths("cuda"):
        cmd += ["-L", str(lib)]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-lcuda"]
    cmd += EXTRA_FLAGS.get(backend, [])
    cmd += [str(src), "-o", str(out)]
    if verbose:
        print(" ".join(cmd), flush=True)
    t0 = time.time()
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log = f"[{backend}] nvcc rc={proc.returncode} in {time.time() - t0:.0f} s\n" + proc.stdout[-4000:] + proc.stderr[-8000:]
    (OUT_DIR / f"libref_{backend}.log").write_text(log)
    if proc.returncode != 0:
        if out.exists():
            out.unlink()
        return None, log
    return out, log


def build(backends=None, verbose=False, force=False, jobs=None):
    """Builds (or finds up to date) the requested extensions, several compilers at a time: each of
    these translation units takes minutes."""
    from concurrent.futures import ThreadPoolExecutor

    names = list(backends or BACKENDS)
    jobs = jobs or int(os.environ.get("MAX_JOBS", "3"))
    with ThreadPoolExecutor(max_workers=max(1, jobs)) as pool:
        outcomes = list(pool.map(lambda b: build_one(b, verbose, force), names))
    results = {}
    for b, (path, log) in zip(names, outcomes):
        results[b] = path
        if verbose or path is None:
            print(log, flush=True)
    return results


if __name__ == "__main__":
    names = [a for a in sys.argv[1:] if not a.startswith("-")]
    print(build(names or None, verbose=True, force="--force" in sys.argv))
