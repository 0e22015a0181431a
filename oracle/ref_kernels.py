"""Loader for the reference's own Blackwell extensions, compiled by `oracle/build_ref_kernels.py`.

TEST / BASELINE INFRASTRUCTURE ONLY: the package never imports this module.  It is used to pin
the oracle (and through it the CUDA kernels) to what the reference's quantizers, packers and
CUTLASS GEMMs produce on a B200, and to time those GEMMs beside this library's on the same GPU.

The libraries register `torch.ops.robotics_mxfp8.*`, `torch.ops.robotics_cutlass_fp8.*`,
`torch.ops.robotics_cutlass_fp4.*`, ... exactly as the reference's own loader would
(src/robotics_kernels/blackwell/extension_loader.py:19-64).  Their large-tile GEMMs use cluster
multicast copies, so they are only loaded by single-GPU processes.
"""

import os
from pathlib import Path

REF_DIR = Path(__file__).resolve().parent / "_ref"
NAMESPACES = {
    "mxfp8": "robotics_mxfp8",
    "fp8": "robotics_cutlass_fp8",
    "fp4": "robotics_cutlass_fp4",
    "fp4_mixed": "robotics_cutlass_fp4_mixed",
    "fp4_mx": "robotics_cutlass_fp4_mx",
    "mxfp8_swiglu": "robotics_mxfp8_swiglu",
}
_loaded = {}


def library_path(backend):
    return REF_DIR / f"libref_{backend}.so"


def load(backend):
    """-> (torch.ops namespace, None) or (None, reason)."""
    if backend in _loaded:
        return _loaded[backend]
    import torch

    result = None
    path = library_path(backend)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        result = (None, "reference extensions are single-GPU only (cluster multicast copies)")
    elif not path.exists():
        result = (None, f"{path.name} was not built (oracle/build_ref_kernels.py)")
    elif not torch.cuda.is_available():
        result = (None, "no CUDA device")
    else:
        try:
            torch.ops.load_library(str(path))
            result = (getattr(torch.ops, NAMESPACES[backend]), None)
        except (OSError, RuntimeError) as error:
            result = (None, f"{path.name} failed to load: {error}")
    _loaded[backend] = result
    return result


def available(backend):
    return load(backend)[0] is not None
