"""ctypes binding of ``librk_b200.so`` (the C ABI declared in ``include/rk_b200.h``).

The library is the only compute path: if it is missing or a call fails, the wrappers raise.
There is no PyTorch or CPU fallback behind these calls.
"""

import ctypes
import os
import threading
from pathlib import Path

import torch

RK_OK = 0
RK_EINVAL = -1
RK_EUNSUPPORTED = -2
RK_ECUDA = -3
RK_EWORKSPACE = -4
RK_EDEVICE = -5

ACT_PLAIN, ACT_LUT_MUL, ACT_LUT = 0, 1, 2
OP_W8A8, OP_W4A4, OP_W4A16, OP_FP8, OP_MXFP8, OP_NVFP4 = range(6)
WORKSPACE_HEADER = 256

_vp, _i64, _int, _sz, _f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t, ctypes.c_float

# name -> (restype, argtypes); mirrors include/rk_b200.h one to one
SIGNATURES = {
    "rk_version": (_int, []),
    "rk_last_error_string": (ctypes.c_char_p, []),
    "rk_supports_device": (_int, [_int, _int]),
    "rk_workspace_bytes": (_sz, [_int, _i64, _i64, _i64]),
    "rk_sf_bytes": (_sz, [_i64, _i64]),
    "rk_read_status": (_int, [_vp, ctypes.POINTER(_int), _vp]),
    "rk_debug_wait_expiry": (_int, [_int, _int]),
    "rk_probe_rcp_approx_448": (_int, [ctypes.POINTER(ctypes.c_uint32)]),
    "rk_quant_rows": (_int, [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _int, _int, _vp, _vp, _vp]),
    "rk_quant_weight_int": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp]),
    "rk_quant_rows_modulated": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _int, _f32, _vp, _vp, _vp, _int, _vp, _vp, _vp]),
    "rk_rmsnorm_quant_rows": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _f32, _int, _vp, _vp, _vp, _vp, _vp]),
    "rk_rmsnorm_tensor_scale": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _f32, _f32, _vp, _vp, _vp, _vp, _sz, _vp]),
    "rk_lut_mul_tensor_scale": (_int, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _f32, _vp, _vp, _vp, _sz, _vp]),
    "rk_gated_rmsnorm_quant_rows": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _f32, _int, _vp, _vp, _vp, _vp, _vp]),
    "rk_gemm_int": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp, _sz, _vp]),
    "rk_gemm_int_residual": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _i64, _int, _int, _vp, _sz, _vp]),
    "rk_gemm_int_acc": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp, _sz, _vp]),
    "rk_gemm_int4_noalloc": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "rk_pack_w4_g128": (_int, [_vp, _i64, _i64, _vp, _vp, _vp]),
    "rk_gemm_w4a16_g128": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _sz, _vp]),
    "rk_quant_tensor_fp8": (_int, [_vp, _i64, _vp, _vp, _vp, _sz, _vp]),
    "rk_quant_tensor_fp8_with_scale": (_int, [_vp, _i64, _vp, _vp, _vp]),
    "rk_rmsnorm_quant_fp8": (_int, [_vp, _vp, _vp, _i64, _i64, _f32, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "rk_swiglu_quant_fp8": (_int, [_vp, _i64, _i64, _vp, _vp, _vp, _vp, _sz, _vp]),
    "rk_gemm_fp8": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _sz, _vp]),
    "rk_gemm_fp8_producer": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _sz, _vp]),
    "rk_gemm_fp8_column_parallel": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _i64, _i64, _vp, _int, _int, _vp, _vp, _sz, _vp]),
    "rk_wait_peers": (_int, [_vp, _int, _vp, _vp, _sz, _vp]),
    "rk_peer_alloc": (_int, [_sz, ctypes.POINTER(ctypes.c_void_p), _vp]),
    "rk_peer_open": (_int, [_vp, _int, ctypes.POINTER(ctypes.c_void_p), ]),
    "rk_peer_close": (_int, [_vp]),
    "rk_peer_free": (_int, [_vp]),
    "rk_pack_mxfp8": (_int, [_vp, _i64, _i64, _vp, _vp, _vp]),
    "rk_rmsnorm_bf16": (_int, [_vp, _vp, _vp, _i64, _i64, _f32, _vp, _vp, _vp]),
    "rk_silu_mul_bf16": (_int, [_vp, _i64, _i64, _int, _vp, _vp]),
    "rk_swiglu_pack_mxfp8": (_int, [_vp, _i64, _i64, _vp, _vp, _vp, _vp]),
    "rk_swiglu_pack_nvfp4_layout": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp]),
    "rk_pack_mxfp4_weight": (_int, [_vp, _i64, _i64, _vp, _vp, _vp]),
    "rk_pack_mxfp8_act_w4a8": (_int, [_vp, _i64, _i64, _vp, _vp, _vp]),
    "rk_swiglu_pack_mxfp8_w4a8": (_int, [_vp, _i64, _i64, _int, _vp, _vp, _vp]),
    "rk_gemm_w4a8_mx": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _sz, _vp]),
    "rk_gemm_mxfp8": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _sz, _vp]),
    "rk_pack_nvfp4": (_int, [_vp, _i64, _i64, _vp, _vp, _vp, _vp]),
    "rk_rmsnorm_pack_nvfp4": (_int, [_vp, _vp, _vp, _i64, _i64, _f32, _vp, _vp, _vp, _vp, _vp]),
    "rk_swiglu_pack_nvfp4": (_int, [_vp, _i64, _i64, _vp, _vp, _vp]),
    "rk_nvfp4_global_scale": (_int, [_vp, _i64, _vp, _vp, _sz, _vp]),
    "rk_gemm_nvfp4": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _sz, _vp]),
    "rk_gemm_nvfp4_swiglu": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _sz, _vp]),
    "rk_gemm_mxfp8_swiglu": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _sz, _vp]),
    "rk_gemm_nvfp4_gated_act": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _f32, _vp, _vp, _i64, _i64, _i64, _int, _vp, _sz, _vp]),
    "rk_rope_cache_update": (_int, [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _int,
                                    _vp, _vp, _i64, _i64, _vp]),
    "rk_rope_cache_update_vt": (_int, [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp,
                                       _int, _vp, _vp, _i64, _i64, _vp, _i64, _vp]),
    "rk_attention_prefix": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _f32, _vp, _sz,
                                   _vp]),
}

_lock = threading.Lock()
_lib = None


def library_path():
    """Location of the shared library: ``RK_B200_SO`` if set, else next to this file."""
    override = os.environ.get("RK_B200_SO")
    return Path(override) if override else Path(__file__).resolve().parent / "librk_b200.so"


def load():
    """Load the library once and declare every signature.  Raises RuntimeError when it is missing."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = library_path()
        if not path.exists():
            raise RuntimeError(
                f"{path} does not exist: build it with robotics-the-speedup-paradox_b200/build.py "
                "(there is no fallback implementation)"
            )
        lib = ctypes.CDLL(str(path))
        missing = [name for name in SIGNATURES if not hasattr(lib, name)]
        if missing:
            raise RuntimeError(f"{path} lacks entry points {missing}")
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
        return lib


def backend_status():
    """(available, error) without raising, in the manner of the reference's extension loaders
    (src/robotics_kernels/blackwell/extension_loader.py:19-64)."""
    try:
        load()
    except (OSError, RuntimeError) as error:
        return False, str(error)
    return True, None


def last_error():
    return load().rk_last_error_string().decode()


def check(code, what):
    """Translate a return code into the exception type the reference surface raises."""
    if code == RK_OK:
        return
    message = f"{what}: {last_error()} (code {code})"
    if code == RK_EINVAL:
        raise ValueError(message)
    raise RuntimeError(message)


def ptr(tensor):
    return None if tensor is None else ctypes.c_void_p(tensor.data_ptr())


def stream_ptr(device=None):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


# ---- per (device, stream) scratch buffers ---------------------------------------------------
_workspaces = {}


def workspace(device, nbytes):
    """Zero-initialised scratch tensor for the current stream of `device`, at least `nbytes` long.

    Kernels keep the buffer zero-filled between calls, so it is cleared only when (re)allocated.
    Growing allocates a larger buffer for later calls; the smaller ones are kept for the life of
    the process, because a CUDA graph captured earlier on this stream handle (torch reuses its
    pooled handles) may still write its scratch and its status word there on replay.
    """
    device = torch.device(device)
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    buffers = _workspaces.setdefault(key, [])
    if not buffers or buffers[-1].numel() < nbytes:
        size = max(int(nbytes), 1 << 20)
        buffers.append(torch.zeros(size, dtype=torch.uint8, device=device))
    return buffers[-1]


def gemm_workspace(op, device, m, n, k):
    need = load().rk_workspace_bytes(op, m, n, k)
    return workspace(device, need)


def read_status(buf, device=None):
    """Device status word of a workspace tensor; `buf=None` reads the scratch array built into the
    library (the one `rk_gemm_int4_noalloc` uses) on `device`."""
    code = ctypes.c_int(0)
    device = buf.device if buf is not None else torch.device(device if device is not None else "cuda")
    with torch.cuda.device(device):
        rc = load().rk_read_status(ptr(buf), ctypes.byref(code), stream_ptr(device))
    check(rc, "rk_read_status")
    return code.value
