"""Fused SwiGLU producer for MXFP8 activations: SiLU by table lookup, times up, block-32 pack.

Mirror of the reference's ``src/robotics_kernels/blackwell/mxfp8_swiglu.py`` (``make_bf16_silu_table``,
``silu_mul_pack_mxfp8``, ``load_mxfp8_swiglu_extension``); the operator
``robotics_mxfp8_swiglu::silu_mul_pack`` (blackwell/csrc/mxfp8_swiglu.cu:20-117) is `rk_swiglu_pack_mxfp8`.
"""

import torch

from . import _lib


def load_mxfp8_swiglu_extension(path=None):
    """The operator lives in the one kernel library; True once that library loads."""
    _lib.load()
    return True


def make_bf16_silu_table(device="cuda"):
    """SiLU evaluated on all 65536 bf16 bit patterns (reference: mxfp8_swiglu.py:37-40)."""
    raw = torch.arange(65536, device=device, dtype=torch.int32).to(torch.uint16)
    return torch.nn.functional.silu(raw.view(torch.bfloat16)).contiguous()


def silu_mul_pack_mxfp8(gate_up, intermediate_size, silu_table):
    """gate_up bf16 [..., 2 * inter] (gate first) -> (e4m3 [..., inter], swizzled UE8M0 scale bytes):
    bf16(table[gate] * up) packed in 32-element blocks."""
    inter = int(intermediate_size)
    if not gate_up.is_cuda or gate_up.dtype != torch.bfloat16 or not gate_up.is_contiguous() or gate_up.dim() < 2:
        raise ValueError("gate_up must be contiguous CUDA BF16")
    if inter <= 0 or inter % 32 or gate_up.shape[-1] != 2 * inter:
        raise ValueError("gate_up last dimension must be twice a K32-aligned intermediate size")
    if (not silu_table.is_cuda or silu_table.device != gate_up.device or silu_table.dtype != torch.bfloat16
            or not silu_table.is_contiguous() or silu_table.numel() != 65536):
        raise ValueError("silu_table must be contiguous CUDA BF16 with 65536 entries")
    rows = gate_up.numel() // gate_up.shape[-1]
    lib = _lib.load()
    packed = torch.empty((*gate_up.shape[:-1], inter), dtype=torch.float8_e4m3fn, device=gate_up.device)
    scales = torch.empty(lib.rk_sf_bytes(rows, inter // 32), dtype=torch.uint8, device=gate_up.device)
    with torch.cuda.device(gate_up.device):
        code = lib.rk_swiglu_pack_mxfp8(_lib.ptr(gate_up), rows, inter, _lib.ptr(silu_table), _lib.ptr(packed), _lib.ptr(scales),
                                        _lib.stream_ptr(gate_up.device))
    _lib.check(code, "silu_mul_pack_mxfp8")
    return packed, scales
