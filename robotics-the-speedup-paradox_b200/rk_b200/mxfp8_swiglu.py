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


_TABLES = {}


def cutlass_swiglu_mxfp8_packed(packed_input, input_scale, packed_interleaved_weight, weight_scale, silu_table=None):
    """MXFP8 gate/up GEMM + SwiGLU + MXFP8 output in one kernel (`rk_gemm_mxfp8_swiglu`); the call shape of the
    reference's ``cute_mxfp8_swiglu.cutlass_swiglu_mxfp8_packed``.  The weight rows are interleaved in blocks of
    64 (64 up rows, then their 64 gate rows: `rk_b200.fp4_linear.interleave_gate_up_rows` before packing).
    Returns (e4m3 [M, N / 2], swizzled UE8M0 scale bytes) - exactly `mxfp8_linear` followed by `silu_mul_pack_mxfp8`."""
    if packed_input.dtype != torch.float8_e4m3fn or packed_interleaved_weight.dtype != torch.float8_e4m3fn:
        raise TypeError("MXFP8 operands must use torch.float8_e4m3fn")
    if input_scale.dtype != torch.uint8 or weight_scale.dtype != torch.uint8:
        raise TypeError("MXFP8 scale factors must be uint8 E8M0 payloads")
    tensors = (packed_input, input_scale, packed_interleaved_weight, weight_scale)
    if not all(t.is_cuda and t.is_contiguous() for t in tensors) or len({t.device for t in tensors}) != 1:
        raise ValueError("MXFP8 operands must be contiguous CUDA tensors on one device")
    if packed_input.ndim != 2 or packed_interleaved_weight.ndim != 2:
        raise ValueError("MXFP8 operands must be rank two")
    m, k = packed_input.shape
    n = packed_interleaved_weight.shape[0]
    if packed_interleaved_weight.shape[1] != k or n % 256 or k % 32:
        raise ValueError(f"invalid MXFP8 Gate-Up shape M={m}, N={n}, K={k}")
    device = packed_input.device
    if silu_table is None:
        key = device.index if device.index is not None else torch.cuda.current_device()
        if key not in _TABLES:
            _TABLES[key] = make_bf16_silu_table(device)
        silu_table = _TABLES[key]
    lib = _lib.load()
    packed = torch.empty((m, n // 2), dtype=torch.float8_e4m3fn, device=device)
    scales = torch.empty(lib.rk_sf_bytes(m, n // 2 // 32), dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        ws = _lib.gemm_workspace(_lib.OP_MXFP8, device, m, n, k)
        code = lib.rk_gemm_mxfp8_swiglu(_lib.ptr(packed_input), _lib.ptr(input_scale), _lib.ptr(packed_interleaved_weight),
                                        _lib.ptr(weight_scale), _lib.ptr(silu_table), _lib.ptr(packed), _lib.ptr(scales), m, n, k,
                                        0, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(device))
    _lib.check(code, "cutlass_swiglu_mxfp8_packed")
    return packed, scales
