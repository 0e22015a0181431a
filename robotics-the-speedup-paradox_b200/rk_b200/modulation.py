"""BF16 AdaLN modulation (optionally LayerNorm and a gated residual first) packed straight into
symmetric integer activation buffers, and the Gemma RMSNorm analogue.

Host-side mirror of the reference's ``src/robotics_kernels/ampere_ada/modulation.py``
(``prepare_modulation``, ``prepare_norm_modulation``, ``prepare_residual_norm_modulation``,
``PackedActivations``); the arithmetic runs in ``librk_b200.so``.  ``prepare_rmsnorm`` is the
same fusion for the Gemma norms (models/pi05/modeling_gemma.py:62-106), which the reference
leaves unfused.
"""

from dataclasses import dataclass, replace
import math

import torch

from . import _lib
from .integer import PackedActivation

MAX_FUSED_K = 8192


def _check_eps(eps):
    if eps is None or not isinstance(eps, (int, float)) or not math.isfinite(eps) or eps <= 0:
        raise ValueError("LayerNorm epsilon must be finite and positive")
    return float(eps)


def prepare_modulation(x, scale, shift, bits):
    return _prepare(x, scale, shift, bits)


def prepare_norm_modulation(x, scale, shift, bits, *, eps):
    """Fuse non-affine LayerNorm into packing; FP32 reduction order may differ."""
    return _prepare(x, scale, shift, bits, eps=_check_eps(eps))


def prepare_residual_norm_modulation(x, y, gate, scale, shift, bits, *, eps):
    """Return the exact BF16 residual and its fused normalized integer pack."""
    return _prepare(x, scale, shift, bits, eps=_check_eps(eps), residual=(y, gate))


def _prepare(x, scale, shift, bits, *, eps=None, residual=None):
    if bits not in (4, 8) or x.ndim != 3 or not x.is_cuda or x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError("Modulation packing requires contiguous CUDA BF16 B,T,D and bits=4 or 8")
    b, tokens, k = x.shape
    if min(b, tokens, k) < 1 or k > 65536:
        raise ValueError("Unsupported modulation dimensions")
    for value in (scale, shift):
        if value.shape != (b, 1, k) or value.dtype != x.dtype or value.device != x.device:
            raise ValueError("Modulation scale and shift must match B,1,D, dtype and device")
    scale, shift = scale.contiguous(), shift.contiguous()
    y = gate = residual_out = None
    if residual is not None:
        y, gate = residual
        if (
            y.shape != x.shape or y.dtype != x.dtype or y.device != x.device or not y.is_contiguous()
            or gate.shape != (b, 1, k) or gate.dtype != x.dtype or gate.device != x.device
        ):
            raise ValueError("Residual operands must match BF16 input and B,1,D gate")
        gate = gate.contiguous()
        residual_out = torch.empty_like(x)
    if k > MAX_FUSED_K:
        raise RuntimeError(f"Fused modulation packing supports feature widths up to {MAX_FUSED_K}")
    rows, padded = b * tokens, (k + 127) // 128 * 128
    data = torch.empty(
        (rows, padded if bits == 8 else padded // 2), device=x.device,
        dtype=torch.int8 if bits == 8 else torch.uint8,
    )
    scales = torch.empty(rows, device=x.device, dtype=torch.float32)
    with torch.cuda.device(x.device):
        code = _lib.load().rk_quant_rows_modulated(
            _lib.ptr(x), _lib.ptr(scale), _lib.ptr(shift), rows, k, tokens, 0 if eps is None else 1,
            0.0 if eps is None else eps, _lib.ptr(y), _lib.ptr(gate), _lib.ptr(residual_out), bits,
            _lib.ptr(data), _lib.ptr(scales), _lib.stream_ptr(x.device),
        )
    _lib.check(code, "prepare_modulation")
    packed = PackedActivation(data, scales, (b, tokens), k, bits)
    return packed if residual is None else (residual_out, packed)


def prepare_rmsnorm(x, weight, bits, *, eps, residual=None, gate=None, shift=None, tokens=0, return_sum=False,
                    return_normed=False):
    """Gemma RMSNorm -> integer pack in one pass.

    ``weight`` is the learned ``[K]`` vector (plain norm, ``tokens=0``) or the adaptive scale
    ``[rows/tokens, K]`` with ``shift`` of the same shape.  ``residual`` (same shape as ``x``) is
    added first - multiplied by ``gate`` ``[rows/tokens, K]`` when one is given (the gated residual
    of the adaptive layers); ``return_sum`` / ``return_normed`` also return those BF16 tensors.
    """
    if bits not in (4, 8) or not x.is_cuda or x.dtype != torch.bfloat16 or not x.is_contiguous() or x.ndim < 2:
        raise ValueError("RMSNorm packing requires contiguous CUDA BF16 rows and bits=4 or 8")
    k = x.shape[-1]
    rows = x.numel() // k
    if k > MAX_FUSED_K:
        raise RuntimeError(f"Fused RMSNorm packing supports feature widths up to {MAX_FUSED_K}")
    eps = _check_eps(eps)
    weight = weight.contiguous()
    expect = k if tokens == 0 else (rows // max(tokens, 1)) * k
    if weight.dtype != x.dtype or weight.numel() != expect or (shift is not None and shift.numel() != expect):
        raise ValueError("RMSNorm scale / shift do not match the input")
    if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype or not residual.is_contiguous()):
        raise ValueError("Residual must match the BF16 input")
    padded = (k + 127) // 128 * 128
    data = torch.empty((rows, padded if bits == 8 else padded // 2), device=x.device,
                       dtype=torch.int8 if bits == 8 else torch.uint8)
    scales = torch.empty(rows, device=x.device, dtype=torch.float32)
    sum_out = torch.empty_like(x) if return_sum else None
    norm_out = torch.empty_like(x) if return_normed else None
    if gate is not None and (residual is None or tokens < 1 or gate.dtype != x.dtype or gate.numel() != expect):
        raise ValueError("A gate needs a residual branch, tokens >= 1 and one BF16 row per batch entry")
    shift = None if shift is None else shift.contiguous()
    with torch.cuda.device(x.device):
        if gate is None:
            code = _lib.load().rk_rmsnorm_quant_rows(
                _lib.ptr(x), _lib.ptr(residual), _lib.ptr(weight), _lib.ptr(shift), tokens, rows, k, eps, bits,
                _lib.ptr(sum_out), _lib.ptr(norm_out), _lib.ptr(data), _lib.ptr(scales), _lib.stream_ptr(x.device),
            )
        else:
            code = _lib.load().rk_gated_rmsnorm_quant_rows(
                _lib.ptr(x), _lib.ptr(residual), _lib.ptr(gate.contiguous()), _lib.ptr(weight), _lib.ptr(shift), tokens,
                rows, k, eps, bits, _lib.ptr(sum_out), _lib.ptr(norm_out), _lib.ptr(data), _lib.ptr(scales),
                _lib.stream_ptr(x.device),
            )
    _lib.check(code, "prepare_rmsnorm")
    packed = PackedActivations({bits: PackedActivation(data, scales, tuple(x.shape[:-1]), k, bits)})
    extras = tuple(t for t in (sum_out, norm_out) if t is not None)
    return (packed, *extras) if extras else packed


@dataclass
class PackedActivations:
    """Internal model boundary carrying only the requested integer formats
    (reference: modulation.py:239-265)."""

    packs: dict
    _robotics_packed_input = True

    def for_bits(self, bits):
        if bits not in self.packs:
            raise ValueError("A consumer requested an unprepared integer format")
        return self.packs[bits]

    def with_leading_shape(self, shape):
        shape = tuple(shape)
        if not shape or min(shape) < 1 or any(
            math.prod(shape) != pack.data.shape[0] for pack in self.packs.values()
        ):
            raise ValueError("Packed leading shape must preserve the row count")
        return PackedActivations({bits: replace(pack, shape=shape) for bits, pack in self.packs.items()})
