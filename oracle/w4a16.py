"""CPU oracle for the W4A16 group-wise int4 path.  Test infrastructure.

The format is defined by the benchmark configuration, not by the reference (whose W4A16 uses
E2M1 weights with 16-wide groups, blackwell/csrc/fp4_mixed_cutlass_linear.cu:27,205-206).
Quantisation follows the reference's int4 rules (src/robotics_kernels/ampere_ada/integer.py:250-263:
symmetric, limit 7, two's-complement nibbles) and its mixed-input scale orientation ([K/group, N],
blackwell/csrc/fp4_mixed_cutlass_linear.cu:89-90,122).  Nibble order inside the packed bytes is this
format's own: eight consecutive weights k0..k7 occupy four bytes, byte b = k_b | k_{b+4} << 4.
PARITY UNPINNED: no reference code or test produces this format.
"""

import numpy as np

from .formats import bf16_round, f32

GROUP = 128


def pack_nibbles8(q):
    """int8 codes [N, K] (K % 8 == 0) -> uint8 [N, K/2]: byte b of each 4-byte word = k_b | k_{b+4} << 4."""
    n, k = q.shape
    u = (q.astype(np.int16) & 15).astype(np.uint8).reshape(n, k // 8, 8)
    return np.ascontiguousarray((u[:, :, :4] | (u[:, :, 4:] << 4)).reshape(n, k // 2))


def unpack_nibbles8(packed):
    """Inverse of `pack_nibbles8`: uint8 [N, K/2] -> int8 codes [N, K] (two's-complement nibbles)."""
    n, half = packed.shape
    b = np.asarray(packed, dtype=np.uint8).reshape(n, half // 4, 4)
    u = np.concatenate([b & 15, b >> 4], axis=2).astype(np.int16)  # k0..k3, k4..k7
    return np.where(u >= 8, u - 16, u).astype(np.int8).reshape(n, half * 2)


def pack_weight(w):
    """w [N, K] (bf16 values) -> (packed uint8 [N, K/2], scales float32 [K/128, N] holding bf16 values, codes int8 [N, K])."""
    w = f32(w)
    n, k = w.shape
    if k % GROUP:
        raise ValueError("K must be a multiple of 128")
    g = w.reshape(n, k // GROUP, GROUP)
    amax = np.abs(g).max(axis=2)
    s = bf16_round(np.where(amax > 0, (amax / np.float32(7.0)).astype(np.float32), np.float32(1.0)))
    s = np.where(s > 0, s, np.float32(1.0)).astype(np.float32)
    q = np.rint((g / s[:, :, None]).astype(np.float32))
    q = np.clip(q, -7, 7).astype(np.int8).reshape(n, k)
    return pack_nibbles8(q), np.ascontiguousarray(s.T), q


def dequantize(packed, scales):
    q = unpack_nibbles8(packed).astype(np.float32)
    n, k = q.shape
    s = f32(scales).T  # [N, K/128]
    return (q.reshape(n, k // GROUP, GROUP) * s[:, :, None]).astype(np.float32).reshape(n, k)


def gemm(x, packed, scales, bias=None):
    """bf16( fp32 matmul(x, dequantized weights) (+ bias) ); returns (bf16-rounded, unrounded float64)."""
    w = dequantize(packed, scales).astype(np.float64)
    acc = f32(x).astype(np.float64) @ w.T
    if bias is not None:
        acc = acc + f32(bias).astype(np.float64)[None, :]
    return bf16_round(acc.astype(np.float32)), acc


def dequantize_folded(packed, scales):
    """Weights as the wide-batch kernel forms them: bf16(q * s), one rounding per weight - the
    "dequantize to bf16, then multiply" order of the reference's mixed-input GEMM
    (blackwell/csrc/fp4_mixed_cutlass_linear.cu:190-260)."""
    return bf16_round(dequantize(packed, scales))


def gemm_folded(x, packed, scales, bias=None):
    """As `gemm`, with the group scale folded into bf16 weights before the product."""
    w = dequantize_folded(packed, scales).astype(np.float64)
    acc = f32(x).astype(np.float64) @ w.T
    if bias is not None:
        acc = acc + f32(bias).astype(np.float64)[None, :]
    return bf16_round(acc.astype(np.float32)), acc
