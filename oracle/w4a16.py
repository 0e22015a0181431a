"""CPU oracle for the W4A16 group-wise int4 path.  Test infrastructure.

The format is defined by the benchmark configuration, not by the reference (whose W4A16 uses
E2M1 weights with 16-wide groups, blackwell/csrc/fp4_mixed_cutlass_linear.cu:27,205-206).
Conventions follow the reference's int4 packing (src/robotics_kernels/ampere_ada/integer.py:250-263:
symmetric, limit 7, two's-complement nibbles, low nibble = even k) and its mixed-input scale
orientation ([K/group, N], blackwell/csrc/fp4_mixed_cutlass_linear.cu:89-90,122).
PARITY UNPINNED: no reference code or test produces this format.
"""

import numpy as np

from .formats import bf16_round, f32
from .integer import pack_nibbles, unpack_nibbles

GROUP = 128


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
    return pack_nibbles(q), np.ascontiguousarray(s.T), q


def dequantize(packed, scales):
    q = unpack_nibbles(packed).astype(np.float32)
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
