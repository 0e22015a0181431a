"""CPU oracle for the per-tensor FP8 (E4M3) path.  Test infrastructure.

Follows blackwell/csrc/fp8_cutlass_linear.cu:61-101 (`bf16_amax_kernel`, `finalize_scale_kernel`,
`bf16_to_fp8_kernel`) with IEEE fp32 arithmetic (the reference builds with fast-math, so its
device reciprocal is approximate; see the module docstring of ``oracle``), and the epilogue
``bf16(scale_a * scale_b * acc + bias[n])`` (:636-643).  PARITY UNPINNED by reference tests.
"""

import numpy as np

from .formats import bf16_round, e4m3_decode, e4m3_encode, f32

FP8_MAX = np.float32(448.0)
MIN_SCALE = np.float32(1e-12)


def tensor_scale(x, divisor=FP8_MAX):
    a = np.abs(f32(x))
    a = np.where(np.isfinite(a), a, np.float32(0))
    amax = a.max() if a.size else np.float32(0)
    return np.maximum((np.float32(amax) / np.float32(divisor)).astype(np.float32), MIN_SCALE).astype(np.float32)


def quantize_with_scale(x, scale):
    inverse = (np.float32(1.0) / np.float32(scale)).astype(np.float32)
    v = (f32(x) * inverse).astype(np.float32)
    v = np.minimum(FP8_MAX, np.maximum(-FP8_MAX, v))
    return e4m3_encode(v)


def quantize(x):
    s = tensor_scale(x)
    return quantize_with_scale(x, s), s


def gemm(a_codes, scale_a, b_codes, scale_b, bias=None):
    """Returns (bf16-rounded output, float64 unrounded)."""
    a = e4m3_decode(a_codes).astype(np.float64)
    b = e4m3_decode(b_codes).astype(np.float64)
    acc = (a @ b.T) * float(np.float32(scale_a) * np.float32(scale_b))
    if bias is not None:
        acc = acc + f32(bias).astype(np.float64)[None, :]
    return bf16_round(acc.astype(np.float32)), acc


# ---- fused producers (blackwell/csrc/fp8_cutlass_linear.cu:145-389) ------------------------------

def rms_norm(x, residual, weight, eps):
    """s = bf16(x + residual); r = rsqrt(mean(s^2) + eps); y = bf16(bf16(s * r) * weight).
    Returns (summed, normalized) as float32 arrays holding bf16 values.  The sum of squares is taken
    in float64 and rounded once (the kernel's fp32 tree order is not part of the contract); the
    device rsqrt is approximate, which the bf16 roundings absorb except at rare ties."""
    s = f32(x)
    if residual is not None:
        s = bf16_round((s + f32(residual)).astype(np.float32))
    k = s.shape[-1]
    mean = (np.square(s.astype(np.float64)).sum(axis=-1) / k).astype(np.float32)
    r = (1.0 / np.sqrt((mean + np.float32(eps)).astype(np.float64))).astype(np.float32)
    y = bf16_round((s * r[..., None]).astype(np.float32))
    y = bf16_round((y * f32(weight)[None, :]).astype(np.float32))
    return s, y


def add_rms_norm_quantize(x, residual, weight, eps):
    """Returns (summed, normalized, codes, scale)."""
    s, y = rms_norm(x, residual, weight, eps)
    codes, scale = quantize(y)
    return s, y, codes, scale


def swiglu(gate_up, inter):
    """bf16( gate / (1 + exp(-gate)) * up ) evaluated in fp32 (fp8_cutlass_linear.cu:271-279)."""
    g = f32(gate_up[:, :inter])
    u = f32(gate_up[:, inter:2 * inter])
    with np.errstate(over="ignore"):
        e = np.exp(-g.astype(np.float64)).astype(np.float32)
    act = (g / (np.float32(1.0) + e)).astype(np.float32)
    return bf16_round((act * u).astype(np.float32))


def quantize_swiglu(gate_up, inter, scale=None):
    a = swiglu(gate_up, inter)
    if scale is None:
        scale = tensor_scale(a)
    return quantize_with_scale(a, scale), np.float32(scale), a
