"""CPU oracle for the MXFP8 and NVFP4 block-scaled paths.  Test infrastructure.

MXFP8 follows blackwell/csrc/mxfp8_common.cuh:14-32 and blackwell/csrc/mxfp8_cutlass_linear.cu:31-80
(`pack_bf16_mxfp8_kernel`); NVFP4 follows blackwell/csrc/fp4_cutlass_linear.cu:686-690,789-841
(`sfa_offset`, `pack_matrix_fp4_ue_rowmajor_kernel`).  IEEE fp32 arithmetic throughout, except the
one approximate reciprocal the MXFP8 source asks for by name, which is a recorded constant.
PARITY UNPINNED by reference tests (the reference has none for these operators).
"""

import numpy as np

from .formats import (RCP_APPROX_448_BITS, bf16_round, e2m1_decode, e2m1_encode, e4m3_decode, e4m3_encode, f32,
                      f32_from_bits, ue4m3_decode, ue4m3_encode, ue8m0_decode, ue8m0_encode_roundup)


def sf_bytes(rows, groups):
    return ((rows + 127) // 128) * ((groups + 3) // 4) * 512


def sf_offsets(rows, groups):
    """Byte offset of scale factor (row, group) in the 128-row x 4-factor swizzled layout."""
    r = np.arange(rows, dtype=np.int64)[:, None]
    g = np.arange(groups, dtype=np.int64)[None, :]
    kt = (groups + 3) // 4
    return ((r // 128) * kt + g // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + g % 4


def swizzle_sf(sf):
    """[rows, groups] uint8 -> flat swizzled buffer (padding zero)."""
    rows, groups = sf.shape
    out = np.zeros(sf_bytes(rows, groups), dtype=np.uint8)
    out[sf_offsets(rows, groups)] = sf
    return out


def unswizzle_sf(buf, rows, groups):
    return np.asarray(buf, dtype=np.uint8)[sf_offsets(rows, groups)]


# ---- MXFP8 -------------------------------------------------------------------------------------

def pack_mxfp8(x):
    """x [rows, K] -> (codes uint8 [rows, K], sf uint8 [rows, K/32], swizzled sf buffer)."""
    x = f32(x)
    rows, k = x.shape
    if k % 32:
        raise ValueError("K must be a multiple of 32")
    b = x.reshape(rows, k // 32, 32)
    finite = np.isfinite(b).all(axis=2)
    amax = np.abs(np.where(np.isfinite(b), b, 0)).max(axis=2).astype(np.float32)
    mult = f32_from_bits(np.uint32(RCP_APPROX_448_BITS))
    sf = ue8m0_encode_roundup((amax * mult).astype(np.float32))
    sf = np.where(finite, sf, 255).astype(np.uint8)
    inverse = ue8m0_decode((254 - sf.astype(np.int64)) & 255)
    with np.errstate(invalid="ignore", over="ignore"):
        v = (b * inverse[:, :, None]).astype(np.float32)
    codes = e4m3_encode(v).reshape(rows, k)
    return codes, sf, swizzle_sf(sf)


def dequant_mxfp8(codes, sf):
    rows, k = codes.shape
    v = e4m3_decode(codes).reshape(rows, k // 32, 32).astype(np.float64)
    return (v * ue8m0_decode(sf).astype(np.float64)[:, :, None]).reshape(rows, k)


# ---- NVFP4 -------------------------------------------------------------------------------------

def pack_nvfp4(x, global_scale=None):
    """x [rows, K] -> (packed uint8 [rows, K/2], sf uint8 [rows, K/16], swizzled sf buffer)."""
    x = f32(x)
    if global_scale is not None:
        x = (x / np.float32(global_scale)).astype(np.float32)
    rows, k = x.shape
    if k % 32:
        raise ValueError("K must be a multiple of 32")
    b = x.reshape(rows, k // 16, 16)
    amax = np.abs(b).max(axis=2).astype(np.float32)
    scale = np.where(amax > 0, (amax / np.float32(6.0)).astype(np.float32), np.float32(1.0)).astype(np.float32)
    sf = ue4m3_encode(scale)
    deq = ue4m3_decode(sf)
    deq = np.where(deq > 0, deq, scale).astype(np.float32)
    reciprocal = (np.float32(1.0) / deq).astype(np.float32)
    v = (b * reciprocal[:, :, None]).astype(np.float32)
    codes = e2m1_encode(v).reshape(rows, k).astype(np.uint8)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    return packed, sf, swizzle_sf(sf)


def swiglu_bf16_steps(gate_up, inter):
    """SwiGLU with every intermediate rounded to bf16, the way the reference's NVFP4 producer computes
    it in packed bf16 arithmetic (blackwell/csrc/fp4_cutlass_linear.cu:1029-1033):
    e = bf16(exp(-g)); d = bf16(1 + e); r = bf16(1 / d); a = bf16(bf16(g * r) * up)."""
    g = f32(gate_up[:, :inter])
    u = f32(gate_up[:, inter:2 * inter])
    with np.errstate(over="ignore"):
        e = bf16_round(np.exp(-g.astype(np.float64)).astype(np.float32))
    d = bf16_round((np.float32(1.0) + e).astype(np.float32))
    with np.errstate(divide="ignore"):
        r = bf16_round((np.float32(1.0) / d).astype(np.float32))
    return bf16_round((bf16_round((g * r).astype(np.float32)) * u).astype(np.float32))


def swiglu_pack_nvfp4(gate_up, inter):
    a = swiglu_bf16_steps(gate_up, inter)
    return pack_nvfp4(a) + (a,)


def rms_norm_pack_nvfp4(x, residual, weight, eps):
    """(residual add +) RMSNorm -> NVFP4 (blackwell/csrc/fp4_cutlass_linear.cu:843-929).
    Returns (summed, normalized, packed, sf, swizzled sf)."""
    from .fp8 import rms_norm

    s, y = rms_norm(x, residual, weight, eps)
    return (s, y) + pack_nvfp4(y)


def dequant_nvfp4(packed, sf, global_scale=None):
    p = np.asarray(packed, dtype=np.uint8)
    rows = p.shape[0]
    codes = np.empty((rows, p.shape[1] * 2), dtype=np.uint8)
    codes[:, 0::2] = p & 15
    codes[:, 1::2] = p >> 4
    k = codes.shape[1]
    v = e2m1_decode(codes).reshape(rows, k // 16, 16).astype(np.float64)
    out = (v * ue4m3_decode(sf).astype(np.float64)[:, :, None]).reshape(rows, k)
    if global_scale is not None:
        out = out * float(np.float32(global_scale))
    return out


# ---- W4A8 MX: MXFP4 weights x MXFP8 activations (blackwell/csrc/fp4_mx_cutlass_linear.cu:47-179) ------

def ceil_pow2_ue8m0(v):
    """UE8M0 byte of the smallest power of two >= v (`ceil_power_of_two`, :47-58): 127 (= 1.0) for v <= 0
    or NaN; inputs below the smallest normal number map to byte 1."""
    v = f32(v)
    bits = v.view(np.uint32)
    e = (bits >> 23).astype(np.int64)
    e = e + ((bits & 0x7FFFFF) != 0)
    e = np.where((bits >> 23) == 0, 1, e)
    e = np.minimum(e, 254)
    return np.where(v > 0, e, 127).astype(np.uint8)


def pack_mxfp8_ceil(x):
    """Activation side: per 32 k, s = ceil_pow2(amax / 448), q = e4m3(clamp(x / s, +-448)) (:103-132)."""
    x = f32(x)
    rows, k = x.shape
    b = x.reshape(rows, k // 32, 32)
    amax = np.abs(b).max(axis=2).astype(np.float32)
    sf = ceil_pow2_ue8m0((amax / np.float32(448.0)).astype(np.float32))
    inverse = ue8m0_decode((254 - sf.astype(np.int64)) & 255)
    v = np.clip((b * inverse[:, :, None]).astype(np.float32), -448.0, 448.0)
    return e4m3_encode(v).reshape(rows, k), sf, swizzle_sf(sf)


def pack_mxfp4_ceil(w):
    """Weight side: per 32 k, s = ceil_pow2(amax / 6), q = e2m1(w / s), low nibble = even k (:59-100)."""
    w = f32(w)
    rows, k = w.shape
    b = w.reshape(rows, k // 32, 32)
    amax = np.abs(b).max(axis=2).astype(np.float32)
    sf = ceil_pow2_ue8m0((amax / np.float32(6.0)).astype(np.float32))
    inverse = ue8m0_decode((254 - sf.astype(np.int64)) & 255)
    codes = e2m1_encode((b * inverse[:, :, None]).astype(np.float32)).reshape(rows, k).astype(np.uint8)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    return packed, sf, swizzle_sf(sf)


def dequant_mxfp4(packed, sf):
    p = np.asarray(packed, dtype=np.uint8)
    rows = p.shape[0]
    codes = np.empty((rows, p.shape[1] * 2), dtype=np.uint8)
    codes[:, 0::2] = p & 15
    codes[:, 1::2] = p >> 4
    k = codes.shape[1]
    v = e2m1_decode(codes).reshape(rows, k // 32, 32).astype(np.float64)
    return (v * ue8m0_decode(sf).astype(np.float64)[:, :, None]).reshape(rows, k)


def deinterleave_gate_up(gate_up, inter):
    """Interleaved layout (blocks of 128 columns: 64 up values, then their 64 gate values;
    blackwell/csrc/fp4_cutlass_linear.cu:958-965) -> [gate | up]."""
    g = np.asarray(gate_up)
    rows = g.shape[0]
    blocks = g.reshape(rows, inter // 64, 2, 64)
    return np.concatenate([blocks[:, :, 1, :].reshape(rows, inter), blocks[:, :, 0, :].reshape(rows, inter)], axis=1)


def swiglu_f32(gate_up, inter):
    """gate / (1 + exp(-gate)) * up in fp32, NOT rounded to bf16 (the W4A8-MX producer, :134-179)."""
    g = f32(gate_up[:, :inter])
    u = f32(gate_up[:, inter:2 * inter])
    with np.errstate(over="ignore"):
        e = np.exp(-g.astype(np.float64)).astype(np.float32)
    return ((g / (np.float32(1.0) + e)).astype(np.float32) * u).astype(np.float32)


def gemm_dequantized(a, b, bias=None):
    """bf16(a . b^T (+ bias)) on dequantized float64 operands; returns (bf16-rounded, float64)."""
    acc = a @ b.T
    if bias is not None:
        acc = acc + f32(bias).astype(np.float64)[None, :]
    return bf16_round(acc.astype(np.float32)), acc


def rel_frobenius(actual, expected):
    e = np.asarray(expected, dtype=np.float64)
    d = np.asarray(actual, dtype=np.float64) - e
    return float(np.sqrt((d * d).sum()) / max(np.sqrt((e * e).sum()), 1e-30))


def silu_mul_pack_mxfp8(gate_up, inter, table):
    """`robotics_mxfp8_swiglu::silu_mul_pack` (blackwell/csrc/mxfp8_swiglu.cu:20-78): the value packed is
    bf16( table[bits(gate)] * up ), `table` the 65536 SiLU values as float32; then `pack_mxfp8`.
    gate_up float32 [rows, 2 * inter] holding bf16 values, gate first.  -> (codes, scales, swizzled)."""
    from .formats import bf16_bits, bf16_round

    gate_up = np.asarray(gate_up, dtype=np.float32)
    gate, up = gate_up[:, :inter], gate_up[:, inter:]
    silu = np.asarray(table, dtype=np.float32)[bf16_bits(gate).astype(np.int64)]
    return pack_mxfp8(bf16_round((silu * up).astype(np.float32)))
