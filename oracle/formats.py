"""Bit-level number formats used by the quantized-linear path (CPU oracle; test infrastructure).

bf16 values travel through the oracle as float32 arrays whose values are exactly
representable in bf16.  8-bit and 4-bit codes travel as uint8 arrays.

Conversions restated here and the device instruction / library routine each one
stands for in the reference:

* ``e4m3_encode``  - ``cvt.rn.satfinite.e4m3x2.f32`` (``__nv_cvt_float_to_fp8(.., __NV_SATFINITE, __NV_E4M3)``,
  blackwell/csrc/fp8_cutlass_linear.cu:96-100; ``NumericArrayConverter<float_e4m3_t,float,4>``,
  blackwell/csrc/mxfp8_cutlass_linear.cu:77).
* ``ue4m3_encode`` - ``cutlass::float_ue4m3_t(float)`` (blackwell/csrc/fp4_cutlass_linear.cu:822).
* ``ue8m0_encode_roundup`` - ``cvt.rp.satfinite.ue8m0x2.f32`` behind ``NumericConverter<float_ue8m0_t,float>``
  (blackwell/csrc/mxfp8_common.cuh:24-27).
* ``e2m1_encode``  - ``__nv_cvt_float2_to_fp4x2(.., __NV_E2M1, cudaRoundNearest)``
  (blackwell/csrc/fp4_cutlass_linear.cu:832-835).
"""

import numpy as np

# Bit pattern of rcp.approx.ftz.f32(448.0f).  The MXFP8 packer multiplies the block
# maximum by this value (blackwell/csrc/mxfp8_common.cuh:25).  The correctly rounded
# fp32 reciprocal of 448 is 0x3B124925; a GPU test asserts that the B200 instruction
# returns exactly this pattern.
RCP_APPROX_448_BITS = 0x3B124925


def f32(x):
    return np.asarray(x, dtype=np.float32)


def f32_from_bits(bits):
    return np.asarray(bits, dtype=np.uint32).view(np.float32)


def bits_from_f32(x):
    return np.ascontiguousarray(f32(x)).view(np.uint32)


def bf16_bits(x):
    """Round float32 to bf16 (round-to-nearest-even, NaN kept quiet); return uint16 bit patterns."""
    u = bits_from_f32(x).astype(np.uint64)
    nan = np.isnan(f32(x))
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    out = np.where(nan, (u >> 16) | 0x40, rounded)
    return out.astype(np.uint16)


def bf16_from_bits(b):
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def bf16_round(x):
    """float32 -> bf16 -> float32."""
    return bf16_from_bits(bf16_bits(x))


def _encode_minifloat(x, ebits, mbits, bias, maxval, nan_code):
    x = f32(x)
    a = np.abs(x).astype(np.float64)
    sign = np.signbit(x).astype(np.int64)
    nan = np.isnan(a)
    a = np.where(nan, 0.0, np.minimum(a, maxval))
    emin = 1 - bias
    _, ex = np.frexp(a)
    e = np.maximum(ex.astype(np.int64) - 1, emin)
    step = np.exp2((e - mbits).astype(np.float64))
    val = np.minimum(np.rint(a / step) * step, maxval)
    _, ex2 = np.frexp(val)
    e2 = np.maximum(ex2.astype(np.int64) - 1, emin)
    sub = val < 2.0 ** emin
    mant = np.where(sub, val / 2.0 ** (emin - mbits),
                    (val / np.exp2(e2.astype(np.float64)) - 1.0) * (1 << mbits))
    expf = np.where(sub, 0, e2 + bias)
    code = (expf << mbits) | mant.astype(np.int64) | (sign << (ebits + mbits))
    return np.where(nan, nan_code, code).astype(np.uint8)


def _decode_minifloat(code, ebits, mbits, bias):
    c = np.asarray(code, dtype=np.int64)
    sign = (c >> (ebits + mbits)) & 1
    expf = (c >> mbits) & ((1 << ebits) - 1)
    mant = c & ((1 << mbits) - 1)
    emin = 1 - bias
    val = np.where(expf == 0, mant * 2.0 ** (emin - mbits),
                   (1.0 + mant / float(1 << mbits)) * np.exp2((expf - bias).astype(np.float64)))
    return np.where(sign == 1, -val, val).astype(np.float32)


def e4m3_encode(x):
    """float32 -> E4M3 (fn variant: no inf, max 448), RN-even, saturate-to-finite.  NaN -> 0x7F."""
    return _encode_minifloat(x, 4, 3, 7, 448.0, 0x7F)


def e4m3_decode(code):
    c = np.asarray(code, dtype=np.uint8)
    out = _decode_minifloat(c, 4, 3, 7)
    return np.where((c & 0x7F) == 0x7F, np.float32(np.nan), out).astype(np.float32)


def ue4m3_encode(x):
    """Non-negative float32 -> unsigned E4M3 scale byte (same bit layout as positive E4M3)."""
    return _encode_minifloat(np.maximum(f32(x), 0), 4, 3, 7, 448.0, 0x7F)


def ue4m3_decode(code):
    return e4m3_decode(np.asarray(code, dtype=np.uint8) & 0x7F)


def e2m1_encode(x):
    """float32 -> E2M1 nibble (0..15), RN-even, saturate to +-6."""
    return _encode_minifloat(x, 2, 1, 1, 6.0, 0x7)


def e2m1_decode(code):
    return _decode_minifloat(np.asarray(code, dtype=np.uint8) & 0xF, 2, 1, 1)


def ue8m0_encode_roundup(x):
    """Non-negative float32 -> UE8M0 byte: the smallest power of two >= x (biased by 127).

    Saturates at 254 (2^127); NaN gives 255; anything <= 2^-127 gives 0.
    """
    x = f32(x)
    b = bits_from_f32(x).astype(np.int64)
    expf = (b >> 23) & 0xFF
    mant = b & 0x7FFFFF
    up = np.where(expf == 0, np.where(mant > 0x400000, 1, 0), expf + (mant != 0))
    up = np.minimum(up, 254)
    up = np.where(np.signbit(x) & ~np.isnan(x), 0, up)
    return np.where(np.isnan(x), 255, up).astype(np.uint8)


def ue8m0_decode(code):
    """UE8M0 byte -> float32 (2^(code-127)); 255 is NaN."""
    c = np.asarray(code, dtype=np.int64)
    val = np.exp2((c - 127).astype(np.float64)).astype(np.float32)
    return np.where(c == 255, np.float32(np.nan), val).astype(np.float32)
