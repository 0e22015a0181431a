"""CPU oracle for the symmetric integer path (W8A8 / W4A4).  Test infrastructure.

Follows, line by line:

* row quantizer          - src/robotics_kernels/ampere_ada/integer.py:52-119 (``_activation_values``, ``_prepare``)
* weight quantizer       - src/robotics_kernels/ampere_ada/integer.py:247-263 (``IntegerLinear.from_linear``)
* GEMM + dequant epilogue - src/robotics_kernels/ampere_ada/csrc/integer_gemm.cu:47-59 (EVT tree
  ``Mul0(Acc,Row) -> Mul1(.,Col) -> Add(.,Bias) -> bf16``; built with ``--fmad=false``)
* known-answer formula   - tests/gpu/test_integer_linear.py:30-37
* AdaLN modulation pack  - src/robotics_kernels/ampere_ada/modulation.py:13-146

bf16 tensors are float32 numpy arrays holding bf16-representable values.
"""

import numpy as np

from .formats import bf16_round, f32


def limit_for(bits):
    if bits not in (4, 8):
        raise ValueError("bits must be 4 or 8")
    return (1 << (bits - 1)) - 1


def pad128(k):
    return (k + 127) // 128 * 128


def pack_nibbles(q):
    """int codes [rows, K even] -> bytes [rows, K/2]; low nibble holds the even index."""
    q = np.asarray(q).astype(np.int32) & 15
    return (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(p):
    """bytes [rows, K/2] -> signed int8 codes [rows, K] (two's-complement nibbles)."""
    p = np.asarray(p, dtype=np.uint8).astype(np.int32)
    lo = p & 15
    hi = p >> 4
    out = np.empty((p.shape[0], p.shape[1] * 2), dtype=np.int32)
    out[:, 0::2] = lo
    out[:, 1::2] = hi
    return np.where(out >= 8, out - 16, out).astype(np.int8)


def activation_values(x, up=None, lut=None):
    """Pre-quantization values of ``_activation_values``: plain, LUT[x], or bf16(LUT[x] * up)."""
    x = f32(x)
    if lut is None:
        return x
    from .formats import bf16_bits
    value = f32(lut)[bf16_bits(x).astype(np.int64)]
    if up is not None:
        value = bf16_round(value * f32(up))
    return value


def quantize_rows(x, bits, up=None, lut=None):
    """Per-row symmetric absmax quantization.

    scale = max|x| * fl32(1/limit) (1.0 for an all-zero row); q = clamp(rint(x / scale), +-limit)
    with IEEE fp32 division; K zero-padded to a multiple of 128; int4 packed two per byte.
    Returns (data, scales, values) with data int8 [rows, Kpad] or uint8 [rows, Kpad/2].
    """
    limit = limit_for(bits)
    v = activation_values(x, up, lut)
    rows, k = v.shape
    maximum = np.abs(v).max(axis=1) if k else np.zeros(rows, np.float32)
    reciprocal = np.float32(1.0 / limit)
    scale = np.where(maximum > 0, (maximum * reciprocal).astype(np.float32), np.float32(1.0)).astype(np.float32)
    with np.errstate(invalid="ignore", divide="ignore", over="ignore"):
        q = np.rint((v / scale[:, None]).astype(np.float32))
    q = np.minimum(np.maximum(q, -limit), limit)
    q = np.where(np.isnan(q), 0, q).astype(np.int32)
    kp = pad128(k)
    full = np.zeros((rows, kp), dtype=np.int32)
    full[:, :k] = q
    data = full.astype(np.int8) if bits == 8 else pack_nibbles(full)
    return data, scale, v


def quantize_weight(w, bits):
    """Per-output-channel symmetric weight quantization with true division.

    s = max_k|w| / limit (1.0 when zero); q = clamp(round_half_even(w / s)); N padded to x8
    (scale pad 1.0), K padded to x128.  Returns (packed, scales[Npad], codes int8 [Npad, Kpad]).
    """
    limit = limit_for(bits)
    w = f32(w)
    if not np.isfinite(w).all():
        raise ValueError("Weights must be finite")
    n, k = w.shape
    maximum = np.abs(w).max(axis=1)
    scales = np.where(maximum > 0, (maximum / np.float32(limit)).astype(np.float32), np.float32(1.0)).astype(np.float32)
    q = np.rint((w / scales[:, None]).astype(np.float32))
    q = np.minimum(np.maximum(q, -limit), limit).astype(np.int8)
    npad = (n + 7) // 8 * 8
    kp = pad128(k)
    codes = np.zeros((npad, kp), dtype=np.int8)
    codes[:n, :k] = q
    sp = np.ones(npad, dtype=np.float32)
    sp[:n] = scales
    packed = codes if bits == 8 else pack_nibbles(codes)
    return packed, sp, codes


def int_matmul(a_codes, b_codes):
    """Exact int32 accumulators of A[M,K] . B[N,K]^T (float64 BLAS is exact for these magnitudes)."""
    acc = np.asarray(a_codes, dtype=np.float64) @ np.asarray(b_codes, dtype=np.float64).T
    return acc.astype(np.int64).astype(np.int32)


def dequant_epilogue(acc, sa, sb, bias=None):
    """bf16( fl(fl(float(acc) * sa[m]) * sb[n]) (+ float(bias[n])) ), every step rounded to fp32."""
    t = np.asarray(acc, dtype=np.int32).astype(np.float32)
    t = (t * f32(sa)[:, None]).astype(np.float32)
    t = (t * f32(sb)[None, :]).astype(np.float32)
    if bias is not None:
        t = (t + f32(bias)[None, :]).astype(np.float32)
    return bf16_round(t)


def gemm(a_data, sa, b_data, sb, bias, bits):
    """Oracle for ``robotics_integer::gemm``: packed operands in, (bf16 out [M,Npad], int32 acc) out."""
    a = a_data if bits == 8 else unpack_nibbles(a_data)
    b = b_data if bits == 8 else unpack_nibbles(b_data)
    acc = int_matmul(a, b)
    return dequant_epilogue(acc, sa, sb, bias), acc


def linear(x, w, bias, bits, up=None, lut=None):
    """quantize activations + weights, GEMM, epilogue; output sliced to the logical N."""
    a, sa, _ = quantize_rows(x, bits, up, lut)
    b, sb, _ = quantize_weight(w, bits)
    n = np.asarray(w).shape[0]
    pb = None
    if bias is not None:
        pb = np.zeros(b.shape[0], dtype=np.float32)
        pb[:n] = f32(bias)
    out, acc = gemm(a, sa, b, sb, pb, bits)
    return out[:, :n], acc[:, :n]


def known_answer(x, w, bias, bits):
    """The reference GPU test's own formula (true division for both scales, fp32 matmul)."""
    limit = np.float32(limit_for(bits))
    x = f32(x)
    w = f32(w)
    ws = (np.maximum(np.abs(w).max(axis=1), np.float32(1e-30)) / limit).astype(np.float32)
    xs = (np.maximum(np.abs(x).max(axis=1), np.float32(1e-30)) / limit).astype(np.float32)
    qw = np.clip(np.rint((w / ws[:, None]).astype(np.float32)), -limit, limit).astype(np.float32)
    qx = np.clip(np.rint((x / xs[:, None]).astype(np.float32)), -limit, limit).astype(np.float32)
    t = (qx @ qw.T).astype(np.float32)
    t = (t * xs[:, None]).astype(np.float32)
    t = (t * ws[None, :]).astype(np.float32)
    t = (t + f32(bias)[None, :]).astype(np.float32)
    return bf16_round(t)


# --- AdaLN modulation feeding the row quantizer (modulation.py:13-146) -----------------------

def modulated_values(x, scale, shift, tokens):
    """bf16(bf16(x * bf16(1 + scale)) + shift); scale/shift rows are shared by `tokens` consecutive rows."""
    x = f32(x)
    rows = x.shape[0]
    idx = np.arange(rows) // tokens
    sc = f32(scale)[idx]
    sh = f32(shift)[idx]
    factor = bf16_round((np.float32(1.0) + sc).astype(np.float32))
    product = bf16_round((x * factor).astype(np.float32))
    return bf16_round((product + sh).astype(np.float32))


def layer_norm_values(x, eps):
    """Non-affine LayerNorm in fp32 (two-pass mean/variance), result rounded to bf16."""
    x = f32(x)
    k = x.shape[1]
    mean = (x.sum(axis=1, dtype=np.float32) / np.float32(k)).astype(np.float32)
    centered = (x - mean[:, None]).astype(np.float32)
    var = ((centered * centered).sum(axis=1, dtype=np.float32) / np.float32(k)).astype(np.float32)
    inv = (np.float32(1.0) / np.sqrt((var + np.float32(eps)).astype(np.float32))).astype(np.float32)
    return bf16_round((centered * inv[:, None]).astype(np.float32))


def gated_residual_values(x, y, gate, tokens):
    """bf16(x + bf16(y * gate)); gate rows shared by `tokens` consecutive rows."""
    x = f32(x)
    idx = np.arange(x.shape[0]) // tokens
    product = bf16_round((f32(y) * f32(gate)[idx]).astype(np.float32))
    return bf16_round((x + product).astype(np.float32))


def prepare_modulation(x, scale, shift, tokens, bits, norm_eps=None, y=None, gate=None):
    """Oracle for prepare_modulation / prepare_norm_modulation / prepare_residual_norm_modulation.

    Returns (data, scales, residual_or_None).
    """
    residual = None
    v = f32(x)
    if y is not None:
        residual = gated_residual_values(v, y, gate, tokens)
        v = residual
    if norm_eps is not None:
        v = layer_norm_values(v, norm_eps)
    v = modulated_values(v, scale, shift, tokens)
    data, s, _ = quantize_rows(v, bits)
    return data, s, residual
