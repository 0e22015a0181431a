"""GPU parity of the per-tensor FP8, MXFP8 and NVFP4 paths: quantized codes and scales bit-exact
against the CPU oracle, GEMMs within 1e-2 relative Frobenius error of dequantize -> matmul."""

import ctypes

import numpy as np
import pytest
import torch

from oracle import blockscale as OB
from oracle import formats as F
from oracle import fp8 as OF
from rk_b200 import _lib

pytestmark = pytest.mark.gpu
TOL = 1e-2
# the last three take the CTA-pair kernel (512 activation rows and more): ragged n and K, full size
SHAPES = [(16, 128, 128), (64, 256, 512), (100, 520, 448), (300, 264, 320), (600, 328, 320), (1100, 520, 448),
          (816, 16384, 2048)]


@pytest.fixture(scope="module")
def H():
    import gpu_helpers

    return gpu_helpers


def out_buffer(H, m, n):
    buf = torch.full((m + 2, n), 7.0, dtype=torch.bfloat16, device=H.DEVICE)
    return buf, buf[1:m + 1]


def check_canaries(buf, m):
    assert (buf[0] == 7.0).all() and (buf[m + 1] == 7.0).all()


def test_rcp_approx_constant_matches_the_oracle(H):
    value = ctypes.c_uint32(0)
    H.call("rk_probe_rcp_approx_448", ctypes.byref(value))
    assert value.value == F.RCP_APPROX_448_BITS


# ---------------------------------------------------------------- per-tensor FP8
def fp8_quant(H, x):
    ws = _lib.workspace(H.DEVICE, 1 << 20)
    q = torch.empty(x.shape, dtype=torch.uint8, device=H.DEVICE)
    s = torch.zeros(1, dtype=torch.float32, device=H.DEVICE)
    H.call("rk_quant_tensor_fp8", _lib.ptr(x), x.numel(), _lib.ptr(q), _lib.ptr(s), _lib.ptr(ws), ws.numel(),
           H.stream())
    return q, s


@pytest.mark.parametrize("shape", SHAPES)
def test_fp8_quantize_and_gemm(H, shape):
    m, n, k = shape
    x, w, bias = H.randn_bf16((m, k), 1.0, 7), H.randn_bf16((n, k), 0.02, 8), H.randn_bf16((n,), 0.01, 9)
    if m > 16:
        x[3, 5] = float("inf")  # non-finite values are skipped by the amax and saturate to 448
    qa, sa = fp8_quant(H, x.to(H.DEVICE))
    qb, sb = fp8_quant(H, w.to(H.DEVICE))
    xin = H.to_np(x)
    ea, esa = OF.quantize(xin)
    eb, esb = OF.quantize(H.to_np(w))
    assert sa.item() == esa and sb.item() == esb
    assert np.array_equal(qa.cpu().numpy(), ea) and np.array_equal(qb.cpu().numpy(), eb)
    buf, out = out_buffer(H, m, n)
    ws = _lib.gemm_workspace(_lib.OP_FP8, H.DEVICE, m, n, k)
    H.call("rk_gemm_fp8", _lib.ptr(qa), _lib.ptr(sa), _lib.ptr(qb), _lib.ptr(sb), _lib.ptr(bias.to(H.DEVICE)),
           _lib.ptr(out), m, n, k, 0, _lib.ptr(ws), ws.numel(), H.stream())
    assert _lib.read_status(ws) == 0
    check_canaries(buf, m)
    _, want = OF.gemm(ea, esa, eb, esb, H.to_np(bias))
    assert H.rel_frobenius(H.to_np(out), want) < TOL
    assert H.workspace_is_clean(ws)


def test_fp8_quantize_with_supplied_scale(H):
    x = H.randn_bf16((33, 160), 3.0, 2)
    scale = torch.tensor([0.0125], dtype=torch.float32, device=H.DEVICE)
    q = torch.empty(x.shape, dtype=torch.uint8, device=H.DEVICE)
    H.call("rk_quant_tensor_fp8_with_scale", _lib.ptr(x.to(H.DEVICE)), x.numel(), _lib.ptr(scale), _lib.ptr(q),
           H.stream())
    assert np.array_equal(q.cpu().numpy(), OF.quantize_with_scale(H.to_np(x), np.float32(0.0125)))


# ---------------------------------------------------------------- MXFP8
def mx_pack(H, x):
    rows, k = x.shape
    q = torch.empty((rows, k), dtype=torch.uint8, device=H.DEVICE)
    sf = torch.full((_lib.load().rk_sf_bytes(rows, k // 32),), 0x63, dtype=torch.uint8, device=H.DEVICE)
    H.call("rk_pack_mxfp8", _lib.ptr(x), rows, k, _lib.ptr(q), _lib.ptr(sf), H.stream())
    return q, sf


@pytest.mark.parametrize("shape", SHAPES)
def test_mxfp8_pack_and_gemm(H, shape):
    m, n, k = shape
    x, w, bias = H.randn_bf16((m, k), 1.0, 10), H.randn_bf16((n, k), 0.02, 11), H.randn_bf16((n,), 0.01, 12)
    x[0, :32] = 0                # an all-zero block
    x[1, 0:4] = torch.tensor([3.5, -1.75, 448.0, 0.4375]).to(torch.bfloat16)  # amax = 448 * 2^0: power-of-two edge
    qa, sfa = mx_pack(H, x.to(H.DEVICE))
    qb, sfb = mx_pack(H, w.to(H.DEVICE))
    ca, sa, swa = OB.pack_mxfp8(H.to_np(x))
    cb, sb, swb = OB.pack_mxfp8(H.to_np(w))
    assert np.array_equal(sfa.cpu().numpy(), swa) and np.array_equal(sfb.cpu().numpy(), swb)
    assert np.array_equal(qa.cpu().numpy(), ca) and np.array_equal(qb.cpu().numpy(), cb)
    buf, out = out_buffer(H, m, n)
    ws = _lib.gemm_workspace(_lib.OP_MXFP8, H.DEVICE, m, n, k)
    H.call("rk_gemm_mxfp8", _lib.ptr(qa), _lib.ptr(sfa), _lib.ptr(qb), _lib.ptr(sfb), _lib.ptr(bias.to(H.DEVICE)),
           _lib.ptr(out), m, n, k, 0, _lib.ptr(ws), ws.numel(), H.stream())
    assert _lib.read_status(ws) == 0
    check_canaries(buf, m)
    _, want = OB.gemm_dequantized(OB.dequant_mxfp8(ca, sa), OB.dequant_mxfp8(cb, sb), H.to_np(bias))
    assert H.rel_frobenius(H.to_np(out), want) < TOL


def test_mxfp8_nonfinite_block_gets_nan_scale(H):
    x = H.randn_bf16((4, 64), 1.0, 13)
    x[2, 40] = float("nan")
    _, sf = mx_pack(H, x.to(H.DEVICE))
    assert OB.unswizzle_sf(sf.cpu().numpy(), 4, 2)[2, 1] == 255
    assert np.array_equal(sf.cpu().numpy(), OB.pack_mxfp8(H.to_np(x))[2])


# ---------------------------------------------------------------- NVFP4
def nv_pack(H, x, global_scale=None):
    rows, k = x.shape
    q = torch.empty((rows, k // 2), dtype=torch.uint8, device=H.DEVICE)
    sf = torch.full((_lib.load().rk_sf_bytes(rows, k // 16),), 0x63, dtype=torch.uint8, device=H.DEVICE)
    H.call("rk_pack_nvfp4", _lib.ptr(x), rows, k, _lib.ptr(global_scale), _lib.ptr(q), _lib.ptr(sf), H.stream())
    return q, sf


@pytest.mark.parametrize("shape", SHAPES)
def test_nvfp4_pack_and_gemm_reference_mode(H, shape):
    """No per-tensor scale (alpha = 1), as in the reference."""
    m, n, k = shape
    x, w, bias = H.randn_bf16((m, k), 1.0, 13), H.randn_bf16((n, k), 0.02, 14), H.randn_bf16((n,), 0.01, 15)
    x[0, :16] = 0
    qa, sfa = nv_pack(H, x.to(H.DEVICE))
    qb, sfb = nv_pack(H, w.to(H.DEVICE))
    pa, sa, swa = OB.pack_nvfp4(H.to_np(x))
    pb, sb, swb = OB.pack_nvfp4(H.to_np(w))
    assert np.array_equal(sfa.cpu().numpy(), swa) and np.array_equal(sfb.cpu().numpy(), swb)
    assert np.array_equal(qa.cpu().numpy(), pa) and np.array_equal(qb.cpu().numpy(), pb)
    buf, out = out_buffer(H, m, n)
    ws = _lib.gemm_workspace(_lib.OP_NVFP4, H.DEVICE, m, n, k)
    H.call("rk_gemm_nvfp4", _lib.ptr(qa), _lib.ptr(sfa), None, _lib.ptr(qb), _lib.ptr(sfb), None,
           _lib.ptr(bias.to(H.DEVICE)), _lib.ptr(out), m, n, k, 0, _lib.ptr(ws), ws.numel(), H.stream())
    assert _lib.read_status(ws) == 0
    check_canaries(buf, m)
    _, want = OB.gemm_dequantized(OB.dequant_nvfp4(pa, sa), OB.dequant_nvfp4(pb, sb), H.to_np(bias))
    assert H.rel_frobenius(H.to_np(out), want) < TOL


@pytest.mark.parametrize("divisor", [0.0123, 2.0 ** -9, float(np.float32(1.9999999) * np.float32(2.0 ** -7)), 2.0 ** -50, 3.0e5])
def test_nvfp4_pack_division_by_the_tensor_scale_is_exact(H, divisor):
    """The packer divides by the per-tensor scale with a reciprocal and an exact residual correction where
    that is provably the IEEE quotient, and with the IEEE division elsewhere (zeros of either sign, tiny
    and huge values, a divisor whose significand is all ones, divisors outside 2^-40 .. 2^40): every bf16
    value with an exponent in -70 .. 70, both signs, and the zeros give the oracle's codes and scale bytes."""
    bits = np.arange(65536, dtype=np.uint32)
    vals = (bits << 16).view(np.float32)
    mag = np.abs(vals)
    keep = (mag == 0) | ((mag >= 2.0 ** -70) & (mag <= 2.0 ** 70))
    vals = vals[keep]
    rng = np.random.default_rng(5)
    vals = np.concatenate([vals, rng.permutation(vals)])  # blocks of neighbours and blocks of mixed magnitudes
    pad = (-len(vals)) % 64
    vals = np.concatenate([vals, np.zeros(pad, dtype=np.float32)]).reshape(-1, 64)
    x = torch.from_numpy(vals).to(torch.bfloat16)
    assert np.array_equal(H.to_np(x), vals)  # all values are bf16 already
    g = np.float32(divisor)
    q, sf = nv_pack(H, x.to(H.DEVICE), torch.tensor([g], dtype=torch.float32, device=H.DEVICE))
    want_q, _, want_sf = OB.pack_nvfp4(vals, g)
    assert np.array_equal(sf.cpu().numpy(), want_sf)
    assert np.array_equal(q.cpu().numpy(), want_q)


def test_nvfp4_with_per_tensor_scales(H):
    """The benchmark's variant: fp32 per-tensor scale amax / (6 * 448) on both operands."""
    m, n, k = 64, 256, 512
    x, w = H.randn_bf16((m, k), 30.0, 16), H.randn_bf16((n, k), 0.0004, 17)  # ranges a bare UE4M3 scale handles badly
    xd, wd = x.to(H.DEVICE), w.to(H.DEVICE)
    ws = _lib.gemm_workspace(_lib.OP_NVFP4, H.DEVICE, m, n, k)
    ga = torch.zeros(1, device=H.DEVICE)
    gb = torch.zeros(1, device=H.DEVICE)
    H.call("rk_nvfp4_global_scale", _lib.ptr(xd), xd.numel(), _lib.ptr(ga), _lib.ptr(ws), ws.numel(), H.stream())
    H.call("rk_nvfp4_global_scale", _lib.ptr(wd), wd.numel(), _lib.ptr(gb), _lib.ptr(ws), ws.numel(), H.stream())
    ega = OF.tensor_scale(H.to_np(x), np.float32(6.0 * 448.0))
    egb = OF.tensor_scale(H.to_np(w), np.float32(6.0 * 448.0))
    assert ga.item() == ega and gb.item() == egb
    qa, sfa = nv_pack(H, xd, ga)
    qb, sfb = nv_pack(H, wd, gb)
    pa, sa, swa = OB.pack_nvfp4(H.to_np(x), ega)
    pb, sb, swb = OB.pack_nvfp4(H.to_np(w), egb)
    assert np.array_equal(qa.cpu().numpy(), pa) and np.array_equal(sfa.cpu().numpy(), swa)
    assert np.array_equal(qb.cpu().numpy(), pb) and np.array_equal(sfb.cpu().numpy(), swb)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=H.DEVICE)
    H.call("rk_gemm_nvfp4", _lib.ptr(qa), _lib.ptr(sfa), _lib.ptr(ga), _lib.ptr(qb), _lib.ptr(sfb), _lib.ptr(gb), None,
           _lib.ptr(out), m, n, k, 0, _lib.ptr(ws), ws.numel(), H.stream())
    assert _lib.read_status(ws) == 0
    _, want = OB.gemm_dequantized(OB.dequant_nvfp4(pa, sa, ega), OB.dequant_nvfp4(pb, sb, egb))
    assert H.rel_frobenius(H.to_np(out), want) < TOL
