"""GPU parity of the fused producers in front of the FP8 and NVFP4 GEMMs: (residual add +) RMSNorm and
SwiGLU feeding the per-tensor E4M3 quantizer and the NVFP4 packer, checked against the CPU oracle.

The norm and the SiLU contain one transcendental each (`rsqrt`, `exp`) whose device versions are
not correctly rounded; every result is rounded to bf16 right after, so device and oracle agree
except where a value sits on a bf16 rounding boundary.  The tests therefore demand bit equality of
the bf16 intermediates on (almost) all elements, a two-step bound on the rest, and bit equality of
the codes and scale factors with what the oracle makes of the kernel's own bf16 intermediates."""

import numpy as np
import pytest
import torch

from oracle import blockscale as OB
from oracle import formats as F
from oracle import fp8 as OF
from rk_b200 import _lib

pytestmark = pytest.mark.gpu
EPS = 1e-6


@pytest.fixture(scope="module")
def H():
    import gpu_helpers

    return gpu_helpers


def _nearly_identical(got, want, max_fraction=2e-3):
    """bf16 arrays: equal almost everywhere, never further apart than two bf16 steps (a one-step
    difference after the first of two consecutive roundings can double in the second)."""
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    differ = got != want
    assert differ.mean() <= max_fraction
    assert np.all(np.abs(got - want)[differ] <= np.abs(want)[differ] * 2.0 ** -6 + 1e-30)
    return ~differ.reshape(got.shape[0], -1).any(axis=1)  # rows that agree exactly


@pytest.mark.parametrize("shape", [(5, 64), (100, 1024), (816, 2048)])
@pytest.mark.parametrize("with_residual", [True, False])
def test_rmsnorm_to_per_tensor_fp8(H, shape, with_residual):
    from rk_b200.fp8_linear import add_rms_norm_quantize_bf16

    rows, k = shape
    x = H.randn_bf16(shape, 1.0, 21)
    res = H.randn_bf16(shape, 0.5, 22) if with_residual else None
    w = (H.randn_bf16((k,), 0.1, 23).float() + 1.0).to(torch.bfloat16)
    summed, normalized, q, scale = add_rms_norm_quantize_bf16(
        x.to(H.DEVICE), None if res is None else res.to(H.DEVICE), w.to(H.DEVICE), EPS)
    ws, wn, wq, wscale = OF.add_rms_norm_quantize(H.to_np(x), None if res is None else H.to_np(res), H.to_np(w), EPS)
    assert np.array_equal(F.bf16_bits(H.to_np(summed)), F.bf16_bits(ws))  # the residual add is exact arithmetic
    _nearly_identical(H.to_np(normalized), wn)
    # scale and codes follow from the kernel's own normalized values exactly
    own_codes, own_scale = OF.quantize(H.to_np(normalized))
    assert np.float32(scale.item()) == own_scale
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), own_codes)
    assert abs(float(scale.item()) - float(wscale)) <= float(wscale) * 2.0 ** -7


@pytest.mark.parametrize("shape", [(3, 64), (50, 4096), (816, 16384)])
def test_swiglu_to_per_tensor_fp8(H, shape):
    from rk_b200.fp8_linear import quantize_swiglu_bf16, quantize_swiglu_bf16_with_scale

    rows, inter = shape
    gate_up = H.randn_bf16((rows, 2 * inter), 1.5, 31)
    q, scale = quantize_swiglu_bf16(gate_up.to(H.DEVICE), inter)
    wq, wscale, act = OF.quantize_swiglu(H.to_np(gate_up), inter)
    got = q.view(torch.uint8).cpu().numpy()
    # the activation itself is not an output; compare through the codes: identical scale (the maximum is
    # far from a rounding boundary with overwhelming probability) and codes equal almost everywhere
    assert abs(float(scale.item()) - float(wscale)) <= float(wscale) * 2.0 ** -7
    if np.float32(scale.item()) == wscale:
        differ = got != wq
        assert differ.mean() <= 2e-3
        step = np.abs(F.e4m3_decode(got).astype(np.float64) - F.e4m3_decode(wq).astype(np.float64))
        assert np.all(step[differ] <= np.abs(F.e4m3_decode(wq))[differ] * 0.13 + 2.0 ** -9)
    # a caller-supplied scale reproduces the same codes
    again = quantize_swiglu_bf16_with_scale(gate_up.to(H.DEVICE), inter, scale)
    assert torch.equal(again.view(torch.uint8), q.view(torch.uint8))


@pytest.mark.parametrize("shape", [(5, 64), (130, 1024), (816, 2048)])
@pytest.mark.parametrize("with_residual", [True, False])
def test_rmsnorm_to_nvfp4(H, shape, with_residual):
    from rk_b200.fp4_linear import add_rms_norm_fp4_quant_bf16

    rows, k = shape
    x = H.randn_bf16(shape, 1.0, 41)
    res = H.randn_bf16(shape, 0.5, 42) if with_residual else None
    w = (H.randn_bf16((k,), 0.1, 43).float() + 1.0).to(torch.bfloat16)
    summed, normalized, q, sf = add_rms_norm_fp4_quant_bf16(
        x.to(H.DEVICE), None if res is None else res.to(H.DEVICE), w.to(H.DEVICE), EPS)
    ws, wn, wq, wsf, wsf_swizzled = OB.rms_norm_pack_nvfp4(H.to_np(x), None if res is None else H.to_np(res), H.to_np(w), EPS)
    assert np.array_equal(F.bf16_bits(H.to_np(summed)), F.bf16_bits(ws))
    _nearly_identical(H.to_np(normalized), wn)
    # codes and scale factors are exactly what the packer makes of the kernel's own normalized values,
    # padding bytes included
    own_q, own_sf, own_swizzled = OB.pack_nvfp4(H.to_np(normalized))
    assert np.array_equal(q.cpu().numpy(), own_q)
    assert np.array_equal(sf.cpu().numpy(), own_swizzled)


@pytest.mark.parametrize("shape", [(3, 64), (50, 4096), (300, 16384)])
def test_swiglu_to_nvfp4(H, shape):
    from rk_b200.fp4_linear import pack_swiglu_nvfp4

    rows, inter = shape
    gate_up = H.randn_bf16((rows, 2 * inter), 1.5, 51)
    q, sf = pack_swiglu_nvfp4(gate_up.to(H.DEVICE), inter)
    wq, wsf, wswizzled, act = OB.swiglu_pack_nvfp4(H.to_np(gate_up), inter)
    got_q, got_sf = q.cpu().numpy(), OB.unswizzle_sf(sf.cpu().numpy(), rows, inter // 16)
    # a 16-element block is identical unless one of its activations sat on a bf16 rounding boundary
    same_block = (got_sf == wsf) & (got_q.reshape(rows, inter // 16, 8) == wq.reshape(rows, inter // 16, 8)).all(axis=2)
    assert same_block.mean() >= 0.98
    # and the dequantized tensor stays close everywhere
    got_deq = OB.dequant_nvfp4(got_q, got_sf)
    assert H.rel_frobenius(got_deq, OB.dequant_nvfp4(wq, wsf)) < 2e-2
    # padding of the scale-factor buffer is zero
    full = sf.cpu().numpy().copy()
    full[OB.sf_offsets(rows, inter // 16)] = 0
    assert not full.any()


def test_swiglu_modules_end_to_end(H):
    """forward_swiglu of the FP8 and NVFP4 layers against SiLU * up followed by the plain forward."""
    from rk_b200.fp4_linear import Fp4CutlassLinear
    from rk_b200.fp8_linear import Fp8CutlassLinear

    torch.manual_seed(5)
    inter, width = 512, 256
    lin = torch.nn.Linear(inter, width, bias=False, device="cuda", dtype=torch.bfloat16).eval().requires_grad_(False)
    gate_up = torch.randn(4, 7, 2 * inter, device="cuda", dtype=torch.bfloat16)
    reference = torch.nn.functional.silu(gate_up[..., :inter].float()) * gate_up[..., inter:].float()
    want = (reference @ lin.weight.float().T).cpu().numpy()
    for layer in (Fp8CutlassLinear.from_linear(lin, "linear", "down"), Fp4CutlassLinear.from_linear(lin, "linear", "down")):
        if isinstance(layer, Fp8CutlassLinear):
            got = layer.forward_swiglu(gate_up, inter, gate_up.shape[:-1])
            tol = 0.05
        else:
            got = layer.forward_swiglu(gate_up, inter)
            tol = 0.15  # four-bit operands on both sides
        assert got.shape == (4, 7, width)
        assert H.rel_frobenius(H.to_np(got).reshape(-1, width), want.reshape(-1, width)) < tol
    # the interleaved gate/up layout (64 up columns, then their 64 gate columns) gives the same result
    blocks = torch.stack([gate_up[..., inter:].reshape(4, 7, inter // 64, 64), gate_up[..., :inter].reshape(4, 7, inter // 64, 64)],
                         dim=3)
    layer = Fp4CutlassLinear.from_linear(lin, "linear", "down")
    assert torch.equal(layer.forward_swiglu(blocks.reshape(4, 7, 2 * inter).contiguous(), inter, interleaved=True),
                       layer.forward_swiglu(gate_up, inter))


def test_fp8_producer_path_uses_a_unit_activation_scale(H):
    """`forward_producer`: activations go to E4M3 unscaled (saturating at 448), weights keep their scale."""
    from rk_b200.fp8_linear import Fp8CutlassLinear

    torch.manual_seed(9)
    lin = torch.nn.Linear(512, 256, bias=True, device="cuda", dtype=torch.bfloat16).eval().requires_grad_(False)
    x = torch.randn(3, 40, 512, device="cuda", dtype=torch.bfloat16) * 2
    x[0, 0, 0] = 1000.0  # saturates to 448
    layer = Fp8CutlassLinear.from_linear(lin, "linear", "k_proj")
    got = H.to_np(layer.forward_producer(x)).reshape(-1, 256)
    xa = OF.quantize_with_scale(H.to_np(x).reshape(-1, 512), np.float32(1.0))
    wb, ws = OF.quantize(H.to_np(lin.weight))
    want, _ = OF.gemm(xa, np.float32(1.0), wb, ws, H.to_np(lin.bias))
    assert H.rel_frobenius(got, want) < 1e-2
    assert F.e4m3_decode(xa)[0, 0] == 448.0


# ---------------------------------------------------------------- SwiGLU + NVFP4 re-pack inside the gate/up GEMM
@pytest.mark.parametrize("shape", [(130, 256, 256), (816, 1024, 512), (300, 384, 2048), (816, 4096, 2048)])
def test_gate_up_gemm_with_fused_swiglu_repack_equals_the_two_launch_path(H, shape):
    """`rk_gemm_nvfp4_swiglu` (interleaved gate/up weight rows, SwiGLU and the NVFP4 block pack in the
    GEMM's epilogue) against GEMM -> bf16 [M, 2 * inter] -> `rk_swiglu_pack_nvfp4_layout(interleaved)`:
    the fused kernel follows the same arithmetic step for step, so codes and scale factors are equal
    bit for bit; the two-launch path itself is held to the reference's kernels by the golden fixtures."""
    from rk_b200 import fp4_linear as P4

    m, inter, k = shape
    x = H.randn_bf16((m, k), 1.0, 101).to(H.DEVICE)
    w = H.randn_bf16((2 * inter, k), 0.05, 102).to(H.DEVICE)  # [gate | up] along the output channels
    wi = P4.interleave_gate_up_rows(w, inter)
    assert torch.equal(wi[:64], w[inter:inter + 64]) and torch.equal(wi[64:128], w[:64])
    qa, sfa = P4.pack_nvfp4(x)
    qb, sfb = P4.pack_nvfp4(wi)
    two = P4.linear_forward_packed_gemm_bf16(qa, sfa, None, qb, sfb, None, None, k)  # interleaved columns
    q2, sf2 = P4.pack_swiglu_nvfp4(two, inter, interleaved=True)
    q1, sf1 = P4.linear_swiglu_packed_gemm(qa, sfa, None, qb, sfb, None, k)
    ws = _lib.gemm_workspace(_lib.OP_NVFP4, H.DEVICE, m, 2 * inter, k)
    assert _lib.read_status(ws) == 0
    assert torch.equal(q1, q2)
    assert torch.equal(sf1, sf2)
    # and with the fp32 per-tensor scales on both operands (alpha = ga * gb in front of the rounding)
    ga, gb = P4.tensor_global_scale(x), P4.tensor_global_scale(wi)
    qa, sfa = P4.pack_nvfp4(x, ga)
    qb, sfb = P4.pack_nvfp4(wi, gb)
    two = P4.linear_forward_packed_gemm_bf16(qa, sfa, ga, qb, sfb, gb, None, k)
    q2, sf2 = P4.pack_swiglu_nvfp4(two, inter, interleaved=True)
    q1, sf1 = P4.linear_swiglu_packed_gemm(qa, sfa, ga, qb, sfb, gb, k)
    assert torch.equal(q1, q2) and torch.equal(sf1, sf2)


def test_fused_swiglu_gemm_rejects_bad_shapes(H):
    from rk_b200 import fp4_linear as P4

    x = H.randn_bf16((64, 128), 1.0, 103).to(H.DEVICE)
    w = H.randn_bf16((192, 128), 0.05, 104).to(H.DEVICE)  # 2 * inter = 192: not a multiple of 128
    qa, sfa = P4.pack_nvfp4(x)
    qb, sfb = P4.pack_nvfp4(w)
    with pytest.raises(ValueError):
        P4.linear_swiglu_packed_gemm(qa, sfa, None, qb, sfb, None, 128)
    with pytest.raises(ValueError):
        P4.interleave_gate_up_rows(w, 96)


def test_gate_up_swiglu_module_feeds_the_down_projection(H):
    from rk_b200 import fp4_linear as P4

    m, inter, k = 200, 512, 256
    gate = torch.nn.Linear(k, inter, bias=False, dtype=torch.bfloat16)
    up = torch.nn.Linear(k, inter, bias=False, dtype=torch.bfloat16)
    down = torch.nn.Linear(inter, k, bias=False, dtype=torch.bfloat16)
    with torch.no_grad():
        gate.weight.copy_(H.randn_bf16((inter, k), 0.05, 111))
        up.weight.copy_(H.randn_bf16((inter, k), 0.05, 112))
        down.weight.copy_(H.randn_bf16((k, inter), 0.05, 113))
    gate, up, down = (l.to(H.DEVICE).requires_grad_(False) for l in (gate, up, down))
    x = H.randn_bf16((2, m // 2, k), 1.0, 114).to(H.DEVICE)
    fused = P4.Fp4GateUpSwiglu.from_linears(gate, up)
    down_q = P4.Fp4CutlassLinear.from_linear(down, "linear", "down")
    q, sf = fused(x)
    got = down_q.forward_packed(q, sf, None, x.shape[:-1])
    # the same MLP with separate launches: NVFP4 gate and up linears, bf16 [gate | up], SwiGLU pack, down
    gate_q = P4.Fp4CutlassLinear.from_linear(gate, "linear", "gate")
    up_q = P4.Fp4CutlassLinear.from_linear(up, "linear", "up")
    want = down_q.forward_swiglu(torch.cat([gate_q(x), up_q(x)], dim=-1), inter)
    assert torch.equal(got, want)
    # and close to the bf16 MLP
    ref = torch.nn.functional.silu(gate(x).float()) * up(x).float()
    ref = (ref.to(torch.bfloat16) @ down.weight.t()).float()
    assert float((got.float() - ref).norm() / ref.norm()) < 0.35  # two chained 4-bit GEMMs



@pytest.mark.parametrize("interleaved", [False, True])
def test_silu_mul_bf16_equals_the_packers_producer(H, interleaved):
    """`silu_mul_bf16` on its own: the oracle's bf16-step SwiGLU, and exactly the values the NVFP4 SwiGLU
    packer quantizes (packing this output gives the fused packer's bytes)."""
    from oracle import blockscale as OB
    from rk_b200 import fp4_linear as P4

    rows, inter = 70, 192
    gate_up = (H.randn_bf16((2, rows // 2, 2 * inter), 2.0, 41)).to(H.DEVICE)
    out = P4.cutlass_silu_mul_bf16(gate_up, inter, interleaved)
    assert out.shape == (2, rows // 2, inter)
    flat = H.to_np(gate_up).reshape(rows, 2 * inter)
    plain = OB.deinterleave_gate_up(flat, inter) if interleaved else flat
    # the device's exp and reciprocal round a few values the other way at a bf16 boundary (as in the packer tests)
    _nearly_identical(H.to_np(out).reshape(rows, inter), OB.swiglu_bf16_steps(plain, inter), 1e-2)
    q, sf = P4.pack_nvfp4(out.reshape(rows, inter))
    q2, sf2 = P4.pack_swiglu_nvfp4(gate_up.reshape(rows, 2 * inter), inter, interleaved)
    assert torch.equal(q, q2) and torch.equal(sf, sf2)
    with pytest.raises(ValueError):
        P4.cutlass_silu_mul_bf16(gate_up, inter + 8)
    with pytest.raises(ValueError):
        P4.cutlass_silu_mul_bf16(gate_up[..., :200].contiguous(), 100, True)


@pytest.mark.parametrize("with_residual", [False, True])
def test_rms_norm_bf16_equals_the_producers_norm(H, with_residual):
    """The plain norm: the sum is exact; the normalized tensor is the one the FP8 / NVFP4 norm producers write."""
    from oracle import fp8 as OF
    from rk_b200 import fp4_linear as P4

    rows, k = 45, 1024
    x, res = H.randn_bf16((rows, k), 1.0, 51).to(H.DEVICE), H.randn_bf16((rows, k), 1.0, 52).to(H.DEVICE)
    w = (1.0 + 0.1 * H.randn_bf16((k,), 1.0, 53).float()).to(torch.bfloat16).to(H.DEVICE)
    if with_residual:
        summed, normed = P4.add_rms_norm_bf16(x, res, w, 1e-6)
        want_sum, want = OF.rms_norm(H.to_np(x), H.to_np(res), H.to_np(w), 1e-6)
        assert np.array_equal(H.to_np(summed), want_sum)
        ref_sum, ref_norm, _, _ = P4.add_rms_norm_fp4_quant_bf16(x, res, w, 1e-6)
        assert torch.equal(summed, ref_sum)
    else:
        normed = P4.rms_norm_bf16(x, w, 1e-6)
        _, want = OF.rms_norm(H.to_np(x), None, H.to_np(w), 1e-6)
        _, ref_norm, _, _ = P4.add_rms_norm_fp4_quant_bf16(x, None, w, 1e-6)
    assert torch.equal(normed, ref_norm)
    got = H.to_np(normed)
    assert np.abs(got - want).max() <= 2.0 ** -7 * np.abs(want).max()  # summation order of mean(x^2)
    with pytest.raises(ValueError):
        P4.rms_norm_bf16(x[:, :40].contiguous(), w[:40], 1e-6)


@pytest.mark.parametrize("shape", [(300, 512, 256), (816, 1024, 2048), (100, 256, 96)])
def test_mxfp8_gemm_with_swiglu_epilogue_equals_the_two_launches(H, shape):
    """`rk_gemm_mxfp8_swiglu`: the gate/up GEMM whose epilogue applies the table-SiLU SwiGLU producer and packs to
    MXFP8 gives the bytes of `mxfp8_linear` -> bf16 -> `silu_mul_pack_mxfp8` (the accumulators are the same; the
    [M, 2 * inter] bf16 tensor is never written)."""
    from rk_b200 import fp8_linear as P8
    from rk_b200 import mxfp8_swiglu as MS
    from rk_b200.cute_mxfp8_swiglu import cutlass_swiglu_mxfp8_packed
    from rk_b200.fp4_linear import interleave_gate_up_rows

    m, n, k = shape
    inter = n // 2
    x = H.randn_bf16((m, k), 1.0, 91).to(H.DEVICE)
    w = H.randn_bf16((n, k), 0.05, 92).to(H.DEVICE)  # rows: gate (inter), then up (inter)
    table = MS.make_bf16_silu_table(H.DEVICE)
    a, sfa = P8.mxfp8_pack(x)
    b, sfb = P8.mxfp8_pack(w)
    gate_up = P8.mxfp8_linear(a, sfa, b, sfb)
    want_q, want_sf = MS.silu_mul_pack_mxfp8(gate_up, inter, table)
    bi, sfbi = P8.mxfp8_pack(interleave_gate_up_rows(w, inter))
    q, sf = cutlass_swiglu_mxfp8_packed(a, sfa, bi, sfbi, table)
    assert q.shape == (m, inter)
    assert torch.equal(q.view(torch.uint8), want_q.view(torch.uint8))
    assert torch.equal(sf, want_sf)
    q2, sf2 = cutlass_swiglu_mxfp8_packed(a, sfa, bi, sfbi)  # the table built on demand is the same one
    assert torch.equal(q2.view(torch.uint8), want_q.view(torch.uint8)) and torch.equal(sf2, want_sf)


def test_mxfp8_swiglu_gemm_refuses_bad_shapes(H):
    from rk_b200 import fp8_linear as P8
    from rk_b200 import mxfp8_swiglu as MS

    a, sfa = P8.mxfp8_pack(H.randn_bf16((64, 128), 1.0, 1).to(H.DEVICE))
    b, sfb = P8.mxfp8_pack(H.randn_bf16((384, 128), 1.0, 2).to(H.DEVICE))  # 384 % 256 != 0
    with pytest.raises(ValueError):
        MS.cutlass_swiglu_mxfp8_packed(a, sfa, b, sfb)
    with pytest.raises(TypeError):
        MS.cutlass_swiglu_mxfp8_packed(a.view(torch.uint8), sfa, b, sfb)


@pytest.mark.parametrize("global_scale", [True, False])
@pytest.mark.parametrize("shape", [(300, 256, 256), (816, 1024, 2048), (70, 128, 192)])
def test_nvfp4_gate_up_gemm_with_gelu_epilogue_equals_the_two_launches(H, shape, global_scale):
    """`rk_gemm_nvfp4_gated_act`: the fused gate/up GEMM writes GELU(gate) * up and the tensor's scale exactly as
    the plain GEMM on the same interleaved weight followed by `rk_lut_mul_tensor_scale` does."""
    from rk_b200 import fp4_linear as P4
    from rk_b200.integer import prepare_gelu

    m, inter, k = shape
    torch.manual_seed(7)
    gate = torch.nn.Linear(k, inter, bias=False, device=H.DEVICE, dtype=torch.bfloat16)
    up = torch.nn.Linear(k, inter, bias=False, device=H.DEVICE, dtype=torch.bfloat16)
    fused = P4.Fp4GateUpGelu.from_linears(gate, up, global_scale=global_scale)
    x = (H.randn_bf16((m, k), 1.0, 17) * 3).to(torch.bfloat16).to(H.DEVICE)
    q, sf, ga = fused.pack_input(x)
    y = P4.linear_forward_packed_gemm_bf16(q, sf, ga, fused.packed_weight, fused.weight_scale, fused.weight_global_scale, None, k)
    blocks = y.view(m, inter // 64, 2, 64)  # of every 128 columns: 64 up values, then their 64 gate values
    up_y, gate_y = blocks[:, :, 0, :].reshape(m, inter), blocks[:, :, 1, :].reshape(m, inter)
    table = prepare_gelu(x.device, torch.bfloat16, "tanh")
    want, want_scale = P4.table_mul_tensor_scale(gate_y, up_y, table, 6.0 * 448.0 if global_scale else None)
    got, got_scale = fused(x)
    assert got.shape == (m, inter) and torch.equal(got, want)
    assert torch.equal(want, torch.nn.functional.gelu(gate_y, approximate="tanh") * up_y)
    if global_scale:
        assert got_scale.item() == want_scale.item()
        again, scale_again = fused(x)  # the staging word is clear again
        assert torch.equal(again, want) and scale_again.item() == want_scale.item()
    else:
        assert got_scale is None
    # the whole MLP through the down projection
    down = P4.Fp4CutlassLinear.from_linear(torch.nn.Linear(inter, 264, bias=False, device=H.DEVICE, dtype=torch.bfloat16), "linear",
                                           "down", global_scale=global_scale)
    out = fused.forward_into(down, x.reshape(1, m, k))
    assert out.shape == (1, m, 264) and torch.equal(out.reshape(m, 264), down(want))
