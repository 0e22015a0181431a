"""GPU tests of the remaining operator surface: AdaLN / LayerNorm / RMSNorm fused packs, the
FP8 / MXFP8 / NVFP4 Linear modules, module swapping with quantize_linears, CudaGraphCall."""

import numpy as np
import pytest
import torch

from conftest import bf16_from_bits
from oracle import blockscale as OB
from oracle import formats as F
from oracle import fp8 as OF
from oracle import integer as OI

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def H():
    import gpu_helpers

    return gpu_helpers


def _t(a, H):
    return torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).to(H.DEVICE)


def _codes(data, bits):
    a = data.cpu().numpy()
    return a.view(np.int8).astype(np.int32) if bits == 8 else OI.unpack_nibbles(a).astype(np.int32)


# ---------------------------------------------------------------- AdaLN modulation packs
@pytest.mark.parametrize("case", range(2))
@pytest.mark.parametrize("bits", [8, 4])
def test_modulation_pack_matches_reference_fixture(H, golden, case, bits):
    from rk_b200.modulation import prepare_modulation

    x = _t(bf16_from_bits(golden[f"mod{case}_x"]), H)
    scale = _t(bf16_from_bits(golden[f"mod{case}_scale"]), H)
    shift = _t(bf16_from_bits(golden[f"mod{case}_shift"]), H)
    packed = prepare_modulation(x, scale, shift, bits)
    assert np.array_equal(packed.scales.cpu().numpy(), golden[f"mod{case}_b{bits}_plain_s"])
    assert np.array_equal(packed.data.cpu().numpy().view(np.uint8), golden[f"mod{case}_b{bits}_plain_q"])
    assert packed.shape == tuple(x.shape[:2]) and packed.logical_k == x.shape[2]


@pytest.mark.parametrize("case", range(2))
@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("variant", ["norm", "residual"])
def test_layernorm_modulation_pack_close_to_reference_fixture(H, golden, case, bits, variant):
    """Same tolerances as the reference's own LayerNorm-pack test: scales rtol 0.008, codes off by
    at most one in a small fraction of positions; the residual output is exact."""
    from rk_b200.modulation import prepare_norm_modulation, prepare_residual_norm_modulation

    x = _t(bf16_from_bits(golden[f"mod{case}_x"]), H)
    scale = _t(bf16_from_bits(golden[f"mod{case}_scale"]), H)
    shift = _t(bf16_from_bits(golden[f"mod{case}_shift"]), H)
    tag = f"mod{case}_b{bits}_{variant}"
    if variant == "norm":
        packed = prepare_norm_modulation(x, scale, shift, bits, eps=1e-6)
    else:
        y = _t(bf16_from_bits(golden[f"mod{case}_y"]), H)
        gate = _t(bf16_from_bits(golden[f"mod{case}_gate"]), H)
        residual, packed = prepare_residual_norm_modulation(x, y, gate, scale, shift, bits, eps=1e-6)
        assert np.array_equal(H.bits(residual), golden[tag + "_residual"])
    np.testing.assert_allclose(packed.scales.cpu().numpy(), golden[tag + "_s"], rtol=0.008)
    want = golden[tag + "_q"]
    want = want.view(np.int8).astype(np.int32) if bits == 8 else OI.unpack_nibbles(want).astype(np.int32)
    diff = np.abs(_codes(packed.data, bits) - want)
    assert diff.max() <= 1 and (diff != 0).mean() <= 0.01


def test_modulation_pack_at_cosmos_size_matches_oracle(H):
    from rk_b200.modulation import prepare_modulation

    b, tokens, k = 2, 882, 2048
    x = H.randn_bf16((b, tokens, k), 1.0, 1)
    scale = H.randn_bf16((b, 1, k), 0.3, 2)
    shift = H.randn_bf16((b, 1, k), 0.3, 3)
    packed = prepare_modulation(x.to(H.DEVICE), scale.to(H.DEVICE), shift.to(H.DEVICE), 8)
    data, s, _ = OI.prepare_modulation(H.to_np(x).reshape(-1, k), H.to_np(scale).reshape(b, k),
                                       H.to_np(shift).reshape(b, k), tokens, 8)
    assert np.array_equal(packed.scales.cpu().numpy(), s)
    assert np.array_equal(packed.data.cpu().numpy(), data)


def test_packed_activations_carrier_feeds_integer_linear(H):
    from rk_b200.integer import IntegerLinear
    from rk_b200.modulation import PackedActivations, prepare_modulation

    torch.manual_seed(5)
    lin = torch.nn.Linear(256, 64, bias=False, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(2, 7, 256, device="cuda", dtype=torch.bfloat16)
    scale = torch.randn(2, 1, 256, device="cuda", dtype=torch.bfloat16) * 0.2
    shift = torch.randn(2, 1, 256, device="cuda", dtype=torch.bfloat16) * 0.2
    carrier = PackedActivations({8: prepare_modulation(x, scale, shift, 8), 4: prepare_modulation(x, scale, shift, 4)})
    modulated = ((x.float() * (1 + scale.float()).to(torch.bfloat16).float()).to(torch.bfloat16).float()
                 + shift.float()).to(torch.bfloat16)
    for bits in (8, 4):
        layer = IntegerLinear.from_linear(lin, bits=bits)
        assert torch.equal(layer(carrier), layer(modulated))
    with pytest.raises(ValueError):
        PackedActivations({8: carrier.packs[8]}).for_bits(4)
    with pytest.raises(ValueError):
        carrier.with_leading_shape((3, 5))
    assert carrier.with_leading_shape((14,)).for_bits(8).shape == (14,)


# ---------------------------------------------------------------- Gemma RMSNorm -> pack
def _rmsnorm_oracle(x, w, eps, residual=None, shift=None, rows_per=None, gate=None):
    if gate is not None:  # gated residual (common/fused.py:47-58): bf16(x + bf16(branch * gate))
        residual = F.bf16_round((residual * gate[np.arange(x.shape[0]) // rows_per]).astype(np.float32))
    s = x if residual is None else F.bf16_round((x + residual).astype(np.float32))
    var = (s.astype(np.float32) ** 2).mean(axis=1, dtype=np.float32)
    inv = (1.0 / np.sqrt(var + np.float32(eps))).astype(np.float32)
    a = w if rows_per is None else w[np.arange(x.shape[0]) // rows_per]
    t = ((s * inv[:, None]).astype(np.float32) * (np.float32(1.0) + a).astype(np.float32)).astype(np.float32)
    if shift is not None:
        t = (t + shift[np.arange(x.shape[0]) // rows_per]).astype(np.float32)
    return s, F.bf16_round(t)


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("adaptive", [False, True])
def test_rmsnorm_pack(H, bits, adaptive):
    from rk_b200.modulation import prepare_rmsnorm

    rows, k, tokens = 100, 1024, 50
    x = H.randn_bf16((rows, k), 1.0, 1)
    res = H.randn_bf16((rows, k), 1.0, 2)
    if adaptive:
        w, sh = H.randn_bf16((rows // tokens, k), 0.2, 3), H.randn_bf16((rows // tokens, k), 0.2, 4)
        packed, summed, normed = prepare_rmsnorm(x.to(H.DEVICE), w.to(H.DEVICE), bits, eps=1e-6,
                                                 residual=res.to(H.DEVICE), shift=sh.to(H.DEVICE), tokens=tokens,
                                                 return_sum=True, return_normed=True)
        s, n = _rmsnorm_oracle(H.to_np(x), H.to_np(w), 1e-6, H.to_np(res), H.to_np(sh), tokens)
    else:
        w = H.randn_bf16((k,), 0.2, 3)
        packed, summed, normed = prepare_rmsnorm(x.to(H.DEVICE), w.to(H.DEVICE), bits, eps=1e-6,
                                                 residual=res.to(H.DEVICE), return_sum=True, return_normed=True)
        s, n = _rmsnorm_oracle(H.to_np(x), H.to_np(w)[None, :].repeat(rows, 0), 1e-6, H.to_np(res))
    assert np.array_equal(H.bits(summed), F.bf16_bits(s))  # the residual sum is exact
    # the reduction order of mean(s^2) differs from numpy's: normalized values within 1 bf16 ulp
    got_n = H.to_np(normed)
    assert np.abs(got_n - n).max() <= 2.0 ** -7 * np.abs(n).max()
    # the pack is exactly the row quantizer applied to the normalized tensor the kernel produced
    data, sc, _ = OI.quantize_rows(got_n, bits)
    p = packed.for_bits(bits)
    assert np.array_equal(p.scales.cpu().numpy(), sc)
    assert np.array_equal(p.data.cpu().numpy().view(np.uint8), data.view(np.uint8))


@pytest.mark.parametrize("bits", [8, 4])
def test_gated_residual_rmsnorm_pack(H, bits):
    """x + branch * gate (two bf16 roundings, the gated residual of the adaptive layers) in front of
    the adaptive RMSNorm and the row quantizer, one kernel: the new residual stream is exact, the
    pack is the row quantizer applied to the kernel's own normalized values."""
    from rk_b200.modulation import prepare_rmsnorm

    rows, k, tokens = 150, 1024, 50
    x, branch = H.randn_bf16((rows, k), 1.0, 11), H.randn_bf16((rows, k), 1.0, 12)
    w, sh = H.randn_bf16((rows // tokens, k), 0.2, 13), H.randn_bf16((rows // tokens, k), 0.2, 14)
    gate = H.randn_bf16((rows // tokens, k), 0.5, 15)
    packed, summed, normed = prepare_rmsnorm(x.to(H.DEVICE), w.to(H.DEVICE), bits, eps=1e-6, residual=branch.to(H.DEVICE),
                                             gate=gate.to(H.DEVICE), shift=sh.to(H.DEVICE), tokens=tokens,
                                             return_sum=True, return_normed=True)
    s, n = _rmsnorm_oracle(H.to_np(x), H.to_np(w), 1e-6, H.to_np(branch), H.to_np(sh), tokens, H.to_np(gate))
    assert np.array_equal(H.bits(summed), F.bf16_bits(s))
    want_sum = x.to(H.DEVICE) + branch.to(H.DEVICE) * gate.to(H.DEVICE).repeat_interleave(tokens, 0)
    assert torch.equal(summed, want_sum)  # the same two roundings as the tensor ops
    got_n = H.to_np(normed)
    assert np.abs(got_n - n).max() <= 2.0 ** -7 * np.abs(n).max()
    data, sc, _ = OI.quantize_rows(got_n, bits)
    p = packed.for_bits(bits)
    assert np.array_equal(p.scales.cpu().numpy(), sc)
    assert np.array_equal(p.data.cpu().numpy().view(np.uint8), data.view(np.uint8))
    with pytest.raises(ValueError):
        prepare_rmsnorm(x.to(H.DEVICE), w.to(H.DEVICE), bits, eps=1e-6, gate=gate.to(H.DEVICE), shift=sh.to(H.DEVICE),
                        tokens=tokens)  # a gate without a branch


@pytest.mark.parametrize("global_scale", [True, False])
@pytest.mark.parametrize("with_residual", [True, False])
def test_gemma_rmsnorm_pack_nvfp4(H, global_scale, with_residual):
    """(add +) Gemma RMSNorm + per-tensor amax in one kernel, then the block packer: the stream is
    exact, the normalized values within one bf16 ulp of the numpy restatement (reduction order), the
    scale and the pack exactly what the oracle makes of the kernel's own normalized values."""
    from oracle import blockscale as OB
    from rk_b200 import _lib
    from rk_b200.fp4_linear import gemma_rms_norm_pack_nvfp4, pack_nvfp4, tensor_global_scale

    rows, k = 3 * 67, 2048
    x = H.randn_bf16((3, 67, k), 1.0, 21)
    res = H.randn_bf16((3, 67, k), 1.0, 22) if with_residual else None
    w = H.randn_bf16((k,), 0.2, 23)
    carrier, stream = gemma_rms_norm_pack_nvfp4(x.to(H.DEVICE), w.to(H.DEVICE), 1e-6,
                                                residual=None if res is None else res.to(H.DEVICE),
                                                global_scale=global_scale)
    assert carrier.shape == (3, 67, k) and carrier.leading_shape == (3, 67)
    s, n = _rmsnorm_oracle(H.to_np(x).reshape(rows, k), H.to_np(w)[None, :].repeat(rows, 0), 1e-6,
                           None if res is None else H.to_np(res).reshape(rows, k))
    assert np.array_equal(H.bits(stream).reshape(rows, k), F.bf16_bits(s))
    # the normalized tensor the kernel produced, recovered through the unfused path on the same stream
    lib = _lib.load()
    normed = torch.empty((rows, k), dtype=torch.bfloat16, device=H.DEVICE)
    flat = stream.reshape(rows, k).contiguous()
    _lib.check(lib.rk_rmsnorm_tensor_scale(_lib.ptr(flat), None, _lib.ptr(w.to(H.DEVICE)), None, 0, rows, k, 1e-6, 1.0, None,
                                           _lib.ptr(normed), None, None, 0, _lib.stream_ptr(H.DEVICE)), "norm only")
    got_n = H.to_np(normed)
    assert np.abs(got_n - n).max() <= 2.0 ** -7 * np.abs(n).max()
    ga = OF.tensor_scale(got_n, np.float32(6.0 * 448.0)) if global_scale else None
    if global_scale:
        assert carrier.global_scale.item() == ga == tensor_global_scale(normed).item()
    else:
        assert carrier.global_scale is None
    pa, _, swa = OB.pack_nvfp4(got_n, ga)
    assert np.array_equal(carrier.codes.cpu().numpy(), pa) and np.array_equal(carrier.scale_factors.cpu().numpy(), swa)
    q, sf = pack_nvfp4(normed, carrier.global_scale)
    assert torch.equal(q, carrier.codes) and torch.equal(sf, carrier.scale_factors)


def test_gemma_rmsnorm_tensor_scale_ignores_non_finite_and_refuses_bad_arguments(H):
    from rk_b200 import _lib
    from rk_b200.fp4_linear import gemma_rms_norm_pack_nvfp4

    lib = _lib.load()
    k = 256
    x = H.randn_bf16((4, k), 1.0, 31).to(H.DEVICE)
    x[1, 7] = float("inf")  # that row normalizes to NaN / 0: neither may reach the scale
    w = torch.zeros(k, dtype=torch.bfloat16, device=H.DEVICE)
    normed = torch.empty_like(x)
    scale = torch.empty(1, dtype=torch.float32, device=H.DEVICE)
    ws = _lib.workspace(H.DEVICE, _lib.WORKSPACE_HEADER)
    args = lambda kk, div, wsb: (_lib.ptr(x), None, _lib.ptr(w), None, 0, 4, kk, 1e-6, div, None, _lib.ptr(normed),
                                 _lib.ptr(scale), _lib.ptr(ws), wsb, _lib.stream_ptr(H.DEVICE))
    _lib.check(lib.rk_rmsnorm_tensor_scale(*args(k, 448.0, ws.numel())), "scale")
    finite = normed.float()[torch.isfinite(normed.float())]
    assert scale.item() == np.float32(finite.abs().max().item()) / np.float32(448.0)
    assert lib.rk_rmsnorm_tensor_scale(*args(k, 0.0, ws.numel())) == _lib.RK_EINVAL
    assert lib.rk_rmsnorm_tensor_scale(*args(k, 448.0, 8)) == _lib.RK_EWORKSPACE
    assert lib.rk_rmsnorm_tensor_scale(*args(1 << 20, 448.0, ws.numel())) == _lib.RK_EUNSUPPORTED
    with pytest.raises(ValueError):
        gemma_rms_norm_pack_nvfp4(x[:, :40].contiguous(), w[:40], 1e-6)  # K % 32


def test_rmsnorm_tensor_scale_adaptive_mode_equals_the_quantizing_norm(H):
    """Adaptive weights (scale / shift rows per batch entry) and a residual through `rk_rmsnorm_tensor_scale`: the
    stream and the normalized tensor are bit for bit those of `rk_rmsnorm_quant_rows` (the same kernel body),
    and the scale is the maximum of that tensor over the divisor."""
    from rk_b200 import _lib
    from rk_b200.modulation import prepare_rmsnorm

    rows, k, tokens = 150, 1024, 50
    x, res = H.randn_bf16((rows, k), 1.0, 61).to(H.DEVICE), H.randn_bf16((rows, k), 1.0, 62).to(H.DEVICE)
    w, sh = H.randn_bf16((rows // tokens, k), 0.2, 63).to(H.DEVICE), H.randn_bf16((rows // tokens, k), 0.2, 64).to(H.DEVICE)
    _, want_sum, want_norm = prepare_rmsnorm(x, w, 8, eps=1e-6, residual=res, shift=sh, tokens=tokens, return_sum=True,
                                             return_normed=True)
    summed, normed = torch.empty_like(x), torch.empty_like(x)
    scale = torch.empty(1, dtype=torch.float32, device=H.DEVICE)
    ws = _lib.workspace(H.DEVICE, _lib.WORKSPACE_HEADER)
    _lib.check(_lib.load().rk_rmsnorm_tensor_scale(_lib.ptr(x), _lib.ptr(res), _lib.ptr(w), _lib.ptr(sh), tokens, rows, k, 1e-6, 448.0,
                                                   _lib.ptr(summed), _lib.ptr(normed), _lib.ptr(scale), _lib.ptr(ws), ws.numel(),
                                                   _lib.stream_ptr(H.DEVICE)), "adaptive norm + scale")
    assert torch.equal(summed, want_sum) and torch.equal(normed, want_norm)
    assert scale.item() == np.float32(normed.float().abs().max().item()) / np.float32(448.0)
    assert _lib.read_status(ws) == 0
    # the staging words are clear again: a second call gives the same scale
    _lib.check(_lib.load().rk_rmsnorm_tensor_scale(_lib.ptr(x), _lib.ptr(res), _lib.ptr(w), _lib.ptr(sh), tokens, rows, k, 1e-6, 448.0,
                                                   _lib.ptr(summed), _lib.ptr(normed), _lib.ptr(scale), _lib.ptr(ws), ws.numel(),
                                                   _lib.stream_ptr(H.DEVICE)), "second call")
    assert scale.item() == np.float32(normed.float().abs().max().item()) / np.float32(448.0)


@pytest.mark.parametrize("global_scale", [True, False])
def test_fp4_forward_gelu_equals_tensor_ops(H, global_scale):
    """`Fp4CutlassLinear.forward_gelu`: table GELU * up + amax in one kernel, packer, GEMM - the same
    bits as GELU and the product computed with tensor ops in front of `forward`; gate and up may be
    column slices of one wider matrix."""
    from rk_b200.fp4_linear import Fp4CutlassLinear, table_mul_tensor_scale
    from rk_b200.integer import prepare_gelu

    torch.manual_seed(5)
    lin = torch.nn.Linear(1024, 264, bias=False, device="cuda", dtype=torch.bfloat16)
    layer = Fp4CutlassLinear.from_linear(lin, role="linear", target_name="probe", global_scale=global_scale)
    both = torch.randn(2, 75, 2048, device="cuda", dtype=torch.bfloat16) * 2
    gate, up = both[..., :1024], both[..., 1024:]
    want = layer(torch.nn.functional.gelu(gate, approximate="tanh") * up)
    assert torch.equal(layer.forward_gelu(gate, up), want)
    assert torch.equal(layer.forward_gelu(gate.contiguous(), up.contiguous()), want)
    product, scale = table_mul_tensor_scale(gate, up, prepare_gelu(gate.device, gate.dtype, "tanh"), 448.0)
    eager = (torch.nn.functional.gelu(gate, approximate="tanh") * up).reshape(-1, 1024)
    assert torch.equal(product, eager)
    assert scale.item() == np.float32(eager.float().abs().max().item()) / np.float32(448.0)
    with pytest.raises(ValueError):
        table_mul_tensor_scale(gate[..., :1020], up[..., :1020], prepare_gelu(gate.device, gate.dtype, "tanh"))


# ---------------------------------------------------------------- FP8 / MXFP8 / NVFP4 modules
@pytest.mark.parametrize("mode", ["per_tensor", "mxfp8"])
def test_fp8_linear_module(H, mode):
    from rk_b200.fp8_linear import Fp8CutlassLinear, fp8_backend_status

    assert fp8_backend_status().available
    torch.manual_seed(1)
    lin = torch.nn.Linear(512, 264, device="cuda", dtype=torch.bfloat16)
    layer = Fp8CutlassLinear.from_linear(lin, role="linear", target_name="probe", mode=mode)
    x = torch.randn(3, 20, 512, device="cuda", dtype=torch.bfloat16)
    y = layer(x)
    assert y.shape == (3, 20, 264) and y.dtype == torch.bfloat16
    xn, wn, bn = H.to_np(x).reshape(60, 512), H.to_np(lin.weight), H.to_np(lin.bias)
    if mode == "per_tensor":
        ea, sa = OF.quantize(xn)
        eb, sb = OF.quantize(wn)
        _, want = OF.gemm(ea, sa, eb, sb, bn)
        assert np.array_equal(layer.packed_weight.view(torch.uint8).cpu().numpy(), eb)
    else:
        ca, sa, _ = OB.pack_mxfp8(xn)
        cb, sb, swb = OB.pack_mxfp8(wn)
        _, want = OB.gemm_dequantized(OB.dequant_mxfp8(ca, sa), OB.dequant_mxfp8(cb, sb), bn)
        assert np.array_equal(layer.weight_scale.cpu().numpy(), swb)
    assert H.rel_frobenius(H.to_np(y).reshape(60, 264), want) < 1e-2
    with pytest.raises(ValueError):
        layer(torch.zeros(2, 100, device="cuda", dtype=torch.bfloat16))


@pytest.mark.parametrize("global_scale", [False, True])
def test_fp4_linear_module(H, global_scale):
    from rk_b200.fp4_linear import Fp4CutlassLinear

    torch.manual_seed(2)
    lin = torch.nn.Linear(512, 264, bias=False, device="cuda", dtype=torch.bfloat16)
    layer = Fp4CutlassLinear.from_linear(lin, role="linear", target_name="probe", global_scale=global_scale)
    x = torch.randn(60, 512, device="cuda", dtype=torch.bfloat16)
    y = layer(x)
    xn, wn = H.to_np(x), H.to_np(lin.weight)
    ga = OF.tensor_scale(xn, np.float32(6 * 448)) if global_scale else None
    gb = OF.tensor_scale(wn, np.float32(6 * 448)) if global_scale else None
    pa, sa, _ = OB.pack_nvfp4(xn, ga)
    pb, sb, _ = OB.pack_nvfp4(wn, gb)
    assert np.array_equal(layer.packed_weight.cpu().numpy(), pb)
    _, want = OB.gemm_dequantized(OB.dequant_nvfp4(pa, sa, ga), OB.dequant_nvfp4(pb, sb, gb))
    assert H.rel_frobenius(H.to_np(y), want) < 1e-2


# ---------------------------------------------------------------- module swapping
class _Attention(torch.nn.Module):
    def __init__(self, width):
        super().__init__()
        self.q_proj = torch.nn.Linear(width, width, bias=False)
        self.k_proj = torch.nn.Linear(width, 64, bias=False)
        self.v_proj = torch.nn.Linear(width, 64, bias=False)

    def forward(self, x):
        return self.q_proj(x).sum(-1, keepdim=True) + self.k_proj(x).sum(-1, keepdim=True) + self.v_proj(x).sum(
            -1, keepdim=True)


class _Toy(torch.nn.Module):
    def __init__(self, width=256):
        super().__init__()
        self.blocks = torch.nn.ModuleList([_Attention(width) for _ in range(2)])
        self.head = torch.nn.Linear(width, 8).float()  # fp32: must be skipped

    def forward(self, x):
        return sum(b(x) for b in self.blocks)


@pytest.mark.parametrize("precision", ["int8", "int4", "fp8", "mxfp8", "fp4", "w4a16"])
def test_quantize_linears_swaps_and_restores(H, precision):
    from rk_b200.optimizations import quantize_linears

    torch.manual_seed(0)
    model = _Toy().to(device="cuda")
    for block in model.blocks:
        block.to(torch.bfloat16)
    x = torch.randn(5, 256, device="cuda", dtype=torch.bfloat16)
    originals = [block.q_proj for block in model.blocks]
    reference = model(x).float()
    selector = lambda name: "dit" if name.startswith("blocks.") else "text"  # noqa: E731
    with quantize_linears(model, precision, scopes=("dit",), selector=selector) as report:
        assert len(report["modules"]) == 6 and not report["skipped"]
        assert all(not isinstance(block.q_proj, torch.nn.Linear) for block in model.blocks)
        out = model(x).float()
        rel = (out - reference).norm() / reference.norm()
        assert rel < (0.05 if precision in ("int8", "fp8", "mxfp8") else 0.35)
    assert [block.q_proj for block in model.blocks] == originals
    assert torch.equal(model(x).float(), reference)


@pytest.mark.parametrize("options", [dict(shared_quant=True), dict(group_qkv=True), dict(grouped=True, group_views=True)])
def test_shared_and_grouped_integer_projections_are_exact(H, options):
    from rk_b200.optimizations import quantize_linears

    torch.manual_seed(0)
    model = _Toy().to(device="cuda")
    for block in model.blocks:
        block.to(torch.bfloat16)
    x = torch.randn(9, 256, device="cuda", dtype=torch.bfloat16)
    selector = lambda name: "dit" if name.startswith("blocks.") else None  # noqa: E731
    with quantize_linears(model, "int8", scopes=("dit",), selector=selector) as _:
        plain = model(x)
    with quantize_linears(model, "int8", scopes=("dit",), selector=selector, **options) as report:
        assert torch.equal(model(x), plain)
        if "shared_quant" not in options:
            assert len(report["grouped"]) == 2
    assert isinstance(model.blocks[0].q_proj, torch.nn.Linear)


# ---------------------------------------------------------------- CUDA graph helper
def test_cuda_graph_call_replays_and_recaptures(H):
    from rk_b200.graph import CudaGraphCall
    from rk_b200.integer import IntegerLinear

    torch.manual_seed(3)
    lin = torch.nn.Linear(512, 256, bias=False, device="cuda", dtype=torch.bfloat16)
    layer = IntegerLinear.from_linear(lin, bits=8)
    call = CudaGraphCall(lambda t: layer(t), retained_tensors=lambda: [layer.packed_weight])
    for shape in ((50, 512), (50, 512), (8, 512)):
        x = torch.randn(*shape, device="cuda", dtype=torch.bfloat16)
        assert torch.equal(call(x), layer(x))
    assert call.captures == 2 and call.replays == 3

    def broken(t):
        raise RuntimeError("capture failed")

    bad = CudaGraphCall(broken)
    with pytest.raises(RuntimeError):
        bad(torch.zeros(4, 4, device="cuda"))
    assert bad.graph is None and bad.captures == 0
    with pytest.raises(ValueError):
        call(torch.zeros(2, 512))  # CPU tensor
