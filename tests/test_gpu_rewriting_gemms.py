"""GPU parity of the GEMMs that rewrite an operand in shared memory before the MMA:

* W4A4 - both operands packed int4, widened to int8 inside the kernel (bit-exact int32 sums);
* the FP8 "producer" GEMM - bf16 activations converted to e4m3 with unit scale inside the kernel;
* W4A8 MX - MXFP4 weights expanded to e4m3 inside the kernel, MXFP8 activations, power-of-two scales;
* the interleaved gate/up layout of the SwiGLU -> NVFP4 packer.

Integer results are compared bit for bit; floating-point GEMMs against dequantize -> float64 matmul
of the oracle within the 1e-2 relative Frobenius bound of these operators; packers bit for bit."""

import numpy as np
import pytest
import torch

from oracle import blockscale as OB
from oracle import formats as F
from oracle import fp8 as OF
from oracle import integer as OI
from rk_b200 import _lib

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.fixture(scope="module")
def H():
    import gpu_helpers

    return gpu_helpers


# ---------------------------------------------------------------- W4A4 (int4 x int4 -> int32)
@pytest.mark.parametrize("shape", [(1, 40, 256), (50, 80, 256), (130, 264, 384), (512, 2048, 1024), (1764, 2048, 2048)])
@pytest.mark.parametrize("tactic", [0, 5])
def test_w4a4_unpacks_in_kernel_and_is_exact(H, shape, tactic):
    m, n, k = shape
    gen = torch.Generator().manual_seed(31)
    a = torch.randint(-8, 8, (m, k), generator=gen, dtype=torch.int8).numpy()
    b = torch.randint(-8, 8, (n, k), generator=gen, dtype=torch.int8).numpy()
    pa = torch.from_numpy(OI.pack_nibbles(a)).to(H.DEVICE)
    pb = torch.from_numpy(OI.pack_nibbles(b)).to(H.DEVICE)
    sa = (torch.rand(m, generator=gen) * 0.05 + 0.01).to(H.DEVICE)
    sb = (torch.rand(n, generator=gen) * 0.01 + 0.001).to(H.DEVICE)
    bias = (torch.randn(n, generator=gen) * 0.1).to(torch.bfloat16).to(H.DEVICE)
    # only the workspace header is needed: nothing is widened in global memory any more
    ws = torch.zeros(_lib.WORKSPACE_HEADER, dtype=torch.uint8, device=H.DEVICE)
    acc = torch.full((m, n), -1, dtype=torch.int32, device=H.DEVICE)
    H.call("rk_gemm_int_acc", _lib.ptr(pa), _lib.ptr(pb), _lib.ptr(acc), m, n, k, 4, tactic, _lib.ptr(ws), ws.numel(),
           H.stream())
    want_acc = OI.int_matmul(a, b)
    assert np.array_equal(acc.cpu().numpy(), want_acc)
    buf = torch.full((m + 2, n), 7.0, dtype=torch.bfloat16, device=H.DEVICE)
    out = buf[1:m + 1]
    H.call("rk_gemm_int", _lib.ptr(pa), _lib.ptr(sa), _lib.ptr(pb), _lib.ptr(sb), _lib.ptr(bias), _lib.ptr(out), m, n, k, 4,
           tactic, _lib.ptr(ws), ws.numel(), H.stream())
    assert _lib.read_status(ws) == 0
    assert (buf[0] == 7.0).all() and (buf[m + 1] == 7.0).all()
    want = OI.dequant_epilogue(want_acc, sa.cpu().numpy(), sb.cpu().numpy(), bias.float().cpu().numpy())
    assert np.array_equal(H.bits(out), F.bf16_bits(want))


# ---------------------------------------------------------------- FP8 producer GEMM
@pytest.mark.parametrize("shape", [(16, 128, 128), (100, 520, 448), (300, 264, 320), (816, 256, 2048), (816, 1280, 5120)])
def test_fp8_producer_gemm_converts_activations_in_kernel(H, shape):
    from rk_b200 import fp8_linear as P8

    m, n, k = shape
    x, w, bias = H.randn_bf16((m, k), 1.0, 41), H.randn_bf16((n, k), 0.02, 42), H.randn_bf16((n,), 0.01, 43)
    x[0, 0], x[0, 1] = 1000.0, -3000.0  # beyond +-448: clamped by the unit-scale conversion
    xd, wd, bd = x.to(H.DEVICE), w.to(H.DEVICE), bias.to(H.DEVICE)
    wq, wscale = P8.quantize_bf16(wd)
    out = P8.linear_forward_producer(xd, wq, wscale, bd)
    ws = _lib.gemm_workspace(_lib.OP_FP8, H.DEVICE, m, n, k)
    assert _lib.read_status(ws) == 0
    codes = OF.quantize_with_scale(H.to_np(x), np.float32(1.0))
    _, want = OF.gemm(codes, np.float32(1.0), wq.view(torch.uint8).cpu().numpy(), np.float32(wscale.item()), H.to_np(bias))
    assert H.rel_frobenius(H.to_np(out), want) < TOL
    # the two-launch form (conversion kernel, then the FP8 GEMM) computes the same product
    unit = torch.ones(1, device=H.DEVICE)
    two = P8.linear_forward_packed(P8.quantize_bf16_with_scale(xd, unit), unit, wq, wscale, bd)
    assert H.rel_frobenius(H.to_np(out), H.to_np(two)) < 1e-3


# ---------------------------------------------------------------- W4A8 MX
@pytest.mark.parametrize("shape", [(16, 128, 128), (100, 520, 448), (300, 264, 320), (816, 2048, 2048)])
def test_w4a8_mx_packers_and_gemm(H, shape):
    from rk_b200 import fp4_mx_linear as PM

    m, n, k = shape
    x, w, bias = H.randn_bf16((m, k), 1.0, 51), H.randn_bf16((n, k), 0.02, 52), H.randn_bf16((n,), 0.01, 53)
    x[0, :32] = 0                                   # a zero block: scale 1.0
    x[1, 0:3] = torch.tensor([448.0, 3.0, -896.0]).to(torch.bfloat16)  # amax / 448 = 2 exactly: a power of two
    w[0, 0:2] = torch.tensor([6.0, -0.75]).to(torch.bfloat16)          # amax / 6 = 1 exactly
    qa, sfa = PM.pack_mxfp8_activation(x.to(H.DEVICE))
    qb, sfb = PM.pack_mxfp4_weight(w.to(H.DEVICE))
    ca, sa, swa = OB.pack_mxfp8_ceil(H.to_np(x))
    pb, sb, swb = OB.pack_mxfp4_ceil(H.to_np(w))
    assert np.array_equal(sfa.cpu().numpy(), swa) and np.array_equal(sfb.cpu().numpy(), swb)
    assert np.array_equal(qa.view(torch.uint8).cpu().numpy(), ca) and np.array_equal(qb.cpu().numpy(), pb)
    out = PM.linear_w4a8_packed(qa, sfa, qb, sfb, bias.to(H.DEVICE))
    ws = _lib.gemm_workspace(_lib.OP_MXFP8, H.DEVICE, m, n, k)
    assert _lib.read_status(ws) == 0
    _, want = OB.gemm_dequantized(OB.dequant_mxfp8(ca, sa), OB.dequant_mxfp4(pb, sb), H.to_np(bias))
    assert H.rel_frobenius(H.to_np(out), want) < TOL


def test_w4a8_mx_module_and_swiglu_producer(H):
    from rk_b200 import fp4_mx_linear as PM

    m, inter, n = 100, 768, 256
    gate_up = H.randn_bf16((m, 2 * inter), 2.0, 61)
    lin = torch.nn.Linear(inter, n, bias=False, dtype=torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_(H.randn_bf16((n, inter), 0.02, 62))
    layer = PM.Fp4MxLinear.from_linear(lin.to(H.DEVICE).requires_grad_(False), "linear", "down")
    g = H.to_np(gate_up)
    act = OB.swiglu_f32(g, inter)
    ca, sa, swa = OB.pack_mxfp8_ceil(act)
    for interleaved in (False, True):
        src = gate_up
        if interleaved:  # build the interleaved layout from [gate | up]: per 64 columns, up block then gate block
            blocks = torch.stack([gate_up[:, inter:].reshape(m, inter // 64, 64), gate_up[:, :inter].reshape(m, inter // 64, 64)], dim=2)
            src = blocks.reshape(m, 2 * inter).contiguous()
            assert np.array_equal(OB.deinterleave_gate_up(H.to_np(src), inter), g)
        q, sf = PM.pack_swiglu_mxfp8(src.to(H.DEVICE), inter, interleaved)
        # device expf differs from the host's by an ulp at most: nearly all codes identical, scales identical
        assert np.array_equal(sf.cpu().numpy(), swa)
        assert (q.view(torch.uint8).cpu().numpy() != ca).mean() < 0.01
        out = layer.forward_swiglu(src.to(H.DEVICE), inter, interleaved)
        pb, sb, _ = OB.pack_mxfp4_ceil(H.to_np(lin.weight.detach()))
        _, want = OB.gemm_dequantized(OB.dequant_mxfp8(ca, sa), OB.dequant_mxfp4(pb, sb))
        assert H.rel_frobenius(H.to_np(out), want) < TOL


# ---------------------------------------------------------------- interleaved gate/up layout, NVFP4
def test_nvfp4_swiglu_pack_reads_the_interleaved_layout(H):
    from rk_b200 import fp4_linear as P4

    m, inter = 70, 256
    gate_up = H.randn_bf16((m, 2 * inter), 2.0, 71)
    blocks = torch.stack([gate_up[:, inter:].reshape(m, inter // 64, 64), gate_up[:, :inter].reshape(m, inter // 64, 64)], dim=2)
    interleaved = blocks.reshape(m, 2 * inter).contiguous()
    q0, sf0 = P4.pack_swiglu_nvfp4(gate_up.to(H.DEVICE), inter)
    q1, sf1 = P4.pack_swiglu_nvfp4(interleaved.to(H.DEVICE), inter, interleaved=True)
    assert torch.equal(q0, q1) and torch.equal(sf0, sf1)  # same values, different source layout
    with pytest.raises(ValueError):
        P4.pack_swiglu_nvfp4(H.randn_bf16((4, 2 * 96), 1.0, 72).to(H.DEVICE), 96, interleaved=True)
