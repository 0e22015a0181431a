"""GPU parity of the W4A16 int4 group-128 path: packed nibbles and bf16 group scales bit-exact,
GEMM within 1e-2 relative Frobenius error of dequantize -> fp32 matmul (the stated tolerance)."""

import numpy as np
import pytest
import torch

from oracle import formats as F
from oracle import w4a16 as OW
from rk_b200 import _lib

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.fixture(scope="module")
def H():
    import gpu_helpers

    return gpu_helpers


def run_gemm(H, x, q, s, bias, m, n, k, tactic=0):
    buf = torch.full((m + 2, n), 7.0, dtype=torch.bfloat16, device=H.DEVICE)
    out = buf[1:m + 1]
    ws = _lib.gemm_workspace(_lib.OP_W4A16, H.DEVICE, m, n, k)
    H.call("rk_gemm_w4a16_g128", _lib.ptr(x), _lib.ptr(q), _lib.ptr(s), _lib.ptr(bias), _lib.ptr(out), m, n, k,
           tactic, _lib.ptr(ws), ws.numel(), H.stream())
    assert _lib.read_status(ws) == 0
    assert (buf[0] == 7.0).all() and (buf[m + 1] == 7.0).all()
    return out


def pack(H, w):
    n, k = w.shape
    q = torch.empty((n, k // 2), dtype=torch.uint8, device=H.DEVICE)
    s = torch.empty((k // 128, n), dtype=torch.bfloat16, device=H.DEVICE)
    H.call("rk_pack_w4_g128", _lib.ptr(w), n, k, _lib.ptr(q), _lib.ptr(s), H.stream())
    return q, s


@pytest.mark.parametrize("shape", [(128, 128), (1000, 384), (16384, 2048)])
def test_pack_codes_and_scales_bit_exact(H, shape):
    w = H.randn_bf16(shape, 0.02, 6)
    w[5, :128] = 0  # an all-zero group: scale 1.0, codes 0
    q, s = pack(H, w.to(H.DEVICE))
    ep, es, _ = OW.pack_weight(H.to_np(w))
    assert np.array_equal(q.cpu().numpy(), ep)
    assert np.array_equal(H.bits(s), F.bf16_bits(es))
    assert H.to_np(s)[0, 5] == 1.0


@pytest.mark.parametrize("m", [1, 8, 50, 256])
def test_cfg2_gemm_within_tolerance(H, m):
    """BASELINE config 2: N=16384, K=2048, M in {1, 8, 50, 256}."""
    n, k = 16384, 2048
    x = H.randn_bf16((m, k), 1.0, 5)
    w = H.randn_bf16((n, k), 0.02, 6)
    q, s = pack(H, w.to(H.DEVICE))
    out = run_gemm(H, x.to(H.DEVICE), q, s, None, m, n, k)
    ep, es, _ = OW.pack_weight(H.to_np(w))
    _, want = OW.gemm(H.to_np(x), ep, es)
    assert H.rel_frobenius(H.to_np(out), want) < TOL
    # element-wise: the only rounding beyond fp32 accumulation order is the bf16 output cast
    assert np.abs(H.to_np(out) - want).max() <= 2.0 ** -8 * np.abs(want).max() + 1e-6


@pytest.mark.parametrize("shape", [(8, 128, 128), (16, 256, 512), (100, 1000, 384), (130, 136, 256), (300, 256, 128)])
@pytest.mark.parametrize("tactic", [0, 4, 16, 32])
def test_ragged_shapes_and_bias(H, shape, tactic):
    m, n, k = shape
    x = H.randn_bf16((m, k), 1.0, 7)
    w = H.randn_bf16((n, k), 0.02, 8)
    bias = H.randn_bf16((n,), 0.5, 9)
    q, s = pack(H, w.to(H.DEVICE))
    out = run_gemm(H, x.to(H.DEVICE), q, s, bias.to(H.DEVICE), m, n, k, tactic)
    ep, es, _ = OW.pack_weight(H.to_np(w))
    _, want = OW.gemm(H.to_np(x), ep, es, H.to_np(bias))
    assert H.rel_frobenius(H.to_np(out), want) < TOL


@pytest.mark.parametrize("shape", [(65, 256, 256), (128, 136, 384), (129, 1000, 128), (200, 512, 512), (256, 512, 1024),
                                   (300, 256, 640), (816, 384, 256), (520, 256, 2048)])
@pytest.mark.parametrize("tactic", [0, 8])
def test_wide_batches_fold_the_scale_into_bf16_weights(H, shape, tactic):
    """Above 64 activation rows the group scale is folded into the expanded weights (one bf16
    rounding per weight).  The result must (a) stay inside the stated tolerance of the exact
    definition, (b) match the restatement that folds the same way to within fp32 summation order,
    and (c) agree with the per-group-accumulator kernel (tactic bit 1) to the same tolerance.
    With tactic bit 3, above 128 rows an even number of channel tiles runs on CTA pairs."""
    m, n, k = shape
    x = H.randn_bf16((m, k), 1.0, 17)
    w = H.randn_bf16((n, k), 0.02, 18)
    bias = H.randn_bf16((n,), 0.5, 19)
    q, s = pack(H, w.to(H.DEVICE))
    out = H.to_np(run_gemm(H, x.to(H.DEVICE), q, s, bias.to(H.DEVICE), m, n, k, tactic))
    exact_kernel = H.to_np(run_gemm(H, x.to(H.DEVICE), q, s, bias.to(H.DEVICE), m, n, k, 2))
    ep, es, _ = OW.pack_weight(H.to_np(w))
    _, want = OW.gemm(H.to_np(x), ep, es, H.to_np(bias))
    folded_bf16, folded = OW.gemm_folded(H.to_np(x), ep, es, H.to_np(bias))
    assert H.rel_frobenius(out, want) < TOL
    assert H.rel_frobenius(exact_kernel, want) < TOL
    assert H.rel_frobenius(out, exact_kernel) < TOL
    # (b): same values up to the last bf16 digit, and almost everywhere identical
    assert np.abs(out - folded).max() <= 2.0 ** -8 * np.abs(folded).max() + 1e-6
    assert (out != folded_bf16).mean() < 0.02
    assert H.rel_frobenius(out, folded) < H.rel_frobenius(out, want) + 1e-4


@pytest.mark.parametrize("shape", [(1, 256, 4096), (8, 384, 640), (32, 1000, 2048), (20, 128, 1152)])
def test_sixteen_expansion_warps_change_nothing(H, shape):
    """Sixteen expansion warps (four K groups in flight; tactic bit 4 forces them, bit 5 forces eight).  Every
    group still has its own accumulator and the groups are summed in order, so the output must be
    bit-identical to the default kernel's, for long K (ring wrap-around) and odd group counts."""
    m, n, k = shape
    x = H.randn_bf16((m, k), 1.0, 27)
    w = H.randn_bf16((n, k), 0.02, 28)
    bias = H.randn_bf16((n,), 0.5, 29)
    q, s = pack(H, w.to(H.DEVICE))
    base = run_gemm(H, x.to(H.DEVICE), q, s, bias.to(H.DEVICE), m, n, k, 32)
    wide = run_gemm(H, x.to(H.DEVICE), q, s, bias.to(H.DEVICE), m, n, k, 16)
    default = run_gemm(H, x.to(H.DEVICE), q, s, bias.to(H.DEVICE), m, n, k, 0)
    if m == 1 and k in (1024, 2048, 4096):  # one row with no tactic bit set runs on the CUDA cores: other summation order
        assert H.rel_frobenius(H.to_np(default), H.to_np(base)) < 1e-3
    else:
        assert torch.equal(default, base)
    assert torch.equal(base, wide)
    ep, es, _ = OW.pack_weight(H.to_np(w))
    _, want = OW.gemm(H.to_np(x), ep, es, H.to_np(bias))
    assert H.rel_frobenius(H.to_np(wide), want) < TOL


@pytest.mark.parametrize("shape", [(256, 1024), (1000, 2048), (16384, 2048), (136, 4096), (264, 8192), (64, 16384),
                                   (264, 5120)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_single_row_streams_on_cuda_cores(H, shape, with_bias):
    """m = 1 (tactic 0, k % 1024 == 0) takes the weight-streaming kernel: fp32 sums of exactly
    recovered x * q products, within the bf16 output rounding of the definition, equal to the
    tensor-core kernel up to summation order, and exact on integer-valued data."""
    n, k = shape
    x = H.randn_bf16((1, k), 1.0, 31)
    w = H.randn_bf16((n, k), 0.02, 32)
    bias = H.randn_bf16((n,), 0.5, 33) if with_bias else None
    q, s = pack(H, w.to(H.DEVICE))
    dev_bias = None if bias is None else bias.to(H.DEVICE)
    out = H.to_np(run_gemm(H, x.to(H.DEVICE), q, s, dev_bias, 1, n, k, 0))
    tensor_core = H.to_np(run_gemm(H, x.to(H.DEVICE), q, s, dev_bias, 1, n, k, 2))
    ep, es, _ = OW.pack_weight(H.to_np(w))
    _, want = OW.gemm(H.to_np(x), ep, es, None if bias is None else H.to_np(bias))
    assert H.rel_frobenius(out, want) < 3e-3  # bf16 output rounding alone is ~1.5e-3
    assert np.abs(out - want).max() <= 2.0 ** -8 * np.abs(want).max() + 1e-6
    assert H.rel_frobenius(out, tensor_core) < 1e-3
    # small integers everywhere: every partial sum is an exactly representable integer
    xi = torch.randint(-3, 4, (1, k)).to(torch.bfloat16)
    wi = (torch.randint(-7, 8, (n, k)).float()).to(torch.bfloat16)
    wi[:, ::128] = 7.0  # every group's maximum is 7, so its scale is exactly 1
    qi, si = pack(H, wi.to(H.DEVICE))
    got = run_gemm(H, xi.to(H.DEVICE), qi, si, None, 1, n, k, 0)
    exact = (xi.double() @ wi.double().T)
    assert torch.equal(got.cpu().double(), exact.to(torch.bfloat16).double())


def test_linearity_at_full_size(H):
    """Size-independent property: the GEMM is linear in the activations (exact powers of two)."""
    n, k, m = 16384, 2048, 50
    x = H.randn_bf16((m, k), 1.0, 10).to(H.DEVICE)
    w = H.randn_bf16((n, k), 0.02, 11).to(H.DEVICE)
    q, s = pack(H, w)
    y1 = run_gemm(H, x, q, s, None, m, n, k)
    y4 = run_gemm(H, (x * 4).contiguous(), q, s, None, m, n, k)
    assert torch.equal(y4, y1 * 4)
    assert torch.equal(run_gemm(H, x, q, s, None, m, n, k), y1)  # deterministic


def test_module_surface(H):
    from rk_b200.w4a16_linear import W4A16Linear

    torch.manual_seed(3)
    lin = torch.nn.Linear(256, 136, device="cuda", dtype=torch.bfloat16).eval()
    layer = W4A16Linear.from_linear(lin)
    x = torch.randn(2, 5, 256, device="cuda", dtype=torch.bfloat16)
    y = layer(x)
    assert y.shape == (2, 5, 136)
    ep, es, _ = OW.pack_weight(H.to_np(lin.weight))
    _, want = OW.gemm(H.to_np(x.reshape(10, 256)), ep, es, H.to_np(lin.bias))
    assert H.rel_frobenius(H.to_np(y).reshape(10, 136), want) < TOL
    with pytest.raises(ValueError):
        layer(torch.zeros(2, 128, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        W4A16Linear.from_linear(torch.nn.Linear(256, 136, dtype=torch.bfloat16))


def test_invalid_arguments_are_refused_before_any_launch(H):
    lib = _lib.load()
    x = torch.zeros(8, 256, dtype=torch.bfloat16, device=H.DEVICE)
    q = torch.zeros(128, 128, dtype=torch.uint8, device=H.DEVICE)
    s = torch.ones(2, 128, dtype=torch.bfloat16, device=H.DEVICE)
    out = torch.full((8, 128), 3.0, dtype=torch.bfloat16, device=H.DEVICE)
    ws = _lib.gemm_workspace(_lib.OP_W4A16, H.DEVICE, 8, 128, 256)
    args = lambda m, n, k, tactic: (_lib.ptr(x), _lib.ptr(q), _lib.ptr(s), None, _lib.ptr(out), m, n, k, tactic,
                                    _lib.ptr(ws), ws.numel(), H.stream())
    assert lib.rk_gemm_w4a16_g128(*args(8, 128, 200, 0)) == _lib.RK_EINVAL  # k not a multiple of 128
    assert lib.rk_gemm_w4a16_g128(*args(8, 100, 256, 0)) == _lib.RK_EINVAL  # n not a multiple of 8
    assert lib.rk_gemm_w4a16_g128(*args(8, 128, 256, 64)) == _lib.RK_EINVAL  # unknown tactic bit
    assert lib.rk_gemm_w4a16_g128(*args(8, 128, 256, -1)) == _lib.RK_EINVAL
    torch.cuda.synchronize()
    assert (out == 3.0).all()
