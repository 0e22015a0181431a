"""GPU parity of the integer path (row / weight quantizers, W8A8 GEMM + dequant epilogue), called
through the C ABI and through the Linear modules, against the CPU oracle and the golden fixtures
produced by the reference's own kernels.  Bit-exact everywhere."""

import numpy as np
import pytest
import torch

from conftest import bf16_from_bits
from oracle import formats as F
from oracle import integer as OI

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def H():
    import gpu_helpers

    return gpu_helpers


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("shape", [(64, 2048), (3, 130), (50, 256), (5, 9000), (400, 1024), (2, 1), (7, 8191)])
def test_row_quantizer_matches_oracle(H, bits, shape):
    x = H.randn_bf16(shape, 1.0, 11)
    if shape[0] > 2:
        x[1] = 0
    q, s = H.quant_rows(x.to(H.DEVICE), bits)
    eq, es, _ = OI.quantize_rows(H.to_np(x), bits)
    assert np.array_equal(s.cpu().numpy(), es)
    assert np.array_equal(q.cpu().numpy(), eq.view(np.uint8))


@pytest.mark.parametrize("case", range(4))
@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_row_quantizer_matches_reference_fixture(H, golden, case, bits, mode):
    """Same inputs as the reference's Triton kernel saw; same bytes out."""
    x = torch.from_numpy(bf16_from_bits(golden[f"rows{case}_x"])).to(torch.bfloat16).to(H.DEVICE)
    up = lut = None
    if mode == 1:
        up = torch.from_numpy(bf16_from_bits(golden[f"rows{case}_up"])).to(torch.bfloat16).to(H.DEVICE)
    if mode:
        lut = torch.from_numpy(bf16_from_bits(golden["gelu_tanh_lut"])).to(torch.bfloat16).to(H.DEVICE)
    q, s = H.quant_rows(x, bits, up=up, lut=lut, mode=mode)
    tag = f"rows{case}_b{bits}_m{mode}_r0"
    assert np.array_equal(s.cpu().numpy(), golden[tag + "_s"])
    assert np.array_equal(q.cpu().numpy(), golden[tag + "_q"])


def test_row_quantizer_accepts_strided_and_unaligned_rows(H):
    base = H.randn_bf16((9, 300), 1.0, 5).to(H.DEVICE)
    view = base[:, 3:133]  # row stride 300, start offset 3 elements: scalar load path
    q, s = H.quant_rows(view, 8, x_stride=300)
    eq, es, _ = OI.quantize_rows(H.to_np(view), 8)
    assert np.array_equal(s.cpu().numpy(), es) and np.array_equal(q.cpu().numpy(), eq.view(np.uint8))


@pytest.mark.parametrize("case", range(3))
@pytest.mark.parametrize("bits", [8, 4])
def test_weight_quantizer_matches_reference_fixture(H, golden, case, bits):
    w = torch.from_numpy(bf16_from_bits(golden[f"w{case}_w"])).to(torch.bfloat16).to(H.DEVICE)
    q, s = H.quant_weight(w, bits)
    assert np.array_equal(s.cpu().numpy(), golden[f"w{case}_b{bits}_s"])
    assert np.array_equal(q.cpu().numpy(), golden[f"w{case}_b{bits}_q"])


@pytest.mark.parametrize("shape", [(16, 128, 128), (128, 128, 128), (64, 128, 512), (1, 40, 256), (50, 80, 256),
                                   (64, 2048, 2048), (400, 1024, 1024), (300, 520, 384), (1764, 2048, 2048),
                                   (64, 256, 4096), (100, 384, 8192)])  # the last two: few tiles, long K: cluster split-K
@pytest.mark.parametrize("tactic", [0, 1, 2, 5])
def test_int8_accumulators_are_exact(H, shape, tactic):
    m, n, k = shape
    gen = torch.Generator().manual_seed(3)
    a = torch.randint(-127, 128, (m, k), generator=gen, dtype=torch.int8)
    b = torch.randint(-127, 128, (n, k), generator=gen, dtype=torch.int8)
    acc, ws = H.gemm_int_acc(a.to(H.DEVICE), b.to(H.DEVICE), tactic)
    assert np.array_equal(acc.cpu().numpy(), OI.int_matmul(a.numpy(), b.numpy()))
    assert H.workspace_is_clean(ws)


@pytest.mark.parametrize("shape", [(1, 40, 256), (50, 80, 256), (64, 2048, 2048), (400, 1024, 1024), (1764, 2048, 2048)])
def test_int4_accumulators_are_exact(H, shape):
    """W4A4: packed nibbles in, the same int32 sums as the oracle's nibble-unpacked product."""
    m, n, k = shape
    gen = torch.Generator().manual_seed(4)
    a = torch.randint(-7, 8, (m, k), generator=gen, dtype=torch.int8)
    b = torch.randint(-7, 8, (n, k), generator=gen, dtype=torch.int8)
    pa = torch.from_numpy(OI.pack_nibbles(a.numpy())).to(H.DEVICE)
    pb = torch.from_numpy(OI.pack_nibbles(b.numpy())).to(H.DEVICE)
    acc = torch.full((m, n), -12345, dtype=torch.int32, device=H.DEVICE)
    from rk_b200 import _lib

    ws = _lib.gemm_workspace(_lib.OP_W4A4, H.DEVICE, m, n, k)
    H.call("rk_gemm_int_acc", _lib.ptr(pa), _lib.ptr(pb), _lib.ptr(acc), m, n, k, 4, 0, _lib.ptr(ws), ws.numel(),
           H.stream())
    assert _lib.read_status(ws) == 0
    assert np.array_equal(acc.cpu().numpy(), OI.int_matmul(a.numpy(), b.numpy()))
    assert H.workspace_is_clean(ws)


def test_int8_accumulators_at_extreme_codes(H):
    """All codes at +-127 with K = 8192: |acc| reaches 1.3e8, far beyond fp32's exact-integer range."""
    m, n, k = 32, 256, 8192
    a = torch.full((m, k), 127, dtype=torch.int8)
    b = torch.full((n, k), -127, dtype=torch.int8)
    b[::2] = 127
    acc, _ = H.gemm_int_acc(a.to(H.DEVICE), b.to(H.DEVICE))
    assert np.array_equal(acc.cpu().numpy(), OI.int_matmul(a.numpy(), b.numpy()))


@pytest.mark.parametrize("tactic", range(8))
def test_w8a8_cfg1_bit_exact_for_every_tactic(H, tactic):
    """BASELINE config 1: M=64, K=N=2048, bias; quantize + GEMM + epilogue, bf16 output bit-exact."""
    m, n, k = 64, 2048, 2048
    x = H.randn_bf16((m, k), 1.0, 42)
    w = H.randn_bf16((n, k), 0.02, 43)
    bias = H.randn_bf16((n,), 0.01, 44)
    qa, sa = H.quant_rows(x.to(H.DEVICE), 8)
    qb, sb = H.quant_weight(w.to(H.DEVICE), 8)
    out, ws = H.gemm_int(qa, sa, qb, sb, bias.to(H.DEVICE), tactic)
    want, _ = OI.linear(H.to_np(x), H.to_np(w), H.to_np(bias), 8)
    assert np.array_equal(H.bits(out), F.bf16_bits(want))
    assert H.workspace_is_clean(ws)


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("shape", [(1, 37, 130), (50, 80, 256)])
@pytest.mark.parametrize("tactic", [0, 3, 7])
def test_integer_linear_matches_quantized_reference_on_nondefault_stream(H, bits, shape, tactic):
    """The reference's own GPU test (tests/gpu/test_integer_linear.py:12-41)."""
    from rk_b200.integer import IntegerLinear

    m, n, k = shape
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        torch.manual_seed(1)
        original = torch.nn.Linear(k, n, device="cuda", dtype=torch.bfloat16).eval()
        layer = IntegerLinear.from_linear(original, bits=bits, tactic=tactic)
        x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
        actual = layer(x)
    side.synchronize()
    want, _ = OI.linear(H.to_np(x), H.to_np(original.weight), H.to_np(original.bias), bits)
    assert np.array_equal(H.bits(actual), F.bf16_bits(want))
    assert actual.shape == (m, n) and actual.is_contiguous()
    assert layer.backend == f"b200_tcgen05_int{bits}_s32_bf16"
    assert layer.weight.dtype == torch.bfloat16


@pytest.mark.parametrize("case", range(2))
def test_integer_linear_against_known_answer_fixture(H, golden, case):
    """Rows whose activation scale agrees with the test formula's must equal the reference's
    known-answer output bit for bit."""
    from rk_b200.integer import IntegerLinear

    x = torch.from_numpy(bf16_from_bits(golden[f"ka{case}_x"])).to(torch.bfloat16)
    w = torch.from_numpy(bf16_from_bits(golden[f"ka{case}_w"])).to(torch.bfloat16)
    b = torch.from_numpy(bf16_from_bits(golden[f"ka{case}_bias"])).to(torch.bfloat16)
    lin = torch.nn.Linear(w.shape[1], w.shape[0], dtype=torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_(w)
        lin.bias.copy_(b)
    layer = IntegerLinear.from_linear(lin.to(H.DEVICE), bits=8)
    got = H.bits(layer(x.to(H.DEVICE)))
    want = golden[f"ka{case}_b8_out"]
    _, kernel_scales, _ = OI.quantize_rows(H.to_np(x), 8)
    same = kernel_scales == (np.abs(H.to_np(x)).max(axis=1) / np.float32(127)).astype(np.float32)
    assert same.any()
    assert np.array_equal(got[same], want[same])


@pytest.mark.parametrize("bits", [8, 4])
def test_fused_gelu_pack_matches_separate_path(H, bits):
    from rk_b200.integer import IntegerLinear

    torch.manual_seed(2)
    layer = IntegerLinear.from_linear(torch.nn.Linear(256, 80, device="cuda", dtype=torch.bfloat16).eval(), bits=bits)
    gate = torch.randn(17, 256, device="cuda", dtype=torch.bfloat16)
    up = torch.randn_like(gate)
    expected = layer(torch.nn.functional.gelu(gate, approximate="tanh") * up)
    assert torch.equal(layer.forward_gelu(gate, up), expected)
    assert torch.equal(layer.forward_gelu(gate), layer(torch.nn.functional.gelu(gate, approximate="tanh")))


@pytest.mark.parametrize("bits", [8, 4])
def test_grouped_projections_match_individual_layers(H, bits):
    from rk_b200.integer import IntegerLinear, IntegerProjectionGroup, IntegerProjectionSlice

    torch.manual_seed(4)
    sizes, k = (37, 17, 48), 256
    linears = [torch.nn.Linear(k, n, bias=(i != 1), device="cuda", dtype=torch.bfloat16).eval()
               for i, n in enumerate(sizes)]
    layers = [IntegerLinear.from_linear(m, bits=bits) for m in linears]
    group = IntegerProjectionGroup(layers)
    slices = [IntegerProjectionSlice(group, i) for i in range(3)]
    for seed in (0, 1):  # second round: the cached input must be refreshed
        x = H.randn_bf16((9, k), 1.0, seed).to(H.DEVICE)
        for i, layer in enumerate(layers):
            got = slices[i](x)
            assert got.is_contiguous() and torch.equal(got, layer(x))
        assert group._input is None and group._output is None
    with pytest.raises(ValueError):
        IntegerProjectionGroup([layers[0]])


def test_module_error_behaviour(H):
    from rk_b200.integer import IntegerLinear, prepare_activation

    lin = torch.nn.Linear(128, 8, device="cuda", dtype=torch.bfloat16)
    layer = IntegerLinear.from_linear(lin, bits=8)
    with pytest.raises(ValueError):
        layer(torch.zeros(2, 64, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        prepare_activation(torch.zeros(2, 128, device="cuda", dtype=torch.float16), 8)
    with pytest.raises(ValueError):
        prepare_activation(torch.zeros(2, 128, dtype=torch.bfloat16), 8)  # CPU tensor
    with pytest.raises(ValueError):
        IntegerLinear.from_linear(torch.nn.Linear(128, 8, dtype=torch.bfloat16), bits=8)  # CPU weights
    with pytest.raises(ValueError):
        IntegerLinear.from_linear(lin, bits=3)
    bad = torch.nn.Linear(128, 8, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        bad.weight[0, 0] = float("inf")
    with pytest.raises(ValueError):
        IntegerLinear.from_linear(bad, bits=8)


def test_w8a8_under_cuda_graph_replay_with_changed_inputs(H):
    from rk_b200.integer import IntegerLinear

    torch.manual_seed(6)
    lin = torch.nn.Linear(1024, 2048, bias=False, device="cuda", dtype=torch.bfloat16).eval()
    layer = IntegerLinear.from_linear(lin, bits=8)
    static_x = torch.randn(400, 1024, device="cuda", dtype=torch.bfloat16)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            layer(static_x)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            static_y = layer(static_x)
    torch.cuda.current_stream().wait_stream(side)
    for seed in (8, 9):
        x = H.randn_bf16((400, 1024), 1.0, seed)
        static_x.copy_(x.to(H.DEVICE))
        graph.replay()
        torch.cuda.synchronize()
        want, _ = OI.linear(H.to_np(x), H.to_np(lin.weight), None, 8)
        assert np.array_equal(H.bits(static_y), F.bf16_bits(want))


# (m, n, k): swapped whole tiles, a split-K shape, the chunked paths on both sides of the swap threshold, a ragged n
@pytest.mark.parametrize("shape,tokens", [((400, 1024, 2048), 50), ((400, 1024, 4096), 50), ((64, 256, 4096), 1),
                                          ((100, 384, 8192), 100), ((1300, 512, 256), 130), ((816, 264, 384), 816),
                                          ((130, 2048, 128), 65)])
@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("gated", [True, False])
def test_residual_epilogue_equals_the_tensor_ops(H, shape, tokens, bits, gated):
    """`rk_gemm_int_residual`: the projection's epilogue writes stream + y (* gate) with the three roundings
    of the tensor ops on the bf16 output y of the plain GEMM - bit for bit, in every epilogue layout."""
    from rk_b200 import integer as I

    m, n, k = shape
    x = H.randn_bf16((m, k), 1.0, 71).to(H.DEVICE)
    lin = torch.nn.Linear(k, n, bias=True, dtype=torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_(H.randn_bf16((n, k), 0.02, 72))
        lin.bias.copy_(H.randn_bf16((n,), 0.01, 73))
    layer = I.IntegerLinear.from_linear(lin.to(H.DEVICE), bits=bits)
    stream = H.randn_bf16((m, n), 1.0, 74).to(H.DEVICE)
    gate = H.randn_bf16((m // tokens, n), 0.5, 75).to(H.DEVICE) if gated else None
    packed = layer.pack_input(x)
    y = layer.forward_packed(packed)
    want = stream + (y if gate is None else y * gate.repeat_interleave(tokens, 0))
    got = layer.forward_packed(packed, residual=stream, gate=gate)
    assert got.shape == (m, n) and torch.equal(got, want)
    # leading axes and a [B, 1, N] gate, as the decoder layers pass them
    if gated and m % tokens == 0:
        got3 = layer.forward_packed(I.PackedActivation(packed.data, packed.scales, (m // tokens, tokens), packed.logical_k, bits),
                                    residual=stream.reshape(m // tokens, tokens, n), gate=gate[:, None, :])
        assert torch.equal(got3.reshape(m, n), want)


def test_residual_epilogue_refuses_bad_arguments(H):
    from rk_b200 import _lib
    from rk_b200 import integer as I

    lin = torch.nn.Linear(256, 128, bias=False, dtype=torch.bfloat16).to(H.DEVICE)
    layer = I.IntegerLinear.from_linear(lin, bits=8)
    packed = layer.pack_input(H.randn_bf16((60, 256), 1.0, 1).to(H.DEVICE))
    stream = torch.zeros(60, 128, dtype=torch.bfloat16, device=H.DEVICE)
    with pytest.raises(RuntimeError):
        layer.forward_packed(packed, residual=stream, gate=torch.zeros(7, 128, dtype=torch.bfloat16, device=H.DEVICE))  # 60 % 7
    with pytest.raises(RuntimeError):
        layer.forward_packed(packed, residual=stream.float())
    with pytest.raises(RuntimeError):
        I.integer_gemm(packed.data, packed.scales, layer.packed_weight, layer.weight_scale, None, 8, 0, gate=stream[:1])
    lib = _lib.load()
    ws = _lib.gemm_workspace(_lib.OP_W8A8, H.DEVICE, 60, 128, 256)
    out = torch.empty_like(stream)
    args = lambda res, tok: (_lib.ptr(packed.data), _lib.ptr(packed.scales), _lib.ptr(layer.packed_weight), _lib.ptr(layer.weight_scale),
                             None, res, None, tok, _lib.ptr(out), 60, 128, 256, 8, 0, _lib.ptr(ws), ws.numel(), H.stream())
    assert lib.rk_gemm_int_residual(*args(None, 1)) == _lib.RK_EINVAL
    assert lib.rk_gemm_int_residual(*args(_lib.ptr(stream), 7)) == _lib.RK_EINVAL
    assert lib.rk_gemm_int_residual(*args(_lib.ptr(stream), 0)) == _lib.RK_EINVAL
    assert lib.rk_gemm_int_residual(*args(_lib.ptr(stream), 60)) == _lib.RK_OK
