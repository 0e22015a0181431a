"""The column-parallel FP8 GEMM whose epilogue performs the exchange, on ONE GPU.

Two to eight "ranks" are emulated as launches on the same device, one after the other on one stream:
each computes its slab of columns and stores it into BOTH full-width output buffers, then raises its
flag in both flag arrays.  The wait kernels are launched only after both GEMMs (nothing ever waits
for a kernel that has not been launched), so they return at once.  Both buffers must equal the
one-GPU GEMM bit for bit.  The wait's give-up path is exercised with a flag that nothing sets."""

import ctypes

import pytest
import torch

from rk_b200 import _lib

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def H():
    import gpu_helpers

    return gpu_helpers


def _table(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


# slab widths that are and are not multiples of the store chunk; row counts on both sides of the swap threshold (1024)
@pytest.mark.parametrize("m,slab,k,ranks", [(300, 256, 448, 2), (816, 160, 512, 2), (50, 64, 128, 4), (130, 2048, 2048, 2), (1300, 320, 256, 2),
                                            (64, 64, 128, 8), (816, 2048, 2048, 8)])  # the last: the benchmark's projection over eight ranks
def test_two_emulated_ranks_fill_every_buffer(H, m, slab, k, ranks):
    from rk_b200 import fp8_linear as P8

    lib = _lib.load()
    n = slab * ranks
    x, w, bias = H.randn_bf16((m, k), 1.0, 81), H.randn_bf16((n, k), 0.02, 82), H.randn_bf16((n,), 0.01, 83)
    xd, wd, bd = x.to(H.DEVICE), w.to(H.DEVICE), bias.to(H.DEVICE)
    wq, wscale = P8.quantize_bf16(wd)
    xq, xscale = P8.quantize_bf16(xd)
    want = P8.linear_forward_packed(xq, xscale, wq, wscale, bd, tactic=2)  # no split-K: the same summation order

    outs = [torch.full((m + 1, n), 3.0, dtype=torch.bfloat16, device=H.DEVICE) for _ in range(ranks)]
    flags = [torch.zeros(8, dtype=torch.int32, device=H.DEVICE) for _ in range(ranks)]
    counters = [torch.zeros(1, dtype=torch.int32, device=H.DEVICE) for _ in range(ranks)]  # one call counter per rank
    waits = [torch.zeros(1, dtype=torch.int32, device=H.DEVICE) for _ in range(ranks)]  # and one per rank's wait kernel
    ws = _lib.gemm_workspace(_lib.OP_FP8, H.DEVICE, m, slab, k)
    stream = H.stream()
    for epoch in (1, 2):
        for r in range(ranks):
            w_r = wq[r * slab:(r + 1) * slab].contiguous()
            b_r = bd[r * slab:(r + 1) * slab].contiguous()
            H.call("rk_gemm_fp8_column_parallel", _lib.ptr(xq), _lib.ptr(xscale), _lib.ptr(w_r), _lib.ptr(wscale), _lib.ptr(b_r),
                   m, slab, k, _table(outs), None, n, r * slab, _table(flags), r, ranks, _lib.ptr(counters[r]), _lib.ptr(ws),
                   ws.numel(), stream)
        for r in range(ranks):
            H.call("rk_wait_peers", _lib.ptr(flags[r]), ranks, _lib.ptr(waits[r]), _lib.ptr(ws), ws.numel(), stream)
        assert _lib.read_status(ws) == 0
        for r in range(ranks):
            assert flags[r][:ranks].tolist() == [epoch] * ranks
            assert torch.equal(outs[r][:m], want)
            assert (outs[r][m] == 3.0).all()  # the row past the end is untouched
            outs[r][:m].fill_(3.0)


def test_wait_gives_up_on_a_flag_nothing_sets(H):
    lib = _lib.load()
    flags = torch.zeros(8, dtype=torch.int32, device=H.DEVICE)
    counter = torch.full((1,), 4, dtype=torch.int32, device=H.DEVICE)  # four waits so far: this one expects 5
    ws = torch.zeros(_lib.WORKSPACE_HEADER, dtype=torch.uint8, device=H.DEVICE)
    flags[0] = 5  # this rank's own slab is there, the peer's never arrives
    assert lib.rk_debug_wait_expiry(1, 4096) == _lib.RK_OK
    try:
        assert lib.rk_wait_peers(_lib.ptr(flags), 2, _lib.ptr(counter), _lib.ptr(ws), ws.numel(), H.stream()) == _lib.RK_OK
        code = ctypes.c_int(0)
        rc = lib.rk_read_status(_lib.ptr(ws), ctypes.byref(code), H.stream())
    finally:
        assert lib.rk_debug_wait_expiry(0, 0) == _lib.RK_OK
    assert rc == _lib.RK_EDEVICE and code.value == 107 and counter.item() == 5
    # flags that have reached the next count return without a status
    flags[:2] = 6
    assert lib.rk_wait_peers(_lib.ptr(flags), 2, _lib.ptr(counter), _lib.ptr(ws), ws.numel(), H.stream()) == _lib.RK_OK
    assert _lib.read_status(ws) == 0 and counter.item() == 6


def test_module_with_one_rank_equals_the_plain_linear(H):
    from rk_b200 import replicas
    from rk_b200.fp8_linear import Fp8CutlassLinear

    m, n, k = 200, 384, 256
    lin = torch.nn.Linear(k, n, bias=True, dtype=torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_(H.randn_bf16((n, k), 0.02, 91))
        lin.bias.copy_(H.randn_bf16((n,), 0.01, 92))
    lin = lin.to(H.DEVICE).requires_grad_(False)
    single = Fp8CutlassLinear.from_linear(lin, "linear", "gate_up")
    fused = replicas.FusedColumnParallelLinear(single, replicas.RankInfo(0, 1, 0), max_rows=256)
    x = H.randn_bf16((2, 100, k), 1.0, 93).to(H.DEVICE)
    want = single(x).float()
    for _ in range(3):  # the two buffers alternate; the plain linear may split K (another summation order)
        got = fused(x).float()
        assert float((got - want).norm() / want.norm()) < 1e-3
    with pytest.raises(ValueError):
        fused(H.randn_bf16((300, k), 1.0, 94).to(H.DEVICE))
    fused.close()
