"""The allocation-free W4A4 entry point, called through the C ABI.

Some callers cannot allocate device memory at the moment they need a GEMM (a fixed memory plan,
a thread that must not touch the allocator).  `rk_gemm_int4_noalloc` serves them from a scratch
array that is part of the library image.  This test checks it against the ordinary entry point
(`rk_gemm_int`, which takes a caller workspace) on two calls in a row with different inputs, and
that oversize problems are refused.  The file name sorts last so that a stop-at-first-failure run
has already executed every other test."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _operands(seed, m, n, k, device):
    from oracle import integer as OI

    gen = torch.Generator().manual_seed(seed)
    a = torch.randint(-7, 8, (m, k), generator=gen, dtype=torch.int8).numpy()
    b = torch.randint(-7, 8, (n, k), generator=gen, dtype=torch.int8).numpy()
    pa = torch.from_numpy(OI.pack_nibbles(a)).to(device)
    pb = torch.from_numpy(OI.pack_nibbles(b)).to(device)
    sa = (torch.rand(m, generator=gen) * 0.05 + 0.01).to(device)
    sb = (torch.rand(n, generator=gen) * 0.01 + 0.001).to(device)
    bias = (torch.randn(n, generator=gen) * 0.1).to(torch.bfloat16).to(device)
    return a, b, pa, pb, sa, sb, bias


def test_no_alloc_entry_matches_workspace_entry_twice_in_a_row():
    from oracle import formats as F
    from oracle import integer as OI
    from rk_b200 import _lib

    lib = _lib.load()
    device = torch.device("cuda:0")
    stream = _lib.stream_ptr(device)
    for seed, (m, n, k) in ((1, (50, 80, 256)), (2, (400, 1024, 2048))):
        a, b, pa, pb, sa, sb, bias = _operands(seed, m, n, k, device)
        want = torch.empty((m, n), dtype=torch.bfloat16, device=device)
        ws = _lib.gemm_workspace(_lib.OP_W4A4, device, m, n, k)
        _lib.check(lib.rk_gemm_int(_lib.ptr(pa), _lib.ptr(sa), _lib.ptr(pb), _lib.ptr(sb), _lib.ptr(bias),
                                   _lib.ptr(want), m, n, k, 4, 0, _lib.ptr(ws), ws.numel(), stream), "rk_gemm_int")
        got = torch.full((m, n), 7.0, dtype=torch.bfloat16, device=device)

        def call():
            _lib.check(lib.rk_gemm_int4_noalloc(_lib.ptr(pa), _lib.ptr(sa), _lib.ptr(pb), _lib.ptr(sb),
                                                _lib.ptr(bias), _lib.ptr(got), m, n, k, 0, stream),
                       "rk_gemm_int4_noalloc")
            torch.cuda.synchronize(device)

        # The first call on a device loads the kernels and looks up the built-in array; after that a
        # call must leave the driver's free-memory figure untouched (the figure also covers
        # allocations that bypass torch's caching allocator, which torch's own counters do not see).
        call()
        got.fill_(7.0)
        torch.cuda.synchronize(device)
        allocated_before = torch.cuda.memory_allocated(device)
        for attempt in range(3):  # the figure is device-wide: tolerate an unrelated change once or twice
            free_before, _ = torch.cuda.mem_get_info(device)
            call()
            free_after, _ = torch.cuda.mem_get_info(device)
            if free_after >= free_before:
                break
        assert free_after >= free_before, "the call took device memory"
        assert torch.cuda.memory_allocated(device) == allocated_before
        # no bounded wait gave up inside the call: the status word of the built-in array is clear
        assert _lib.read_status(None, device) == 0
        # integer path: the two entry points must agree bit for bit, and with the oracle
        assert torch.equal(got, want)
        expect = OI.dequant_epilogue(OI.int_matmul(a, b), sa.cpu().numpy(), sb.cpu().numpy(),
                                     bias.float().cpu().numpy())
        assert np.array_equal(F.bf16_bits(got.float().cpu().numpy()), F.bf16_bits(expect))


def test_no_alloc_entry_refuses_problems_beyond_its_scratch():
    from rk_b200 import _lib

    lib = _lib.load()
    device = torch.device("cuda:0")
    dummy = torch.zeros(16, dtype=torch.uint8, device=device)
    code = lib.rk_gemm_int4_noalloc(_lib.ptr(dummy), _lib.ptr(dummy), _lib.ptr(dummy), _lib.ptr(dummy), None,
                                    _lib.ptr(dummy), 4096, 8192, 8192, 0, _lib.stream_ptr(device))
    assert code == _lib.RK_EUNSUPPORTED
    assert "scratch" in _lib.last_error()
