"""The give-up path of the kernels' bounded waits, exercised on purpose.

Every device-side wait in the GEMM kernels is limited; when one runs out the kernel records a code in
its status word, drains and returns normally.  `rk_debug_wait_expiry` makes that happen without any
fault: the first pipeline stage of each CTA is announced 16 bytes larger than what is copied, so its
"full" phase never completes, and every wait is limited to a few thousand polls.  The test checks
that the launch returns, that `rk_read_status` reports RK_EDEVICE with the consumer-timeout code,
and that an ordinary launch right afterwards is bit-exact again."""

import ctypes

import numpy as np
import pytest
import torch

from oracle import formats as F
from oracle import integer as OI
from rk_b200 import _lib

pytestmark = pytest.mark.gpu
# device codes 101..106: which role's wait ran out first (consumer of a stage, producer, epilogue, ...);
# the consumer and the epilogue give up at about the same time, either may record its code
RK_DEV_TIMEOUT_CODES = range(101, 107)


def _case(m, n, k, seed):
    gen = torch.Generator().manual_seed(seed)
    a = torch.randint(-127, 128, (m, k), generator=gen, dtype=torch.int8)
    b = torch.randint(-127, 128, (n, k), generator=gen, dtype=torch.int8)
    sa = torch.rand(m, generator=gen) * 0.02 + 0.001
    sb = torch.rand(n, generator=gen) * 0.01 + 0.001
    return a, b, sa, sb


# tactic 2 forbids split-K: (64, 256, 512) then runs the persistent schedule; K = 4096 with tactic 0 takes the cluster split-K one
@pytest.mark.parametrize("shape,tactic", [((64, 256, 512), 2), ((64, 256, 4096), 0), ((300, 1024, 256), 0)])
def test_wait_expiry_sets_status_and_the_next_launch_is_exact(shape, tactic):
    lib = _lib.load()
    device = torch.device("cuda:0")
    m, n, k = shape
    a, b, sa, sb = _case(m, n, k, 5)
    ad, bd, sad, sbd = (t.to(device) for t in (a, b, sa, sb))
    out = torch.zeros((m, n), dtype=torch.bfloat16, device=device)
    ws = _lib.gemm_workspace(_lib.OP_W8A8, device, m, n, k)
    stream = _lib.stream_ptr(device)

    def launch():
        return lib.rk_gemm_int(_lib.ptr(ad), _lib.ptr(sad), _lib.ptr(bd), _lib.ptr(sbd), None, _lib.ptr(out), m, n, k, 8,
                               tactic, _lib.ptr(ws), ws.numel(), stream)

    assert lib.rk_debug_wait_expiry(1, 4096) == _lib.RK_OK
    try:
        assert launch() == _lib.RK_OK  # the launch itself succeeds; the kernel gives up on the device
        code = ctypes.c_int(0)
        rc = lib.rk_read_status(_lib.ptr(ws), ctypes.byref(code), stream)
    finally:
        assert lib.rk_debug_wait_expiry(0, 0) == _lib.RK_OK
    assert rc == _lib.RK_EDEVICE
    assert code.value in RK_DEV_TIMEOUT_CODES
    assert "bounded wait" in _lib.last_error()

    # the status word was cleared by the read; the context is intact and the next launch is exact
    assert launch() == _lib.RK_OK
    assert _lib.read_status(ws) == 0
    want = OI.dequant_epilogue(OI.int_matmul(a.numpy(), b.numpy()), sa.numpy(), sb.numpy(), None)
    assert np.array_equal(F.bf16_bits(out.float().cpu().numpy()), F.bf16_bits(want))


def test_debug_knob_rejects_unreasonable_limits():
    lib = _lib.load()
    assert lib.rk_debug_wait_expiry(1, 3) == _lib.RK_EINVAL
    assert lib.rk_debug_wait_expiry(0, 0) == _lib.RK_OK
