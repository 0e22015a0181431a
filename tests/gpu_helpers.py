"""Helpers shared by the GPU parity tests: seeded inputs, device buffers, C-ABI call wrappers."""

import numpy as np
import torch

from oracle import formats as F
from rk_b200 import _lib

DEVICE = torch.device("cuda:0")


def randn_bf16(shape, std, seed):
    gen = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=gen) * std).to(torch.bfloat16)


def to_np(t):
    """bf16 / f32 tensor -> float32 numpy (exact)."""
    return t.detach().float().cpu().numpy()


def from_np_bf16(a):
    """float32 numpy holding bf16-representable values -> bf16 tensor."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16)


def bits(t):
    return F.bf16_bits(to_np(t))


def stream():
    return _lib.stream_ptr(DEVICE)


def call(name, *args):
    code = getattr(_lib.load(), name)(*args)
    _lib.check(code, name)


def quant_rows(x, bits_, up=None, lut=None, mode=_lib.ACT_PLAIN, x_stride=None):
    rows, k = x.shape
    kp = (k + 127) // 128 * 128
    q = torch.full((rows, kp if bits_ == 8 else kp // 2), 0x5A, dtype=torch.uint8, device=DEVICE)
    s = torch.full((rows,), -1.0, dtype=torch.float32, device=DEVICE)
    call("rk_quant_rows", _lib.ptr(x), rows, k, x_stride or x.stride(0), _lib.ptr(up),
         0 if up is None else up.stride(0), _lib.ptr(lut), mode, bits_, _lib.ptr(q), _lib.ptr(s), stream())
    return q, s


def quant_weight(w, bits_):
    n, k = w.shape
    npad, kp = (n + 7) // 8 * 8, (k + 127) // 128 * 128
    q = torch.full((npad, kp if bits_ == 8 else kp // 2), 0x5A, dtype=torch.uint8, device=DEVICE)
    s = torch.full((npad,), -1.0, dtype=torch.float32, device=DEVICE)
    call("rk_quant_weight_int", _lib.ptr(w), n, k, bits_, _lib.ptr(q), _lib.ptr(s), stream())
    return q, s


def gemm_int_acc(a, b, tactic=0, bits_=8):
    m, n = a.shape[0], b.shape[0]
    kpad = a.shape[1] * (2 if bits_ == 4 else 1)
    acc = torch.full((m, n), -12345, dtype=torch.int32, device=DEVICE)
    ws = _lib.gemm_workspace(_lib.OP_W8A8, DEVICE, m, n, kpad)
    call("rk_gemm_int_acc", _lib.ptr(a), _lib.ptr(b), _lib.ptr(acc), m, n, kpad, bits_, tactic, _lib.ptr(ws),
         ws.numel(), stream())
    assert _lib.read_status(ws) == 0
    return acc, ws


def gemm_int(a, sa, b, sb, bias, tactic=0, bits_=8):
    m, n = a.shape[0], b.shape[0]
    kpad = a.shape[1] * (2 if bits_ == 4 else 1)
    # canary rows around the output catch out-of-bounds stores
    buf = torch.full((m + 2, n), 7.0, dtype=torch.bfloat16, device=DEVICE)
    out = buf[1:m + 1]
    ws = _lib.gemm_workspace(_lib.OP_W8A8, DEVICE, m, n, kpad)
    call("rk_gemm_int", _lib.ptr(a), _lib.ptr(sa), _lib.ptr(b), _lib.ptr(sb), _lib.ptr(bias), _lib.ptr(out), m, n,
         kpad, bits_, tactic, _lib.ptr(ws), ws.numel(), stream())
    assert _lib.read_status(ws) == 0
    assert (buf[0] == 7.0).all() and (buf[m + 1] == 7.0).all(), "store outside the output"
    return out, ws


def workspace_is_clean(ws):
    return not bool(ws.any().item())


def rel_frobenius(actual, expected):
    e = np.asarray(expected, dtype=np.float64)
    d = np.asarray(actual, dtype=np.float64) - e
    return float(np.sqrt((d * d).sum()) / max(np.sqrt((e * e).sum()), 1e-30))
