"""GPU parity of `rk_attention_prefix` (fresh query tokens over a cached key / value prefix) and of
the transposed value cache that `rk_rope_cache_update_vt` maintains for it.

The oracle restates the reference's eager attention (models/pi05/modeling_gemma.py:247-274) with its
rounding points; the kernel follows the same points, so the only freedom is the order of fp32
accumulation inside the two matrix products.  A score that sits on a bf16 rounding boundary may
land on the neighbouring value, which moves one probability by < 1 %: the outputs are compared by
relative Frobenius error (tolerance 5e-3, written below) and by the share of elements that differ by
more than two bf16 steps."""

import numpy as np
import pytest
import torch

from oracle import attention as OA
from rk_b200 import _lib
from rk_b200.gemma_stack import attention_prefix, rope_cache_update, rope_tables

pytestmark = pytest.mark.gpu
DEVICE = torch.device("cuda:0")
TOL = 5e-3

# (batch, tokens, heads, kv_heads, prefix): the action-expert chunk at full size, key slices that end up
# empty, two KV heads with a ragged token count, one token
CASES = [(8, 50, 8, 1, 816), (2, 10, 8, 1, 70), (3, 33, 4, 2, 267), (1, 1, 8, 1, 300), (2, 128, 2, 2, 128)]


def make_inputs(b, t, h, kvh, prefix, seed):
    gen = torch.Generator().manual_seed(seed)
    d = 256
    kv_len = prefix + t
    pitch = (kv_len + 7) // 8 * 8
    q = torch.randn(b, t, h, d, generator=gen).to(torch.bfloat16)
    k = torch.randn(b, kvh, kv_len, d, generator=gen).to(torch.bfloat16)
    v = torch.randn(b, kvh, kv_len, d, generator=gen).to(torch.bfloat16)
    return q, k, v, kv_len, pitch


@pytest.mark.parametrize("case", CASES)
def test_attention_matches_the_eager_oracle(case):
    b, t, h, kvh, prefix = case
    q, k, v, kv_len, pitch = make_inputs(b, t, h, kvh, prefix, 21)
    rows = kv_len + 5  # the caches may be longer than what is valid
    k_all = torch.full((b, kvh, rows, 256), 3.0, dtype=torch.bfloat16)
    k_all[:, :, :kv_len] = k
    vt_all = torch.zeros((b, kvh, 256, pitch), dtype=torch.bfloat16)
    vt_all[..., :kv_len] = v.transpose(-1, -2)
    out = attention_prefix(q.to(DEVICE), k_all.to(DEVICE), vt_all.to(DEVICE), kv_len)
    ws = _lib.workspace(DEVICE, _lib.WORKSPACE_HEADER)
    assert _lib.read_status(ws) == 0
    want = OA.attention(q.permute(0, 2, 1, 3).float().numpy(), k.float().numpy(), v.float().numpy(), 256 ** -0.5)
    got = out.float().cpu().numpy()
    err = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert err < TOL, f"relative Frobenius error {err}"
    step = np.maximum(np.abs(want), 2.0 ** -10) * 2.0 ** -7  # two bf16 steps
    assert (np.abs(got - want) > step).mean() < 0.01


def test_attention_matches_eager_tensor_ops_on_the_device():
    """The same comparison against the reference's four tensor ops run by torch on the GPU."""
    b, t, h, kvh, prefix = 4, 50, 8, 1, 816
    q, k, v, kv_len, pitch = make_inputs(b, t, h, kvh, prefix, 22)
    qd, kd, vd = q.to(DEVICE), k.to(DEVICE), v.to(DEVICE)
    vt_all = torch.zeros((b, kvh, 256, pitch), dtype=torch.bfloat16, device=DEVICE)
    vt_all[..., :kv_len] = vd.transpose(-1, -2)
    out = attention_prefix(qd, kd.contiguous(), vt_all, kv_len)
    qh = qd.permute(0, 2, 1, 3)
    weights = torch.matmul(qh, kd.expand(-1, h, -1, -1).transpose(2, 3)) * 256 ** -0.5
    weights = torch.nn.functional.softmax(weights, dim=-1, dtype=torch.float32).to(torch.bfloat16)
    want = torch.matmul(weights, vd.expand(-1, h, -1, -1)).transpose(1, 2).reshape(b, t, h * 256)
    err = float((out.float() - want.float()).norm() / want.float().norm())
    assert err < TOL, f"relative Frobenius error {err}"


def test_rope_kernel_maintains_the_transposed_value_cache():
    b, t, h, kvh, d, prefix = 2, 50, 8, 1, 256, 96
    gen = torch.Generator().manual_seed(23)
    width = (h + 2 * kvh) * d
    qkv = torch.randn(b, t, width, generator=gen).to(torch.bfloat16).to(DEVICE)
    q, k, v = qkv[..., :h * d], qkv[..., h * d:(h + kvh) * d], qkv[..., (h + kvh) * d:]
    positions = prefix + torch.arange(t, device=DEVICE)[None].expand(b, -1)
    cos, sin = rope_tables(positions, d, 10000.0, torch.bfloat16)
    rows = prefix + t
    pitch = (rows + 7) // 8 * 8
    k_all = torch.zeros((b, kvh, rows, d), dtype=torch.bfloat16, device=DEVICE)
    v_all = torch.zeros_like(k_all)
    vt_all = torch.full((b, kvh, d, pitch), 9.0, dtype=torch.bfloat16, device=DEVICE)
    k_plain, v_plain = torch.zeros_like(k_all), torch.zeros_like(k_all)
    q_vt = rope_cache_update(q, k, v, cos, sin, k_all, v_all, prefix, h, kvh, d, token_major=True, vt_all=vt_all)
    q_plain = rope_cache_update(q, k, v, cos, sin, k_plain, v_plain, prefix, h, kvh, d, token_major=True)
    assert torch.equal(q_vt, q_plain) and torch.equal(k_all, k_plain) and torch.equal(v_all, v_plain)
    assert torch.equal(vt_all[..., prefix:rows], v_all[:, :, prefix:rows].transpose(-1, -2))
    assert (vt_all[..., :prefix] == 9.0).all() and (vt_all[..., rows:] == 9.0).all()  # nothing else was touched


def test_attention_argument_errors():
    lib = _lib.load()
    ws = _lib.workspace(DEVICE, _lib.WORKSPACE_HEADER)
    t = torch.zeros(4096, dtype=torch.bfloat16, device=DEVICE)
    args = lambda **kw: (_lib.ptr(t), _lib.ptr(t), _lib.ptr(t), _lib.ptr(t), kw.get("batch", 1), kw.get("tokens", 4), 8, 1,
                         kw.get("dim", 256), 64, kw.get("pitch", 64), kw.get("kv_len", 64), 0.0625, _lib.ptr(ws), ws.numel(),
                         _lib.stream_ptr(DEVICE))
    assert lib.rk_attention_prefix(*args(dim=128)) == _lib.RK_EUNSUPPORTED
    assert lib.rk_attention_prefix(*args(tokens=200)) == _lib.RK_EINVAL
    assert lib.rk_attention_prefix(*args(kv_len=65)) == _lib.RK_EINVAL
    assert lib.rk_attention_prefix(*args(pitch=60)) == _lib.RK_EINVAL
