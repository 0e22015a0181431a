"""The rotary-embedding restatement against the reference's own formulation run on bf16 tensors
(apply_rotary_pos_emb / rotate_half, models/pi05/modeling_gemma.py:178-209): same bits."""

import numpy as np
import torch

from oracle import formats as F
from oracle import rope as R


def _rotate_half(x):
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def test_rotation_matches_bf16_tensor_ops_bit_for_bit():
    gen = torch.Generator().manual_seed(0)
    for batch, tokens, heads, dim in ((2, 5, 3, 32), (1, 50, 8, 256), (3, 1, 1, 16)):
        q = (torch.randn(batch, tokens, heads, dim, generator=gen) * 3).to(torch.bfloat16)
        positions = torch.arange(tokens)[None].expand(batch, -1) + 816
        inv_freq = 1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        angles = positions.float()[..., None] * inv_freq
        emb = torch.cat((angles, angles), dim=-1)
        cos, sin = emb.cos().to(torch.bfloat16), emb.sin().to(torch.bfloat16)
        want = q * cos[:, :, None] + _rotate_half(q) * sin[:, :, None]
        got = R.rotate(q.float().numpy(), cos.float().numpy()[:, :, None], sin.float().numpy()[:, :, None])
        assert np.array_equal(F.bf16_bits(got), F.bf16_bits(want.float().numpy()))


def test_cache_update_writes_only_the_new_rows():
    rng = np.random.default_rng(1)
    b, t, h, g, d, prefix, rows = 2, 4, 3, 1, 16, 5, 12
    bf = lambda a: F.bf16_round(a.astype(np.float32))
    q, k, v = bf(rng.standard_normal((b, t, h, d))), bf(rng.standard_normal((b, t, g, d))), bf(rng.standard_normal((b, t, g, d)))
    cos, sin = bf(rng.standard_normal((b, t, d))), bf(rng.standard_normal((b, t, d)))
    k_cache, v_cache = np.full((b, g, rows, d), 7.0, np.float32), np.full((b, g, rows, d), 9.0, np.float32)
    q_out = R.cache_update(q, k, v, cos, sin, k_cache, v_cache, prefix)
    assert q_out.shape == (b, h, t, d)
    assert (k_cache[:, :, :prefix] == 7.0).all() and (k_cache[:, :, prefix + t:] == 7.0).all()
    assert (v_cache[:, :, :prefix] == 9.0).all() and (v_cache[:, :, prefix + t:] == 9.0).all()
    assert np.array_equal(v_cache[:, :, prefix:prefix + t], v.transpose(0, 2, 1, 3))
    assert np.array_equal(k_cache[:, 0, prefix:prefix + t], R.rotate(k[:, :, 0], cos, sin))
