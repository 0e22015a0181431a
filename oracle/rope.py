"""CPU restatement of the rotary embedding + key/value cache update (TEST INFRASTRUCTURE ONLY:
imported by tests, never by the product path).

Follows apply_rotary_pos_emb / rotate_half (models/pi05/modeling_gemma.py:178-209) evaluated on
bf16 tensors, which is also the arithmetic of the reference's fused kernels (rope_element,
blackwell/csrc/fp4_cutlass_linear.cu:96-126): every product and the final sum are rounded to bf16,
with fp32 arithmetic in between.  Parity unpinned: the reference holds no stored vectors for this
op; the GPU test additionally compares against the same chain of bf16 tensor ops.
"""

import numpy as np

from . import formats as F


def rotate(x, cos, sin):
    """x [..., d] bf16-valued float32, cos / sin broadcastable to x.  Returns bf16-valued float32."""
    x = np.asarray(x, np.float32)
    half = x.shape[-1] // 2
    partner = np.concatenate([-x[..., half:], x[..., :half]], axis=-1)
    first = F.bf16_round(x * np.asarray(cos, np.float32))
    second = F.bf16_round(partner * np.asarray(sin, np.float32))
    return F.bf16_round(first + second)


def cache_update(q, k, v, cos, sin, k_cache, v_cache, prefix):
    """q [B, t, H, d], k / v [B, t, G, d], cos / sin [B, t, d], caches [B, G, rows, d] (modified in
    place at rows prefix .. prefix + t).  Returns the rotated queries as [B, H, t, d]."""
    t = q.shape[1]
    q_out = rotate(q, cos[:, :, None, :], sin[:, :, None, :]).transpose(0, 2, 1, 3)
    k_rot = rotate(k, cos[:, :, None, :], sin[:, :, None, :]).transpose(0, 2, 1, 3)
    k_cache[:, :, prefix:prefix + t] = k_rot
    v_cache[:, :, prefix:prefix + t] = np.asarray(v, np.float32).transpose(0, 2, 1, 3)
    return q_out
