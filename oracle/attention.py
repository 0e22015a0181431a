"""CPU oracle for the action expert's attention over a cached prefix.  Test infrastructure.

Restates `eager_attention_forward` (src/robotics_bench/models/pi05/modeling_gemma.py:247-274) for bf16
inputs with the rounding points of its tensor ops:
    scores = bf16( bf16(q . k^T) * scaling )          torch.matmul of bf16 tensors, then a bf16 multiply
    probs  = bf16( softmax_fp32(scores) )             softmax(dtype=float32).to(bf16)
    out    = bf16( probs . v )                        torch.matmul of bf16 tensors
Matmul accumulation is carried in float64 here (the order of a GPU's fp32 accumulation is not part of
the contract).  PINNED by `tests/test_oracle_attention.py` against the reference's own function
body executed by torch on CPU bf16 tensors.
"""

import numpy as np

from .formats import bf16_round, f32


def attention(q, k, v, scaling):
    """q [B, H, T, D], k / v [B, KV, S, D] as float32 arrays holding bf16 values -> [B, T, H * D]."""
    q, k, v = f32(q), f32(k), f32(v)
    b, h, t, d = q.shape
    groups = h // k.shape[1]
    kk = np.repeat(k, groups, axis=1).astype(np.float64)
    vv = np.repeat(v, groups, axis=1).astype(np.float64)
    scores = bf16_round((q.astype(np.float64) @ kk.transpose(0, 1, 3, 2)).astype(np.float32))
    scores = bf16_round((scores * np.float32(scaling)).astype(np.float32))
    m = scores.max(axis=-1, keepdims=True)
    e = np.exp((scores - m).astype(np.float32)).astype(np.float32)
    probs = bf16_round((e / e.sum(axis=-1, keepdims=True, dtype=np.float32)).astype(np.float32))
    out = bf16_round((probs.astype(np.float64) @ vv).astype(np.float32))
    return out.transpose(0, 2, 1, 3).reshape(b, t, h * d)
