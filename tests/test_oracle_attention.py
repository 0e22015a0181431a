"""Pins `oracle/attention.py` to the reference's eager attention: the body of
`eager_attention_forward` (src/robotics_bench/models/pi05/modeling_gemma.py:247-274), i.e.
repeat_kv -> matmul * scaling -> softmax(dtype=float32).to(bf16) -> matmul -> transpose, executed by
torch on CPU bf16 tensors.  (The module itself does not import under the installed transformers, so
the four tensor ops are spelled out here exactly as the reference writes them.)"""

import numpy as np
import torch

from oracle import attention as OA


def reference_eager(query, key, value, scaling, groups):
    key_states = key[:, :, None].expand(-1, -1, groups, -1, -1).reshape(key.shape[0], -1, *key.shape[2:])
    value_states = value[:, :, None].expand(-1, -1, groups, -1, -1).reshape(value.shape[0], -1, *value.shape[2:])
    attn_weights = torch.matmul(query, key_states.transpose(2, 3)) * scaling
    attn_weights = torch.nn.functional.softmax(attn_weights, dim=-1, dtype=torch.float32).to(query.dtype)
    attn_output = torch.matmul(attn_weights, value_states)
    return attn_output.transpose(1, 2).contiguous()


def test_oracle_matches_the_reference_tensor_ops():
    gen = torch.Generator().manual_seed(11)
    b, h, kvh, t, s, d = 2, 4, 1, 10, 70, 64
    q = torch.randn(b, h, t, d, generator=gen).to(torch.bfloat16)
    k = torch.randn(b, kvh, s, d, generator=gen).to(torch.bfloat16)
    v = torch.randn(b, kvh, s, d, generator=gen).to(torch.bfloat16)
    want = reference_eager(q, k, v, d ** -0.5, h // kvh).reshape(b, t, h * d).float().numpy()
    got = OA.attention(q.float().numpy(), k.float().numpy(), v.float().numpy(), d ** -0.5)
    # the only freedom is the accumulation order inside the two matmuls: a bf16 result may land on
    # the neighbouring value when the fp32 sum sits at a rounding boundary
    diff = np.abs(got - want)
    assert diff.max() <= 2.0 ** -7 * np.abs(want).max()
    assert (got != want).mean() < 0.02
