"""W4A16 Linear: BF16 activations x group-wise int4 weights (group 128 along K, BF16 group scales).

Plays the role of the reference's ``Fp4CutlassLinear`` in its ``bf16`` activation mode
(``W4A16``: src/robotics_kernels/blackwell/fp4_linear.py:492-521 and fp4_mixed_linear.py), with
the weight format the benchmark configuration asks for: symmetric signed int4, limit 7, two
nibbles per byte (low nibble = even k), one BF16 scale per (128 k, output channel) stored
``[K/128, N]``.  The GEMM runs in ``librk_b200.so``; there is no fallback.
"""

import torch

from . import _lib

GROUP = 128
BACKEND = "b200_tcgen05_w4a16_int4_g128_bf16"


def pack_weight(weight):
    """CUDA BF16 [N, K] -> (packed uint8 [N, K/2], scales bf16 [K/128, N])."""
    if not weight.is_cuda or weight.dtype != torch.bfloat16 or weight.dim() != 2:
        raise ValueError("W4A16 packing requires a CUDA BF16 [N, K] weight")
    n, k = weight.shape
    if k % GROUP:
        raise ValueError("W4A16 packing requires K divisible by 128")
    w = weight.detach().contiguous()
    packed = torch.empty((n, k // 2), device=w.device, dtype=torch.uint8)
    scales = torch.empty((k // GROUP, n), device=w.device, dtype=torch.bfloat16)
    with torch.cuda.device(w.device):
        code = _lib.load().rk_pack_w4_g128(_lib.ptr(w), n, k, _lib.ptr(packed), _lib.ptr(scales),
                                           _lib.stream_ptr(w.device))
    _lib.check(code, "pack_weight")
    return packed, scales


def linear_w4a16(x, packed, scales, bias=None, tactic=0):
    """x BF16 [M, K] contiguous -> BF16 [M, N]."""
    if not x.is_cuda or x.dtype != torch.bfloat16 or x.dim() != 2 or not x.is_contiguous():
        raise ValueError("linear_w4a16 requires a contiguous CUDA BF16 [M, K] input")
    m, k = x.shape
    n = packed.shape[0]
    if packed.shape[1] * 2 != k or scales.shape != (k // GROUP, n):
        raise ValueError("Packed weight or scales do not match the input width")
    out = torch.empty((m, n), device=x.device, dtype=torch.bfloat16)
    with torch.cuda.device(x.device):
        ws = _lib.gemm_workspace(_lib.OP_W4A16, x.device, m, n, k)
        code = _lib.load().rk_gemm_w4a16_g128(
            _lib.ptr(x), _lib.ptr(packed), _lib.ptr(scales), _lib.ptr(bias), _lib.ptr(out), m, n, k, tactic,
            _lib.ptr(ws), ws.numel(), _lib.stream_ptr(x.device),
        )
    _lib.check(code, "linear_w4a16")
    return out


class W4A16Linear(torch.nn.Module):
    def __init__(self, packed, scales, bias, in_features, out_features, tactic=0):
        super().__init__()
        self.register_buffer("packed_weight", packed)
        self.register_buffer("weight_scale", scales)
        self.register_buffer("bias", bias)
        self.register_buffer(
            "_weight_descriptor", torch.empty(0, device=packed.device, dtype=torch.bfloat16), persistent=False
        )
        self.in_features = in_features
        self.out_features = out_features
        self.tactic = tactic
        self.backend = BACKEND

    @property
    def weight(self):
        return self._weight_descriptor

    @classmethod
    def from_linear(cls, linear, *, tactic=0):
        if not linear.weight.is_cuda or linear.weight.dtype != torch.bfloat16:
            raise ValueError("W4A16Linear requires CUDA BF16 weights")
        if not torch.isfinite(linear.weight).all():
            raise ValueError("Weights must be finite")
        n, k = linear.weight.shape
        if n % 8:
            raise ValueError("W4A16Linear requires out_features divisible by 8")
        packed, scales = pack_weight(linear.weight)
        bias = None if linear.bias is None else linear.bias.detach().to(torch.bfloat16).contiguous()
        return cls(packed, scales, bias, k, n, tactic)

    def forward(self, x):
        if x.shape[-1] != self.in_features:
            raise ValueError("Wrong input feature count")
        flat = x.reshape(-1, self.in_features)
        if not flat.is_contiguous():
            flat = flat.contiguous()
        out = linear_w4a16(flat, self.packed_weight, self.weight_scale, self.bias, self.tactic)
        return out.reshape(*x.shape[:-1], self.out_features)
