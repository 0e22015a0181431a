"""W4A8 MX: MXFP4 weights (E2M1 codes, one power-of-two UE8M0 scale per 32 k) against MXFP8
activations packed on the fly, on the B200 tcgen05 kernels.

Host-side mirror of the reference's ``src/robotics_kernels/blackwell/fp4_mx_linear.py`` and of the
``fp8`` activation mode of its ``Fp4CutlassLinear`` (blackwell/fp4_linear.py:492-498, 639-646,
818-832): the operator names ``pack_mxfp4_weight``, ``pack_mxfp8_activation``, ``pack_swiglu_mxfp8``,
``linear_w4a8_packed`` and ``linear_w4a8`` keep their meaning.  The GEMM expands the packed weights
to e4m3 in shared memory (exact) and runs ``kind::mxf8f6f4`` with both scale sets; there is no
fallback.
"""

import torch

from . import _lib

FP8_DTYPE = torch.float8_e4m3fn


def _rows_bf16(x, what, multiple=32):
    if not x.is_cuda or x.dtype != torch.bfloat16 or not x.is_contiguous() or x.dim() != 2 or x.shape[1] % multiple:
        raise ValueError(f"{what} requires contiguous CUDA BF16 [rows, K] with K divisible by {multiple}")


def pack_mxfp4_weight(weight):
    """bf16 [N, K] -> (uint8 [N, K/2] E2M1 codes, uint8 swizzled UE8M0 scale buffer)."""
    _rows_bf16(weight, "pack_mxfp4_weight")
    n, k = weight.shape
    lib = _lib.load()
    q = torch.empty((n, k // 2), device=weight.device, dtype=torch.uint8)
    sf = torch.empty(lib.rk_sf_bytes(n, k // 32), device=weight.device, dtype=torch.uint8)
    with torch.cuda.device(weight.device):
        code = lib.rk_pack_mxfp4_weight(_lib.ptr(weight), n, k, _lib.ptr(q), _lib.ptr(sf), _lib.stream_ptr(weight.device))
    _lib.check(code, "pack_mxfp4_weight")
    return q, sf


def pack_mxfp8_activation(x):
    """bf16 [M, K] -> (e4m3 [M, K], uint8 swizzled UE8M0 scale buffer), power-of-two scales >= amax / 448."""
    _rows_bf16(x, "pack_mxfp8_activation")
    m, k = x.shape
    lib = _lib.load()
    q = torch.empty((m, k), device=x.device, dtype=FP8_DTYPE)
    sf = torch.empty(lib.rk_sf_bytes(m, k // 32), device=x.device, dtype=torch.uint8)
    with torch.cuda.device(x.device):
        code = lib.rk_pack_mxfp8_act_w4a8(_lib.ptr(x), m, k, _lib.ptr(q), _lib.ptr(sf), _lib.stream_ptr(x.device))
    _lib.check(code, "pack_mxfp8_activation")
    return q, sf


def pack_swiglu_mxfp8(gate_up, intermediate_size, interleaved=False):
    """SiLU(gate) * up (fp32, unrounded) -> MXFP8 with power-of-two scales; gate_up bf16 [M, 2 * inter]."""
    inter = int(intermediate_size)
    if (not gate_up.is_cuda or gate_up.dtype != torch.bfloat16 or not gate_up.is_contiguous() or gate_up.dim() != 2
            or gate_up.shape[1] != 2 * inter or inter % (64 if interleaved else 32)):
        raise ValueError("pack_swiglu_mxfp8 requires contiguous CUDA BF16 [rows, 2 * inter], inter divisible by 32 (64 interleaved)")
    m = gate_up.shape[0]
    lib = _lib.load()
    q = torch.empty((m, inter), device=gate_up.device, dtype=FP8_DTYPE)
    sf = torch.empty(lib.rk_sf_bytes(m, inter // 32), device=gate_up.device, dtype=torch.uint8)
    with torch.cuda.device(gate_up.device):
        code = lib.rk_swiglu_pack_mxfp8_w4a8(_lib.ptr(gate_up), m, inter, 1 if interleaved else 0, _lib.ptr(q), _lib.ptr(sf),
                                             _lib.stream_ptr(gate_up.device))
    _lib.check(code, "pack_swiglu_mxfp8")
    return q, sf


def linear_w4a8_packed(packed_input, input_scale, packed_weight, weight_scale, bias=None, tactic=0):
    """e4m3 [M, K] x MXFP4 [N, K/2] -> bf16 [M, N]."""
    m, k = packed_input.shape
    n = packed_weight.shape[0]
    if packed_weight.shape[1] * 2 != k:
        raise ValueError("packed weight width does not match the activation width")
    out = torch.empty((m, n), device=packed_input.device, dtype=torch.bfloat16)
    with torch.cuda.device(packed_input.device):
        ws = _lib.gemm_workspace(_lib.OP_MXFP8, packed_input.device, m, n, k)
        code = _lib.load().rk_gemm_w4a8_mx(_lib.ptr(packed_input), _lib.ptr(input_scale), _lib.ptr(packed_weight),
                                           _lib.ptr(weight_scale), _lib.ptr(bias), _lib.ptr(out), m, n, k, tactic,
                                           _lib.ptr(ws), ws.numel(), _lib.stream_ptr(packed_input.device))
    _lib.check(code, "linear_w4a8_packed")
    return out


def linear_w4a8(x, packed_weight, weight_scale, bias=None):
    flat = x.reshape(-1, x.shape[-1])
    flat = flat if flat.is_contiguous() else flat.contiguous()
    q, sf = pack_mxfp8_activation(flat)
    return linear_w4a8_packed(q, sf, packed_weight, weight_scale, bias).reshape(*x.shape[:-1], packed_weight.shape[0])


class Fp4MxLinear(torch.nn.Module):
    """Quantized replacement of a BF16 ``nn.Linear``: MXFP4 weights, MXFP8 activations (W4A8)."""

    def __init__(self, packed, scales, bias, in_features, out_features, role, target_name):
        super().__init__()
        self.register_buffer("packed_weight", packed)
        self.register_buffer("weight_scale", scales)
        self.register_buffer("bias", bias)
        self.register_buffer("_weight_descriptor", torch.empty(0, device=packed.device, dtype=torch.bfloat16),
                             persistent=False)
        self.in_features, self.out_features = in_features, out_features
        self.role, self.target_name = role, target_name
        self.fp4_activation_mode = "fp8"
        self.fp4_backend = "b200_tcgen05_mxfp4_mxfp8"

    @classmethod
    def from_linear(cls, linear, role, target_name):
        if not linear.weight.is_cuda or linear.weight.dtype != torch.bfloat16:
            raise ValueError("Fp4MxLinear requires CUDA BF16 weights")
        n, k = linear.weight.shape
        if n % 8 or k % 32:
            raise ValueError("Fp4MxLinear requires out_features % 8 == 0 and in_features % 32 == 0")
        packed, scales = pack_mxfp4_weight(linear.weight.detach().contiguous())
        bias = None if linear.bias is None else linear.bias.detach().to(torch.bfloat16).contiguous()
        return cls(packed, scales, bias, k, n, role, target_name)

    @property
    def weight(self):
        return self._weight_descriptor

    def forward(self, x):
        if x.shape[-1] != self.in_features:
            raise ValueError("Wrong input feature count")
        return linear_w4a8(x, self.packed_weight, self.weight_scale, self.bias)

    def forward_swiglu(self, gate_up, intermediate_size, interleaved=False):
        if int(intermediate_size) != self.in_features:
            raise ValueError(f"expected intermediate_size {self.in_features}, got {intermediate_size}")
        flat = gate_up.to(torch.bfloat16).reshape(-1, 2 * self.in_features).contiguous()
        q, sf = pack_swiglu_mxfp8(flat, self.in_features, interleaved)
        out = linear_w4a8_packed(q, sf, self.packed_weight, self.weight_scale, self.bias)
        return out.reshape(*gate_up.shape[:-1], self.out_features)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, role={self.role}, W4A8 MX"
