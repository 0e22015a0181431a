"""NVFP4 Linear on the B200 tcgen05 kernels (E2M1 codes, one UE4M3 scale per 16 k,
``kind::mxf4nvf4.block_scale.scale_vec::4X``), activations quantized on the fly.

Host-side mirror of the reference's ``src/robotics_kernels/blackwell/fp4_linear.py``
(``Fp4CutlassLinear``: ``from_linear(linear, role, target_name)``, ``pack_input``,
``forward_packed``, ``forward``, ``fp4_backend``, status helpers).  ``global_scale=False``
reproduces the reference's format exactly (no per-tensor scale, alpha = 1:
blackwell/csrc/fp4_cutlass_linear.cu:1358); ``global_scale=True`` adds the fp32 per-tensor scale
``amax / (6 * 448)`` on weights and activations that the benchmark configuration asks for.
The reference's other activation modes map to other modules of this package: ``bf16`` (W4A16) to
``W4A16Linear``.
"""

from dataclasses import dataclass

import torch

from . import _lib


@dataclass
class Fp4BackendStatus:
    available: bool
    error: str | None
    backend: str = "b200_tcgen05_nvfp4"

    def to_dict(self):
        return {"available": self.available, "error": self.error, "backend": self.backend}


def fp4_backend_status(device=None):
    ok, error = _lib.backend_status()
    if ok and torch.cuda.is_available():
        major, minor = torch.cuda.get_device_capability(device)
        if not _lib.load().rk_supports_device(major, minor):
            ok, error = False, f"compute capability {major}.{minor} is not supported (sm_100 only)"
    elif ok:
        ok, error = False, "CUDA is not available"
    return Fp4BackendStatus(ok, error)


def require_fp4_backend(device=None):
    status = fp4_backend_status(device)
    if not status.available:
        raise RuntimeError(f"FP4 backend unavailable: {status.to_dict()}")


def tensor_global_scale(x):
    """float32[1] = max(amax / (6 * 448), 1e-12)."""
    scale = torch.empty(1, device=x.device, dtype=torch.float32)
    with torch.cuda.device(x.device):
        ws = _lib.workspace(x.device, _lib.WORKSPACE_HEADER)
        code = _lib.load().rk_nvfp4_global_scale(_lib.ptr(x), x.numel(), _lib.ptr(scale), _lib.ptr(ws), ws.numel(),
                                                 _lib.stream_ptr(x.device))
    _lib.check(code, "tensor_global_scale")
    return scale


def pack_nvfp4(x, global_scale=None):
    """bf16 [rows, K] -> (uint8 [rows, K/2] codes, uint8 swizzled UE4M3 scale buffer); K % 32 == 0."""
    if not x.is_cuda or x.dtype != torch.bfloat16 or not x.is_contiguous() or x.dim() != 2 or x.shape[1] % 32:
        raise ValueError("NVFP4 pack requires contiguous CUDA BF16 [M,K] with K divisible by 32")
    rows, k = x.shape
    lib = _lib.load()
    q = torch.empty((rows, k // 2), device=x.device, dtype=torch.uint8)
    sf = torch.empty(lib.rk_sf_bytes(rows, k // 16), device=x.device, dtype=torch.uint8)
    with torch.cuda.device(x.device):
        code = lib.rk_pack_nvfp4(_lib.ptr(x), rows, k, _lib.ptr(global_scale), _lib.ptr(q), _lib.ptr(sf),
                                 _lib.stream_ptr(x.device))
    _lib.check(code, "pack_nvfp4")
    return q, sf


def add_rms_norm_fp4_quant_bf16(x, residual, weight, epsilon, write_normalized=True):
    """(residual add +) RMSNorm packed straight to NVFP4: -> (summed, normalized or None, codes, scale buffer).

    Mirrors `robotics_cutlass_fp4::add_rms_norm_fp4_quant_bf16` (blackwell/csrc/fp4_cutlass_linear.cu:2538-2608):
    x, residual bf16 [rows, K] (residual may be None), weight bf16 [K], K % 32 == 0."""
    for t, what in ((x, "input"), (weight, "weight")) + (((residual, "residual"),) if residual is not None else ()):
        if not t.is_cuda or t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise ValueError(f"add_rms_norm_fp4_quant_bf16 {what} must be a contiguous CUDA BF16 tensor")
    if x.dim() != 2 or x.shape[1] % 32 or weight.shape != (x.shape[1],) or (residual is not None and residual.shape != x.shape):
        raise ValueError("add_rms_norm_fp4_quant_bf16 requires [rows, K] inputs with K divisible by 32 and weight [K]")
    rows, k = x.shape
    lib = _lib.load()
    summed = torch.empty_like(x) if residual is not None else x
    normalized = torch.empty_like(x) if write_normalized else None
    q = torch.empty((rows, k // 2), device=x.device, dtype=torch.uint8)
    sf = torch.empty(lib.rk_sf_bytes(rows, k // 16), device=x.device, dtype=torch.uint8)
    with torch.cuda.device(x.device):
        code = lib.rk_rmsnorm_pack_nvfp4(_lib.ptr(x), _lib.ptr(residual), _lib.ptr(weight), rows, k, float(epsilon),
                                         _lib.ptr(summed) if residual is not None else None, _lib.ptr(normalized),
                                         _lib.ptr(q), _lib.ptr(sf), _lib.stream_ptr(x.device))
    _lib.check(code, "add_rms_norm_fp4_quant_bf16")
    return summed, normalized, q, sf


def cutlass_silu_mul_bf16(gate_up, intermediate_size, interleaved=False):
    """SiLU(gate) * up in the reference's bf16 steps -> bf16 [..., inter] (`robotics_cutlass_fp4::silu_mul_bf16`,
    blackwell/fp4_linear.py:378-384); gate_up [..., 2 * inter], gate first, or the 64-column interleaved layout."""
    inter = int(intermediate_size)
    if not gate_up.is_cuda or gate_up.dtype != torch.bfloat16 or not gate_up.is_contiguous() or gate_up.numel() == 0:
        raise ValueError("gate_up must be a non-empty contiguous CUDA BF16 tensor")
    if inter <= 0 or inter % 8 or gate_up.shape[-1] != 2 * inter or (interleaved and inter % 64):
        raise ValueError("gate_up last dimension must equal 2 * intermediate_size (a multiple of 8; 64 when interleaved)")
    rows = gate_up.numel() // (2 * inter)
    out = torch.empty((*gate_up.shape[:-1], inter), dtype=torch.bfloat16, device=gate_up.device)
    with torch.cuda.device(gate_up.device):
        code = _lib.load().rk_silu_mul_bf16(_lib.ptr(gate_up), rows, inter, 1 if interleaved else 0, _lib.ptr(out),
                                            _lib.stream_ptr(gate_up.device))
    _lib.check(code, "cutlass_silu_mul_bf16")
    return out


def add_rms_norm_bf16(x, residual, weight, epsilon):
    """(residual add +) RMSNorm with bf16 rounding after each product (`robotics_cutlass_fp4::rms_norm_bf16` /
    `add_rms_norm_bf16`): -> normalized, or (summed, normalized) with a residual."""
    for t, what in ((x, "input"), (weight, "weight")) + (((residual, "residual"),) if residual is not None else ()):
        if not t.is_cuda or t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise ValueError(f"rms_norm_bf16 {what} must be a contiguous CUDA BF16 tensor")
    k = x.shape[-1]
    if k % 16 or weight.shape != (k,) or (residual is not None and residual.shape != x.shape):
        raise ValueError("rms_norm_bf16 requires [..., K] inputs with K divisible by 16 and weight [K]")
    rows = x.numel() // k
    summed = torch.empty_like(x) if residual is not None else None
    normalized = torch.empty_like(x)
    with torch.cuda.device(x.device):
        code = _lib.load().rk_rmsnorm_bf16(_lib.ptr(x), _lib.ptr(residual), _lib.ptr(weight), rows, k, float(epsilon),
                                           _lib.ptr(summed), _lib.ptr(normalized), _lib.stream_ptr(x.device))
    _lib.check(code, "rms_norm_bf16")
    return normalized if residual is None else (summed, normalized)


def rms_norm_bf16(x, weight, epsilon):
    return add_rms_norm_bf16(x, None, weight, epsilon)


class PackedNvfp4Activation:
    """An activation that already is NVFP4 (codes, swizzled block scales, fp32 per-tensor scale or None):
    what a fused norm hands to the `Fp4CutlassLinear` layers that read it.  `shape` is the shape of
    the bf16 tensor it stands for."""

    _robotics_packed_input = True

    def __init__(self, codes, scale_factors, global_scale, leading_shape, features):
        self.codes, self.scale_factors, self.global_scale = codes, scale_factors, global_scale
        self.leading_shape = tuple(leading_shape)
        self.features = int(features)

    @property
    def shape(self):
        return torch.Size((*self.leading_shape, self.features))

    @property
    def device(self):
        return self.codes.device

    def packs_for(self, layer):
        if self.features != layer.in_features:
            raise ValueError("Wrong input feature count")
        if (self.global_scale is None) != (layer.weight_global_scale is None):
            raise ValueError("the packed activation and the layer disagree on per-tensor scales")
        return self.codes, self.scale_factors, self.global_scale


def gemma_rms_norm_pack_nvfp4(x, weight, eps, residual=None, global_scale=True):
    """Gemma RMSNorm (fp32 statistics, x * inv * (1 + w), one rounding to bf16; plain residual add in
    front) handed on as NVFP4: one kernel for add + norm + the tensor's absolute maximum
    (`rk_rmsnorm_tensor_scale`) and the block packer.  x, residual bf16 [..., K] contiguous.
    Returns (PackedNvfp4Activation, residual stream)."""
    if not x.is_cuda or x.dtype != torch.bfloat16 or not x.is_contiguous() or x.shape[-1] % 32:
        raise ValueError("gemma_rms_norm_pack_nvfp4 requires contiguous CUDA BF16 [..., K] with K divisible by 32")
    if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype or not residual.is_contiguous()):
        raise ValueError("the residual must match the input")
    k = x.shape[-1]
    rows = x.numel() // k
    lib = _lib.load()
    normed = torch.empty((rows, k), dtype=torch.bfloat16, device=x.device)
    stream_out = torch.empty_like(x) if residual is not None else x
    ga = torch.empty(1, dtype=torch.float32, device=x.device) if global_scale else None
    with torch.cuda.device(x.device):
        ws = _lib.workspace(x.device, _lib.WORKSPACE_HEADER)
        code = lib.rk_rmsnorm_tensor_scale(_lib.ptr(x), _lib.ptr(residual), _lib.ptr(weight), None, 0, rows, k, float(eps),
                                           6.0 * 448.0, _lib.ptr(stream_out) if residual is not None else None,
                                           _lib.ptr(normed), _lib.ptr(ga), _lib.ptr(ws), ws.numel(),
                                           _lib.stream_ptr(x.device))
    _lib.check(code, "gemma_rms_norm_pack_nvfp4")
    q, sf = pack_nvfp4(normed, ga)
    return PackedNvfp4Activation(q, sf, ga, x.shape[:-1], k), stream_out


def table_mul_tensor_scale(x, up, table, divisor=None):
    """bf16(table[x] * up) as a contiguous [rows, K] matrix plus, with `divisor`, the per-tensor scale
    max(amax / divisor, 1e-12) of it (`rk_lut_mul_tensor_scale`).  x, up: bf16 with dense last axis and
    one row stride (slices of a wider matrix are fine)."""
    k = x.shape[-1]
    x2, up2 = x.reshape(-1, k), up.reshape(-1, k)
    for t in (x2, up2):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.stride(-1) != 1:
            raise ValueError("table_mul_tensor_scale takes CUDA BF16 rows")
    rows = x2.shape[0]
    out = torch.empty((rows, k), dtype=torch.bfloat16, device=x.device)
    scale = torch.empty(1, dtype=torch.float32, device=x.device) if divisor is not None else None
    with torch.cuda.device(x.device):
        ws = _lib.workspace(x.device, _lib.WORKSPACE_HEADER)
        code = _lib.load().rk_lut_mul_tensor_scale(_lib.ptr(x2), x2.stride(0), _lib.ptr(up2), up2.stride(0), _lib.ptr(table),
                                                   rows, k, float(divisor or 1.0), _lib.ptr(out), _lib.ptr(scale),
                                                   _lib.ptr(ws), ws.numel(), _lib.stream_ptr(x.device))
    _lib.check(code, "table_mul_tensor_scale")
    return out, scale


def pack_swiglu_nvfp4(gate_up, intermediate_size, interleaved=False):
    """SiLU(gate) * up (bf16 arithmetic steps) packed straight to NVFP4: gate_up bf16 [rows, 2 * inter], gate
    first, or `interleaved`: blocks of 128 columns with 64 up values followed by their 64 gate values."""
    inter = int(intermediate_size)
    if (not gate_up.is_cuda or gate_up.dtype != torch.bfloat16 or not gate_up.is_contiguous() or gate_up.dim() != 2
            or gate_up.shape[1] != 2 * inter or inter % (64 if interleaved else 32)):
        raise ValueError("SwiGLU NVFP4 pack requires contiguous CUDA BF16 [rows, 2 * inter] with inter divisible by 32 "
                         "(64 for the interleaved layout)")
    rows = gate_up.shape[0]
    lib = _lib.load()
    q = torch.empty((rows, inter // 2), device=gate_up.device, dtype=torch.uint8)
    sf = torch.empty(lib.rk_sf_bytes(rows, inter // 16), device=gate_up.device, dtype=torch.uint8)
    with torch.cuda.device(gate_up.device):
        code = lib.rk_swiglu_pack_nvfp4_layout(_lib.ptr(gate_up), rows, inter, 1 if interleaved else 0, _lib.ptr(q),
                                               _lib.ptr(sf), _lib.stream_ptr(gate_up.device))
    _lib.check(code, "pack_swiglu_nvfp4")
    return q, sf


def linear_forward_packed_gemm_bf16(a, sfa, ga, b, sfb, gb, bias, k, tactic=0):
    m, n = a.shape[0], b.shape[0]
    out = torch.empty((m, n), device=a.device, dtype=torch.bfloat16)
    with torch.cuda.device(a.device):
        ws = _lib.gemm_workspace(_lib.OP_NVFP4, a.device, m, n, k)
        code = _lib.load().rk_gemm_nvfp4(_lib.ptr(a), _lib.ptr(sfa), _lib.ptr(ga), _lib.ptr(b), _lib.ptr(sfb),
                                         _lib.ptr(gb), _lib.ptr(bias), _lib.ptr(out), m, n, k, tactic, _lib.ptr(ws),
                                         ws.numel(), _lib.stream_ptr(a.device))
    _lib.check(code, "linear_forward_packed_gemm_bf16")
    return out


def interleave_gate_up_rows(weight, intermediate_size):
    """Rows of a fused gate/up weight [2 * inter, K] ([gate | up] along the output channels) in the
    64-row interleaved order the fused SwiGLU GEMM reads: of every 128 rows the first 64 are `up`
    channels 64 j .. 64 j + 63, the next 64 their `gate` channels.  inter must be a multiple of 64."""
    inter = intermediate_size
    if weight.shape[0] != 2 * inter or inter % 64:
        raise ValueError("expected a [2 * inter, K] weight with inter a multiple of 64")
    gate = weight[:inter].reshape(inter // 64, 64, -1)
    up = weight[inter:].reshape(inter // 64, 64, -1)
    return torch.stack([up, gate], dim=1).reshape(2 * inter, -1).contiguous()


def linear_swiglu_packed_gemm(a, sfa, ga, b_interleaved, sfb, gb, k, tactic=0):
    """NVFP4 gate/up projection with SwiGLU and the NVFP4 re-pack in the GEMM's epilogue
    (`rk_gemm_nvfp4_swiglu`): packed activations [M, K/2] x interleaved packed weight [2 * inter, K/2]
    -> (codes [M, inter/2], swizzled scale factors) ready for the down projection.  The counterpart
    of `cutlass_swiglu_fp4_packed` (blackwell/cute_fp4_swiglu.py:186-282)."""
    m, n = a.shape[0], b_interleaved.shape[0]
    if n % 128:
        raise ValueError("the fused SwiGLU projection needs 2 * inter to be a multiple of 128")
    q = torch.empty((m, n // 4), device=a.device, dtype=torch.uint8)
    sf = torch.empty(_lib.load().rk_sf_bytes(m, n // 32), device=a.device, dtype=torch.uint8)
    with torch.cuda.device(a.device):
        ws = _lib.gemm_workspace(_lib.OP_NVFP4, a.device, m, n, k)
        code = _lib.load().rk_gemm_nvfp4_swiglu(_lib.ptr(a), _lib.ptr(sfa), _lib.ptr(ga), _lib.ptr(b_interleaved), _lib.ptr(sfb),
                                                _lib.ptr(gb), _lib.ptr(q), _lib.ptr(sf), m, n, k, tactic, _lib.ptr(ws),
                                                ws.numel(), _lib.stream_ptr(a.device))
    _lib.check(code, "linear_swiglu_packed_gemm")
    return q, sf


def linear_gated_act_gemm(a, sfa, ga, b_interleaved, sfb, gb, k, table, divisor=None, tactic=0):
    """NVFP4 gate/up projection whose epilogue writes bf16(table[gate] * up) (`rk_gemm_nvfp4_gated_act`): packed
    activations [M, K/2] x interleaved packed weight [2 * inter, K/2] -> (bf16 [M, inter], per-tensor scale
    max(amax / divisor, 1e-12) or None without a divisor)."""
    m, n = a.shape[0], b_interleaved.shape[0]
    if n % 128:
        raise ValueError("the fused gated projection needs 2 * inter to be a multiple of 128")
    out = torch.empty((m, n // 2), device=a.device, dtype=torch.bfloat16)
    scale = torch.empty(1, device=a.device, dtype=torch.float32) if divisor is not None else None
    with torch.cuda.device(a.device):
        ws = _lib.gemm_workspace(_lib.OP_NVFP4, a.device, m, n, k)
        code = _lib.load().rk_gemm_nvfp4_gated_act(_lib.ptr(a), _lib.ptr(sfa), _lib.ptr(ga), _lib.ptr(b_interleaved), _lib.ptr(sfb),
                                                   _lib.ptr(gb), _lib.ptr(table), float(divisor or 1.0), _lib.ptr(out),
                                                   _lib.ptr(scale), m, n, k, tactic, _lib.ptr(ws), ws.numel(),
                                                   _lib.stream_ptr(a.device))
    _lib.check(code, "linear_gated_act_gemm")
    return out, scale


class Fp4GateUpGelu(torch.nn.Module):
    """The gate and up projections of a GELU-gated MLP as ONE NVFP4 GEMM whose epilogue writes
    GELU(gate) * up (the 65536-entry bf16 table of the integer layers' `forward_gelu`) and collects the
    tensor's maximum: `forward_into(down, x)` packs that product and runs the down projection, and the
    [M, 2 * inter] bf16 gate/up tensor never exists.  The fused weight is packed as one tensor (one
    per-tensor scale for both halves when `global_scale`), its rows in the 64-row interleaved order."""

    def __init__(self, packed, scales, weight_global, in_features, intermediate_size, approximate="tanh"):
        super().__init__()
        self.register_buffer("packed_weight", packed)
        self.register_buffer("weight_scale", scales)
        self.register_buffer("weight_global_scale", weight_global)
        self.in_features = in_features
        self.intermediate_size = intermediate_size
        self.approximate = approximate
        self.fp4_backend = "b200_tcgen05_nvfp4_gelu" + ("_global" if weight_global is not None else "")

    @classmethod
    def from_linears(cls, gate, up, global_scale=False, approximate="tanh"):
        if gate.weight.shape != up.weight.shape or gate.bias is not None or up.bias is not None:
            raise ValueError("gate and up must be bias-free linears of the same shape")
        if not gate.weight.is_cuda or gate.weight.dtype != torch.bfloat16:
            raise ValueError("Fp4GateUpGelu requires CUDA BF16 weights")
        require_fp4_backend(gate.weight.device)
        inter, k = gate.weight.shape
        if inter % 64 or k % 64:
            raise ValueError("Fp4GateUpGelu requires intermediate_size % 64 == 0 and in_features % 64 == 0")
        fused = interleave_gate_up_rows(torch.cat([gate.weight.detach(), up.weight.detach()], dim=0), inter)
        weight_global = tensor_global_scale(fused) if global_scale else None
        packed, scales = pack_nvfp4(fused, weight_global)
        return cls(packed, scales, weight_global, k, inter, approximate)

    def pack_input(self, x):
        if isinstance(x, PackedNvfp4Activation):
            return x.packs_for(self)
        if x.shape[-1] != self.in_features:
            raise ValueError("Wrong input feature count")
        flat = x.reshape(-1, self.in_features)
        flat = flat if flat.is_contiguous() else flat.contiguous()
        ga = tensor_global_scale(flat) if self.weight_global_scale is not None else None
        q, sf = pack_nvfp4(flat, ga)
        return q, sf, ga

    def forward(self, x):
        """-> (bf16 [rows, inter] GELU(gate) * up, its per-tensor scale or None)."""
        from .integer import prepare_gelu

        q, sf, ga = self.pack_input(x)
        table = prepare_gelu(q.device, torch.bfloat16, self.approximate)
        return linear_gated_act_gemm(q, sf, ga, self.packed_weight, self.weight_scale, self.weight_global_scale, self.in_features,
                                     table, 6.0 * 448.0 if self.weight_global_scale is not None else None)

    def forward_into(self, down, x):
        """The whole MLP: this projection, the packer, `down.forward_packed` (an `Fp4CutlassLinear` with the same
        per-tensor-scale setting)."""
        if (down.weight_global_scale is None) != (self.weight_global_scale is None) or down.in_features != self.intermediate_size:
            raise ValueError("the down projection does not match this gate/up projection")
        product, scale = self(x)
        q, sf = pack_nvfp4(product, scale)
        return down.forward_packed(q, sf, scale, x.shape[:-1])


class Fp4CutlassLinear(torch.nn.Module):
    def __init__(self, packed, scales, weight_global, bias, in_features, out_features, role, target_name):
        super().__init__()
        self.register_buffer("packed_weight", packed)
        self.register_buffer("weight_scale", scales)
        self.register_buffer("weight_global_scale", weight_global)
        self.register_buffer("bias", bias)
        self.register_buffer("_weight_descriptor", torch.empty(0, device=packed.device, dtype=torch.bfloat16),
                             persistent=False)
        self.in_features = in_features
        self.out_features = out_features
        self.role = role
        self.target_name = target_name
        self.fp4_backend = "b200_tcgen05_nvfp4" + ("_global" if weight_global is not None else "")

    @classmethod
    def from_linear(cls, linear, role, target_name, global_scale=False):
        if not linear.weight.is_cuda or linear.weight.dtype != torch.bfloat16:
            raise ValueError("Fp4CutlassLinear requires CUDA BF16 weights")
        require_fp4_backend(linear.weight.device)
        n, k = linear.weight.shape
        if n % 8 or k % 64:
            raise ValueError("Fp4CutlassLinear requires out_features % 8 == 0 and in_features % 64 == 0")
        w = linear.weight.detach().contiguous()
        weight_global = tensor_global_scale(w) if global_scale else None
        packed, scales = pack_nvfp4(w, weight_global)
        bias = None if linear.bias is None else linear.bias.detach().to(torch.bfloat16).contiguous()
        return cls(packed, scales, weight_global, bias, k, n, role, target_name)

    @property
    def weight(self):
        return self._weight_descriptor

    def pack_input(self, x):
        if isinstance(x, PackedNvfp4Activation):
            return x.packs_for(self)
        if x.shape[-1] != self.in_features:
            raise ValueError("Wrong input feature count")
        flat = x.reshape(-1, self.in_features)
        if not flat.is_contiguous():
            flat = flat.contiguous()
        ga = tensor_global_scale(flat) if self.weight_global_scale is not None else None
        q, sf = pack_nvfp4(flat, ga)
        return q, sf, ga

    def forward_packed(self, packed, scales, activation_global=None, shape=None):
        out = linear_forward_packed_gemm_bf16(packed, scales, activation_global, self.packed_weight, self.weight_scale,
                                              self.weight_global_scale, self.bias, self.in_features)
        return out if shape is None else out.reshape(*shape, self.out_features)

    def forward(self, x):
        q, sf, ga = self.pack_input(x)
        return self.forward_packed(q, sf, ga, x.shape[:-1])

    def forward_gelu(self, x, up=None, *, approximate="tanh"):
        """GELU(x) (* up) through the 65536-entry bf16 table of the integer layers' `forward_gelu`, the
        per-tensor scale collected by the same kernel, then the block packer and the GEMM."""
        from .integer import prepare_gelu

        if x.shape[-1] != self.in_features:
            raise ValueError("Wrong input feature count")
        if up is None:
            return self.forward(torch.nn.functional.gelu(x, approximate=approximate))
        table = prepare_gelu(x.device, x.dtype, approximate)
        product, ga = table_mul_tensor_scale(x, up, table, 6.0 * 448.0 if self.weight_global_scale is not None else None)
        q, sf = pack_nvfp4(product, ga)
        return self.forward_packed(q, sf, ga, x.shape[:-1])

    def forward_swiglu(self, gate_up, intermediate_size, interleaved=False):
        """SwiGLU, activation packing and this (down) projection (blackwell/fp4_linear.py:805-848 of the
        reference); gate_up [..., 2 * intermediate_size], gate first, or the reference's interleaved
        layout (64 up columns, then their 64 gate columns, per block of 128)."""
        if int(intermediate_size) != self.in_features:
            raise ValueError(f"expected intermediate_size {self.in_features}, got {intermediate_size}")
        if self.weight_global_scale is not None:
            raise RuntimeError("forward_swiglu packs without a per-tensor scale; build the layer with global_scale=False")
        flat = gate_up.to(torch.bfloat16).reshape(-1, 2 * self.in_features).contiguous()
        q, sf = pack_swiglu_nvfp4(flat, self.in_features, interleaved)
        return self.forward_packed(q, sf, None, gate_up.shape[:-1])

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, role={self.role}"


class Fp4GateUpSwiglu(torch.nn.Module):
    """The gate and up projections of a SwiGLU MLP as ONE NVFP4 GEMM whose epilogue applies SwiGLU and
    packs the result to NVFP4 (`linear_swiglu_packed_gemm`): `forward(x)` returns the packed
    activations (codes, scale factors) that the down projection's `forward_packed` consumes, and the
    [M, 2 * inter] bf16 intermediate never exists.  No bias, no per-tensor scale (the reference's
    NVFP4 format); the weight rows are stored in the 64-row interleaved order."""

    def __init__(self, packed, scales, in_features, intermediate_size):
        super().__init__()
        self.register_buffer("packed_weight", packed)
        self.register_buffer("weight_scale", scales)
        self.in_features = in_features
        self.intermediate_size = intermediate_size
        self.fp4_backend = "b200_tcgen05_nvfp4_swiglu"

    @classmethod
    def from_linears(cls, gate, up):
        if gate.weight.shape != up.weight.shape or gate.bias is not None or up.bias is not None:
            raise ValueError("gate and up must be bias-free linears of the same shape")
        if not gate.weight.is_cuda or gate.weight.dtype != torch.bfloat16:
            raise ValueError("Fp4GateUpSwiglu requires CUDA BF16 weights")
        require_fp4_backend(gate.weight.device)
        inter, k = gate.weight.shape
        if inter % 64 or k % 64:
            raise ValueError("Fp4GateUpSwiglu requires intermediate_size % 64 == 0 and in_features % 64 == 0")
        fused = interleave_gate_up_rows(torch.cat([gate.weight.detach(), up.weight.detach()], dim=0), inter)
        packed, scales = pack_nvfp4(fused, None)
        return cls(packed, scales, k, inter)

    def forward(self, x):
        if x.shape[-1] != self.in_features:
            raise ValueError("Wrong input feature count")
        flat = x.reshape(-1, self.in_features)
        q, sf = pack_nvfp4(flat if flat.is_contiguous() else flat.contiguous(), None)
        return linear_swiglu_packed_gemm(q, sf, None, self.packed_weight, self.weight_scale, None, self.in_features)

