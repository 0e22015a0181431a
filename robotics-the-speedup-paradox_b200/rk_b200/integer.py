"""INT8 / INT4 Linear modules on the B200 tcgen05 kernels.

Host-side mirror of the reference's ``src/robotics_kernels/ampere_ada/integer.py``: the same
names (``PackedActivation``, ``prepare_activation``, ``IntegerLinear``, ``IntegerProjectionGroup``,
``IntegerProjectionSlice``), the same argument meaning and the same error behaviour, so that
``quantize_linears`` and the model hooks built on them work unchanged.  The arithmetic runs in
``librk_b200.so`` through its C ABI; nothing here computes on the host and there is no fallback.

Formats: symmetric signed row-wise activations and output-channel weights, float32 scales,
int32 accumulation, BF16 output; INT4 uses low-nibble-first bytes (``symmetric-row-v1``).
"""

from dataclasses import dataclass
import weakref

import torch

from . import _lib

BACKEND_FMT = "b200_tcgen05_int{bits}_s32_bf16"
_LUTS = {}


def prepare_gelu(device, dtype, approximate="tanh"):
    """GELU evaluated on all 65536 bf16 bit patterns (reference: common/fused.py:74-83)."""
    key = (torch.device(device), dtype, approximate)
    if key not in _LUTS:
        values = torch.arange(65536, device=device, dtype=torch.int32).to(torch.int16).view(dtype)
        _LUTS[key] = torch.nn.functional.gelu(values, approximate=approximate)
    return _LUTS[key]


@dataclass
class PackedActivation:
    data: torch.Tensor
    scales: torch.Tensor
    shape: tuple
    logical_k: int
    bits: int
    format_version: str = "symmetric-row-v1"


def _pad128(k):
    return (k + 127) // 128 * 128


def prepare_activation(x, bits, *, up=None, gelu=None, pack_reuse=False):
    """Per-row absmax quantization of BF16 rows (reference: integer.py:132-198).

    ``pack_reuse`` selects between two Triton code paths in the reference that produce the
    same bytes; it is accepted and has no effect here.
    """
    if bits not in (4, 8) or not x.is_cuda or x.dtype != torch.bfloat16 or x.stride(-1) != 1 or x.ndim < 2:
        raise ValueError("Expected CUDA BF16 rows with unit feature stride and bits=4 or 8")
    mode = _lib.ACT_PLAIN
    lut = None
    if gelu is not None:
        if gelu not in ("tanh", "none"):
            raise ValueError("Unsupported GELU approximation")
        lut = prepare_gelu(x.device, x.dtype, gelu)
        mode = _lib.ACT_LUT_MUL if up is not None else _lib.ACT_LUT
    if up is not None and (
        gelu is None or up.shape != x.shape or up.device != x.device or up.dtype != x.dtype or up.stride(-1) != 1
    ):
        raise ValueError("Invalid gated activation input")
    k = x.shape[-1]
    if k < 1 or k > 65536:
        raise ValueError("Unsupported activation dimensions")
    rows = x.numel() // k
    if rows < 1:
        raise ValueError("Unsupported activation dimensions")
    try:
        matrix = x.view(rows, k)
        up_matrix = up.view(rows, k) if up is not None else matrix
    except RuntimeError as error:
        raise ValueError("Activation leading dimensions must form regularly strided rows") from error
    pad = _pad128(k)
    data = torch.empty(
        (rows, pad if bits == 8 else pad // 2), device=x.device, dtype=torch.int8 if bits == 8 else torch.uint8
    )
    scales = torch.empty(rows, device=x.device, dtype=torch.float32)
    lib = _lib.load()
    with torch.cuda.device(x.device):
        code = lib.rk_quant_rows(
            _lib.ptr(matrix), rows, k, matrix.stride(0) if rows > 1 else k,
            _lib.ptr(up_matrix) if up is not None else None, up_matrix.stride(0) if rows > 1 else k,
            _lib.ptr(lut), mode, bits, _lib.ptr(data), _lib.ptr(scales), _lib.stream_ptr(x.device),
        )
    _lib.check(code, "prepare_activation")
    return PackedActivation(data, scales, tuple(x.shape[:-1]), k, bits)


def quantize_weight(weight, bits):
    """Per-output-channel quantization of a CUDA BF16 weight [N, K] -> (packed, scales[Npad])."""
    n, k = weight.shape
    npad = (n + 7) // 8 * 8
    kpad = _pad128(k)
    w = weight.detach().contiguous()
    packed = torch.empty(
        (npad, kpad if bits == 8 else kpad // 2), device=w.device, dtype=torch.int8 if bits == 8 else torch.uint8
    )
    scales = torch.empty(npad, device=w.device, dtype=torch.float32)
    with torch.cuda.device(w.device):
        code = _lib.load().rk_quant_weight_int(
            _lib.ptr(w), n, k, bits, _lib.ptr(packed), _lib.ptr(scales), _lib.stream_ptr(w.device)
        )
    _lib.check(code, "quantize_weight")
    return packed, scales


def integer_gemm(a, sa, b, sb, bias, bits, tactic, residual=None, gate=None):
    """``robotics_integer::gemm`` call shape (reference: csrc/integer_gemm.cu:130-176).

    With `residual` [M, N] (bf16, contiguous) the epilogue writes the decoder layer's new residual
    stream instead of the projection: residual + y, or residual + y * gate[row // (M / B)] for a
    `gate` [B, N] (`rk_gemm_int_residual`; the same roundings as the tensor ops)."""
    if not (a.is_cuda and b.is_cuda and sa.is_cuda and sb.is_cuda):
        raise RuntimeError("integer GEMM operands must be CUDA tensors")
    if a.dim() != 2 or b.dim() != 2 or a.size(1) != b.size(1) or not a.is_contiguous() or not b.is_contiguous():
        raise RuntimeError("integer GEMM expects contiguous [M, K] and [N, K] operands with equal K")
    if sa.dtype != torch.float32 or sb.dtype != torch.float32 or sa.numel() != a.size(0) or sb.numel() != b.size(0):
        raise RuntimeError("integer GEMM scales must be float32 with one entry per row / channel")
    if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != b.size(0)):
        raise RuntimeError("integer GEMM bias must be BF16 with one entry per output channel")
    m, n = a.size(0), b.size(0)
    kpad = a.size(1) * (2 if bits == 4 else 1)
    out = torch.empty((m, n), device=a.device, dtype=torch.bfloat16)
    tokens = 1
    if residual is not None:
        if residual.dtype != torch.bfloat16 or tuple(residual.shape) != (m, n) or not residual.is_contiguous():
            raise RuntimeError("integer GEMM residual must be contiguous BF16 [M, N]")
        if gate is not None:
            if gate.dtype != torch.bfloat16 or gate.dim() != 2 or gate.size(1) != n or not gate.is_contiguous() \
                    or gate.size(0) < 1 or m % gate.size(0):
                raise RuntimeError("integer GEMM gate must be contiguous BF16 [B, N] with M divisible by B")
            tokens = m // gate.size(0)
    elif gate is not None:
        raise RuntimeError("integer GEMM: a gate needs a residual")
    with torch.cuda.device(a.device):
        ws = _lib.gemm_workspace(_lib.OP_W8A8 if bits == 8 else _lib.OP_W4A4, a.device, m, n, kpad)
        if residual is None:
            code = _lib.load().rk_gemm_int(
                _lib.ptr(a), _lib.ptr(sa), _lib.ptr(b), _lib.ptr(sb), _lib.ptr(bias), _lib.ptr(out),
                m, n, kpad, bits, tactic, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(a.device),
            )
        else:
            code = _lib.load().rk_gemm_int_residual(
                _lib.ptr(a), _lib.ptr(sa), _lib.ptr(b), _lib.ptr(sb), _lib.ptr(bias), _lib.ptr(residual), _lib.ptr(gate),
                tokens, _lib.ptr(out), m, n, kpad, bits, tactic, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(a.device),
            )
    if code == _lib.RK_EINVAL:
        raise RuntimeError(f"integer GEMM: {_lib.last_error()}")
    _lib.check(code, "integer GEMM")
    return out


class IntegerLinear(torch.nn.Module):
    def __init__(
        self, packed, scales, bias, in_features, out_features, bits, tactic=0, pack_reuse=False,
        biasless_epilogue=False,
    ):
        super().__init__()
        self.register_buffer("packed_weight", packed)
        self.register_buffer("weight_scale", scales)
        self.register_buffer("bias", bias)
        self.register_buffer(
            "_weight_descriptor", torch.empty(0, device=packed.device, dtype=torch.bfloat16), persistent=False
        )
        self.in_features = in_features
        self.out_features = out_features
        self.bits = bits
        self.tactic = tactic
        self.pack_reuse = pack_reuse
        self.biasless_epilogue = biasless_epilogue
        self.backend = BACKEND_FMT.format(bits=bits)
        _lib.load()

    @property
    def weight(self):
        return self._weight_descriptor

    @classmethod
    def from_linear(cls, linear, *, bits=8, tactic=0, pack_reuse=False, biasless_epilogue=False):
        if bits not in (4, 8) or not linear.weight.is_cuda or linear.weight.dtype != torch.bfloat16:
            raise ValueError("IntegerLinear requires CUDA BF16 weights and bits=4 or 8")
        _lib.load()
        w = linear.weight.detach()
        if not torch.isfinite(w).all():
            raise ValueError("Weights must be finite")
        n, k = w.shape
        npad = (n + 7) // 8 * 8
        packed, scales = quantize_weight(w, bits)
        bias = (
            None
            if linear.bias is None
            else torch.nn.functional.pad(linear.bias.detach().to(torch.bfloat16), (0, npad - n))
        )
        return cls(packed, scales, bias, k, n, bits, tactic, pack_reuse, biasless_epilogue)

    def pack_input(self, x):
        if getattr(x, "_robotics_packed_input", False):
            packed = x.for_bits(self.bits)
            if packed.logical_k != self.in_features:
                raise ValueError("Wrong prepared input feature count")
            return packed
        if x.shape[-1] != self.in_features:
            raise ValueError("Wrong input feature count")
        return prepare_activation(x, self.bits, pack_reuse=self.pack_reuse)

    def forward_packed(self, packed, residual=None, gate=None):
        """`residual` [..., out_features] (+ `gate` [B, out_features] or [B, 1, out_features]): the GEMM's
        epilogue returns the updated residual stream residual + y (* gate) instead of y."""
        if (
            packed.logical_k != self.in_features
            or packed.bits != self.bits
            or packed.format_version != "symmetric-row-v1"
        ):
            raise ValueError("Incompatible activation pack")
        if residual is not None:
            if self.out_features != self.packed_weight.shape[0]:
                raise ValueError("The residual epilogue needs out_features to be a multiple of 8")
            residual = residual.reshape(-1, self.out_features)
            residual = residual if residual.is_contiguous() else residual.contiguous()
            if gate is not None:
                gate = gate.reshape(-1, self.out_features)
                gate = gate if gate.is_contiguous() else gate.contiguous()
        # The reference's biasless epilogue skips the bias visitor; with a null bias the kernel's
        # epilogue is already that one, so both settings take the same path.
        output = integer_gemm(
            packed.data, packed.scales, self.packed_weight, self.weight_scale, self.bias, self.bits, self.tactic,
            residual=residual, gate=gate,
        )
        if self.out_features != output.shape[1]:
            output = output[:, : self.out_features].contiguous()
        return output.reshape(*packed.shape, self.out_features)

    def forward_gelu(self, x, up=None, *, approximate="tanh", residual=None, gate=None):
        if x.shape[-1] != self.in_features:
            raise ValueError("Wrong input feature count")
        return self.forward_packed(
            prepare_activation(x, self.bits, up=up, gelu=approximate, pack_reuse=self.pack_reuse),
            residual=residual, gate=gate,
        )

    def forward(self, x, residual=None, gate=None):
        return self.forward_packed(self.pack_input(x), residual=residual, gate=gate)


class IntegerProjectionGroup(torch.nn.Module):
    """Init-time packed concatenation; one GEMM per homogeneous sibling group
    (reference: integer.py:329-402)."""

    def __init__(self, linears, *, contiguous_outputs=True):
        super().__init__()
        if len(linears) < 2 or any(not isinstance(m, IntegerLinear) for m in linears):
            raise ValueError("At least two integer projections are required")
        first = linears[0]

        def signature(m):
            return (m.in_features, m.bits, m.tactic, m.pack_reuse, m.biasless_epilogue, m.packed_weight.device)

        if any(signature(m) != signature(first) for m in linears):
            raise ValueError("Projection format, input width, tactic and device must match")
        self.sizes = tuple(m.out_features for m in linears)
        self.contiguous_outputs = contiguous_outputs
        physical = [m.packed_weight.shape[0] for m in linears]
        self.offsets = tuple(sum(physical[:i]) for i in range(len(linears)))
        bias = None
        if any(m.bias is not None for m in linears):
            bias = torch.cat(
                [
                    m.bias
                    if m.bias is not None
                    else torch.zeros(m.packed_weight.shape[0], device=m.packed_weight.device, dtype=torch.bfloat16)
                    for m in linears
                ]
            )
        self.linear = IntegerLinear(
            torch.cat([m.packed_weight for m in linears]),
            torch.cat([m.weight_scale for m in linears]),
            bias,
            first.in_features,
            sum(physical),
            first.bits,
            first.tactic,
            first.pack_reuse,
            first.biasless_epilogue,
        )
        self._input = self._output = None
        self._remaining = set()

    def project(self, x, index):
        if self._input is not x or index not in self._remaining:
            self._input = x
            self._output = self.linear(x)
            self._remaining = set(range(len(self.sizes)))
        output = self._output.narrow(-1, self.offsets[index], self.sizes[index])
        if self.contiguous_outputs:
            output = output.contiguous()
        self._remaining.remove(index)
        if not self._remaining:
            self._input = self._output = None
        return output


class IntegerProjectionSlice(torch.nn.Module):
    def __init__(self, group, index):
        super().__init__()
        object.__setattr__(self, "_group", weakref.ref(group))
        self.index = index
        self.in_features = group.linear.in_features
        self.out_features = group.sizes[index]

    @property
    def weight(self):
        return self._group().linear.weight

    @property
    def bits(self):
        return self._group().linear.bits

    def forward(self, x):
        return self._group().project(x, self.index)
