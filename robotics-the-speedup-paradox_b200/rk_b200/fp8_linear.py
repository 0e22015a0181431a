"""FP8 Linear on the B200 tcgen05 kernels: per-tensor E4M3 (``kind::f8f6f4``) and MXFP8
(E4M3 with one UE8M0 scale per 32 k, ``kind::mxf8f6f4.block_scale``).

Host-side mirror of the reference's ``src/robotics_kernels/blackwell/fp8_linear.py``
(``Fp8CutlassLinear``: ``from_linear(linear, role, target_name)``, ``pack_input``,
``forward_packed``, ``forward_mxfp8``, ``forward``, ``fp8_backend``, status helpers) and of
``mxfp8_linear.py`` (``pack`` / ``linear``).  The reference reaches MXFP8 only for a few prefill
roles chosen by environment variables (fp8_linear.py:30,565); here it is a mode of the module.
Arithmetic runs in ``librk_b200.so``; there is no fallback.
"""

from dataclasses import dataclass
import os

import torch

from . import _lib

FP8_DTYPE = torch.float8_e4m3fn
PREFILL_SCALE_REFRESH_INTERVAL_ENV = "ROBOTICS_FP8_PREFILL_SCALE_REFRESH_INTERVAL"
# roles whose multi-row (prefill) calls may keep an activation scale for several calls
PERIODIC_PREFILL_SCALE_ROLES = frozenset(
    {"attn_q", "attn_k", "attn_v", "attn_qkv", "attn_o", "mlp_gate", "mlp_up", "mlp_gate_up", "mlp_down"})
_NEVER = 2 ** 31 - 1


@dataclass
class Fp8BackendStatus:
    available: bool
    error: str | None
    backend: str = "b200_tcgen05_e4m3"

    def to_dict(self):
        return {"available": self.available, "error": self.error, "backend": self.backend}


def fp8_backend_status(device=None):
    ok, error = _lib.backend_status()
    if ok and torch.cuda.is_available():
        major, minor = torch.cuda.get_device_capability(device)
        if not _lib.load().rk_supports_device(major, minor):
            ok, error = False, f"compute capability {major}.{minor} is not supported (sm_100 only)"
    elif ok:
        ok, error = False, "CUDA is not available"
    return Fp8BackendStatus(ok, error)


def require_fp8_backend(device=None):
    status = fp8_backend_status(device)
    if not status.available:
        raise RuntimeError(f"FP8 backend unavailable: {status.to_dict()}")


def _check_bf16(x, what):
    if not x.is_cuda or x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError(f"{what} must be a contiguous CUDA BF16 tensor")


# ---- per-tensor E4M3 -------------------------------------------------------------------------
def quantize_bf16(x):
    """-> (e4m3 tensor of x's shape, float32 scale[1]); scale = max(amax / 448, 1e-12)."""
    _check_bf16(x, "quantize_bf16 input")
    q = torch.empty(x.shape, device=x.device, dtype=FP8_DTYPE)
    scale = torch.empty(1, device=x.device, dtype=torch.float32)
    with torch.cuda.device(x.device):
        ws = _lib.workspace(x.device, _lib.WORKSPACE_HEADER)
        code = _lib.load().rk_quant_tensor_fp8(_lib.ptr(x), x.numel(), _lib.ptr(q), _lib.ptr(scale), _lib.ptr(ws),
                                               ws.numel(), _lib.stream_ptr(x.device))
    _lib.check(code, "quantize_bf16")
    return q, scale


def quantize_bf16_with_scale(x, scale):
    _check_bf16(x, "quantize_bf16_with_scale input")
    q = torch.empty(x.shape, device=x.device, dtype=FP8_DTYPE)
    with torch.cuda.device(x.device):
        code = _lib.load().rk_quant_tensor_fp8_with_scale(_lib.ptr(x), x.numel(), _lib.ptr(scale), _lib.ptr(q),
                                                          _lib.stream_ptr(x.device))
    _lib.check(code, "quantize_bf16_with_scale")
    return q


def add_rms_norm_quantize_bf16(x, residual, weight, epsilon):
    """(residual add +) RMSNorm -> per-tensor E4M3: -> (summed, normalized, e4m3 codes, float32 scale[1]).

    Mirrors `robotics_cutlass_fp8::add_rms_norm_quantize_bf16` (blackwell/csrc/fp8_cutlass_linear.cu:913-960):
    x, residual bf16 [rows, K] (residual may be None: then `summed` is x itself), weight bf16 [K]."""
    _check_bf16(x, "add_rms_norm_quantize_bf16 input")
    if x.dim() != 2 or x.shape[1] % 16:
        raise ValueError("add_rms_norm_quantize_bf16 requires [rows, K] with K divisible by 16")
    if residual is not None:
        _check_bf16(residual, "add_rms_norm_quantize_bf16 residual")
        if residual.shape != x.shape:
            raise ValueError("residual must have the shape of the input")
    _check_bf16(weight, "add_rms_norm_quantize_bf16 weight")
    if weight.shape != (x.shape[1],):
        raise ValueError("weight must have one entry per column")
    rows, k = x.shape
    summed = torch.empty_like(x) if residual is not None else x
    normalized = torch.empty_like(x)
    q = torch.empty(x.shape, device=x.device, dtype=FP8_DTYPE)
    scale = torch.empty(1, device=x.device, dtype=torch.float32)
    with torch.cuda.device(x.device):
        ws = _lib.workspace(x.device, _lib.WORKSPACE_HEADER)
        code = _lib.load().rk_rmsnorm_quant_fp8(_lib.ptr(x), _lib.ptr(residual), _lib.ptr(weight), rows, k, float(epsilon),
                                                _lib.ptr(summed) if residual is not None else None, _lib.ptr(normalized),
                                                _lib.ptr(q), _lib.ptr(scale), _lib.ptr(ws), ws.numel(),
                                                _lib.stream_ptr(x.device))
    _lib.check(code, "add_rms_norm_quantize_bf16")
    return summed, normalized, q, scale


def quantize_swiglu_bf16(gate_up, intermediate_size, scale=None):
    """SiLU(gate) * up -> per-tensor E4M3: gate_up bf16 [rows, 2 * intermediate_size] (gate first).
    -> (e4m3 [rows, intermediate_size], float32 scale[1]); `scale` given = `quantize_swiglu_bf16_with_scale`
    (blackwell/csrc/fp8_cutlass_linear.cu:962-1009)."""
    _check_bf16(gate_up, "quantize_swiglu_bf16 input")
    inter = int(intermediate_size)
    if gate_up.dim() != 2 or gate_up.shape[1] != 2 * inter or inter % 16:
        raise ValueError("quantize_swiglu_bf16 requires [rows, 2 * intermediate_size], intermediate_size divisible by 16")
    rows = gate_up.shape[0]
    q = torch.empty((rows, inter), device=gate_up.device, dtype=FP8_DTYPE)
    out_scale = scale if scale is not None else torch.empty(1, device=gate_up.device, dtype=torch.float32)
    with torch.cuda.device(gate_up.device):
        ws = _lib.workspace(gate_up.device, _lib.WORKSPACE_HEADER)
        code = _lib.load().rk_swiglu_quant_fp8(_lib.ptr(gate_up), rows, inter, _lib.ptr(scale), _lib.ptr(q),
                                               _lib.ptr(out_scale), _lib.ptr(ws), ws.numel(),
                                               _lib.stream_ptr(gate_up.device))
    _lib.check(code, "quantize_swiglu_bf16")
    return q, out_scale


def quantize_swiglu_bf16_with_scale(gate_up, intermediate_size, scale):
    return quantize_swiglu_bf16(gate_up, intermediate_size, scale)[0]


def linear_forward_packed(a, scale_a, b, scale_b, bias=None, tactic=0):
    """e4m3 [M, K] x e4m3 [N, K]^T -> bf16 [M, N] = bf16(scale_a * scale_b * acc + bias)."""
    m, k = a.shape
    n = b.shape[0]
    out = torch.empty((m, n), device=a.device, dtype=torch.bfloat16)
    with torch.cuda.device(a.device):
        ws = _lib.gemm_workspace(_lib.OP_FP8, a.device, m, n, k)
        code = _lib.load().rk_gemm_fp8(_lib.ptr(a), _lib.ptr(scale_a), _lib.ptr(b), _lib.ptr(scale_b), _lib.ptr(bias),
                                       _lib.ptr(out), m, n, k, tactic, _lib.ptr(ws), ws.numel(),
                                       _lib.stream_ptr(a.device))
    _lib.check(code, "linear_forward_packed")
    return out


def linear_forward_producer(x, weight, weight_scale, bias=None, tactic=0):
    """bf16 [M, K] x e4m3 [N, K]^T with a unit activation scale: the activations are converted to e4m3
    inside the GEMM kernel (`rk_gemm_fp8_producer`), no quantizer launch and no e4m3 copy in memory."""
    _check_bf16(x, "linear_forward_producer input")
    m, k = x.shape
    n = weight.shape[0]
    out = torch.empty((m, n), device=x.device, dtype=torch.bfloat16)
    with torch.cuda.device(x.device):
        ws = _lib.gemm_workspace(_lib.OP_FP8, x.device, m, n, k)
        code = _lib.load().rk_gemm_fp8_producer(_lib.ptr(x), _lib.ptr(weight), _lib.ptr(weight_scale), _lib.ptr(bias),
                                                _lib.ptr(out), m, n, k, tactic, _lib.ptr(ws), ws.numel(),
                                                _lib.stream_ptr(x.device))
    _lib.check(code, "linear_forward_producer")
    return out


# ---- periodic reuse of the dynamic activation scale ----------------------------------------------
def resolve_fp8_prefill_scale_refresh_interval(value=None):
    """How many prefill calls share one dynamic activation scale: a positive integer, or
    "static" / "once" / "never" for a scale measured on the first call only.  `None` reads
    ROBOTICS_FP8_PREFILL_SCALE_REFRESH_INTERVAL (default 1 = a fresh scale on every call).
    Reference: blackwell/fp8_linear.py:90-115."""
    text = str(os.environ.get(PREFILL_SCALE_REFRESH_INTERVAL_ENV, "1") if value is None else value).strip().lower()
    if text in ("static", "once", "never"):
        return _NEVER
    try:
        interval = int(text)
    except ValueError as error:
        raise ValueError(f"{PREFILL_SCALE_REFRESH_INTERVAL_ENV} must be a positive integer or 'static'") from error
    if interval <= 0:
        raise ValueError(f"{PREFILL_SCALE_REFRESH_INTERVAL_ENV} must be positive")
    return interval


class Fp8PrefillScaleState:
    """Per-module memory of the last measured activation scale (reference: blackwell/fp8_linear.py:147-239).

    The per-tensor quantizer needs two passes over the activations because its scale is global: an
    amax reduction, then the conversion.  Between consecutive multi-row calls of one layer the
    amax moves little, so with an interval n > 1 only every n-th call measures (`refreshes`); the
    calls in between convert with the remembered scale in a single pass (`reuses`).  Single-row
    calls and ineligible roles always measure."""

    def __init__(self, interval=None, *, eligible=True):
        self.eligible = bool(eligible)
        self.configure(interval)

    def configure(self, interval=None):
        self.interval = resolve_fp8_prefill_scale_refresh_interval(interval) if self.eligible else 1
        self.scale = None
        self.prefill_calls = self.refreshes = self.reuses = self.operator_fallbacks = 0

    def enabled_for(self, tensor, columns):
        return self.interval > 1 and tensor.numel() // int(columns) > 1

    def _due(self):
        return self.scale is None or self.prefill_calls % self.interval == 0

    def _run(self, enabled, measure, convert):
        if not enabled:
            return measure()
        if self._due():
            packed, scale = measure()
            self.scale = scale
            self.refreshes += 1
        else:
            packed, scale = convert(self.scale), self.scale
            self.reuses += 1
        self.prefill_calls += 1
        return packed, scale

    def quantize(self, tensor):
        """-> (e4m3 codes, float32 scale[1]) of a contiguous bf16 tensor."""
        return self._run(self.enabled_for(tensor, tensor.shape[-1]), lambda: quantize_bf16(tensor),
                         lambda scale: quantize_bf16_with_scale(tensor, scale))

    def quantize_swiglu(self, gate_up, intermediate_size):
        inter = int(intermediate_size)
        return self._run(self.enabled_for(gate_up, 2 * inter), lambda: quantize_swiglu_bf16(gate_up, inter),
                         lambda scale: quantize_swiglu_bf16_with_scale(gate_up, inter, scale))

    def to_dict(self):
        return {"eligible": self.eligible, "interval": self.interval, "prefill_calls": self.prefill_calls,
                "refreshes": self.refreshes, "reuses": self.reuses, "operator_fallbacks": self.operator_fallbacks}


def _fp8_prefill_scale_states(model):
    states = {}
    for module in model.modules():
        state = getattr(module, "_prefill_scale_state", None)
        if isinstance(state, Fp8PrefillScaleState) and state.eligible:
            states[id(state)] = state
    return list(states.values())


def configure_fp8_prefill_scale_refresh(model, interval=None):
    """Sets the interval of every eligible layer of a loaded model and resets their counters."""
    states = _fp8_prefill_scale_states(model)
    if not states:
        return {"interval": 1, "states": 0}
    resolved = resolve_fp8_prefill_scale_refresh_interval(interval)
    for state in states:
        state.configure(resolved)
    return {"interval": resolved, "states": len(states)}


def fp8_prefill_scale_refresh_stats(model):
    states = _fp8_prefill_scale_states(model)
    totals = {"states": len(states), "prefill_calls": 0, "refreshes": 0, "reuses": 0, "operator_fallbacks": 0}
    for state in states:
        for key in ("prefill_calls", "refreshes", "reuses", "operator_fallbacks"):
            totals[key] += getattr(state, key)
    totals["intervals"] = sorted({state.interval for state in states})
    return totals


# ---- MXFP8 -----------------------------------------------------------------------------------
def mxfp8_pack(x):
    """bf16 [rows, K] -> (e4m3 [rows, K], uint8 swizzled UE8M0 scale buffer); K % 32 == 0."""
    _check_bf16(x, "mxfp8 pack input")
    if x.dim() != 2 or x.shape[1] % 32:
        raise ValueError("MXFP8 pack requires contiguous CUDA BF16 [M,K] with K divisible by 32")
    rows, k = x.shape
    lib = _lib.load()
    q = torch.empty((rows, k), device=x.device, dtype=FP8_DTYPE)
    sf = torch.empty(lib.rk_sf_bytes(rows, k // 32), device=x.device, dtype=torch.uint8)
    with torch.cuda.device(x.device):
        code = lib.rk_pack_mxfp8(_lib.ptr(x), rows, k, _lib.ptr(q), _lib.ptr(sf), _lib.stream_ptr(x.device))
    _lib.check(code, "mxfp8 pack")
    return q, sf


def mxfp8_linear(a, sfa, b, sfb, bias=None, tactic=0):
    m, k = a.shape
    n = b.shape[0]
    out = torch.empty((m, n), device=a.device, dtype=torch.bfloat16)
    with torch.cuda.device(a.device):
        ws = _lib.gemm_workspace(_lib.OP_MXFP8, a.device, m, n, k)
        code = _lib.load().rk_gemm_mxfp8(_lib.ptr(a), _lib.ptr(sfa), _lib.ptr(b), _lib.ptr(sfb), _lib.ptr(bias),
                                         _lib.ptr(out), m, n, k, tactic, _lib.ptr(ws), ws.numel(),
                                         _lib.stream_ptr(a.device))
    _lib.check(code, "mxfp8 linear")
    return out


class Fp8CutlassLinear(torch.nn.Module):
    """Quantized replacement of a BF16 ``nn.Linear``; ``mode`` is "per_tensor" or "mxfp8"."""

    def __init__(self, weight_q, weight_scale, bias, in_features, out_features, role, target_name, mode):
        super().__init__()
        self.register_buffer("packed_weight", weight_q)
        self.register_buffer("weight_scale", weight_scale)
        self.register_buffer("bias", bias)
        self.register_buffer("_weight_descriptor", torch.empty(0, device=weight_q.device, dtype=torch.bfloat16),
                             persistent=False)
        self.in_features = in_features
        self.out_features = out_features
        self.role = role
        self.target_name = target_name
        self.mode = mode
        self._unit_scale = None  # lazily created scalar 1.0 for the producer path
        self._prefill_scale_state = Fp8PrefillScaleState(eligible=mode == "per_tensor" and role in PERIODIC_PREFILL_SCALE_ROLES)
        self.fp8_backend = "b200_tcgen05_e4m3" if mode == "per_tensor" else "b200_tcgen05_mxfp8_e4m3_ue8m0"

    @classmethod
    def from_linear(cls, linear, role, target_name, mode="per_tensor"):
        if mode not in ("per_tensor", "mxfp8"):
            raise ValueError("mode must be per_tensor or mxfp8")
        if not linear.weight.is_cuda or linear.weight.dtype != torch.bfloat16:
            raise ValueError("Fp8CutlassLinear requires CUDA BF16 weights")
        require_fp8_backend(linear.weight.device)
        n, k = linear.weight.shape
        if n % 8 or k % (16 if mode == "per_tensor" else 32):
            raise ValueError("Fp8CutlassLinear requires out_features % 8 == 0 and in_features % 16 (32 for MXFP8) == 0")
        w = linear.weight.detach().contiguous()
        if mode == "per_tensor":
            weight_q, weight_scale = quantize_bf16(w)
        else:
            weight_q, weight_scale = mxfp8_pack(w)
        bias = None if linear.bias is None else linear.bias.detach().to(torch.bfloat16).contiguous()
        return cls(weight_q, weight_scale, bias, k, n, role, target_name, mode)

    @property
    def weight(self):
        return self._weight_descriptor

    def _rows(self, x):
        if x.shape[-1] != self.in_features:
            raise ValueError("Wrong input feature count")
        flat = x.reshape(-1, self.in_features)
        return flat if flat.is_contiguous() else flat.contiguous()

    def pack_input(self, x):
        flat = self._rows(x)
        return self._prefill_scale_state.quantize(flat) if self.mode == "per_tensor" else mxfp8_pack(flat)

    def forward_packed(self, packed, scale, shape=None):
        if self.mode == "per_tensor":
            out = linear_forward_packed(packed, scale, self.packed_weight, self.weight_scale, self.bias)
        else:
            out = mxfp8_linear(packed, scale, self.packed_weight, self.weight_scale, self.bias)
        return out if shape is None else out.reshape(*shape, self.out_features)

    def forward_swiglu(self, gate_up, intermediate_size, leading_shape):
        """SiLU * up, dynamic E4M3 packing and this (down) projection; gate_up [..., 2 * intermediate_size]
        (blackwell/fp8_linear.py:679-691 of the reference)."""
        if self.mode != "per_tensor":
            raise RuntimeError("forward_swiglu packs per-tensor E4M3; this layer was packed as MXFP8")
        if int(intermediate_size) != self.in_features:
            raise ValueError(f"expected intermediate_size {self.in_features}, got {intermediate_size}")
        flat = gate_up.to(torch.bfloat16).reshape(-1, 2 * self.in_features).contiguous()
        packed, scale = self._prefill_scale_state.quantize_swiglu(flat, self.in_features)
        return self.forward_packed(packed, scale, leading_shape)

    def forward_producer(self, x):
        """BF16 activations converted to E4M3 with a unit activation scale inside the GEMM's main loop: the
        semantics of `linear_forward_producer` (blackwell/csrc/fp8_cutlass_linear.cu:727-856, 1268-1315),
        which the reference uses for small projections to skip the dynamic activation scale and the
        quantizer pass.  One launch; the converted activations never reach global memory."""
        if self.mode != "per_tensor":
            raise RuntimeError("forward_producer is a per-tensor path; this layer was packed as MXFP8")
        flat = self._rows(x)
        out = linear_forward_producer(flat, self.packed_weight, self.weight_scale, self.bias)
        return out.reshape(*x.shape[:-1], self.out_features)

    def forward_mxfp8(self, x):
        if self.mode != "mxfp8":
            raise RuntimeError("This layer was packed per-tensor; build it with mode='mxfp8'")
        return self.forward(x)

    def forward(self, x):
        packed, scale = self.pack_input(x)
        return self.forward_packed(packed, scale, x.shape[:-1])

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, mode={self.mode}, role={self.role}"
