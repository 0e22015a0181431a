"""Random-init Gemma-architecture stacks that host the quantized linears: the 2B VLM prefix pass
(18 layers, width 2048, 8 query heads / 1 KV head, head_dim 256, GeGLU MLP 16384) and the
action-expert flow-matching loop (18 layers, width 1024, MLP 4096, adaptive RMSNorm, chunk 50 x 32,
10 Euler steps over a cached prefix KV).

This is the caller side of the hot path: norms, RoPE, attention and residuals follow the reference's
owned runtime.  Attention is torch's fused scaled_dot_product_attention (bf16 flash arithmetic, which
differs from the reference's eager fp32 softmax in its rounding points) unless
``GemmaAttention.fused_attention`` routes the action expert through ``rk_attention_prefix``, which
reproduces the eager arithmetic (models/pi05/modeling_gemma.py:62-106,
126-128, 185-274, 315-443; models/pi05/modeling_pi05.py:673-720, 793-889).  Every bf16
``nn.Linear`` is a plain module so that ``quantize_linears`` can swap it; the fp32 adaptive-norm
``dense`` layers and the fp32 action projections stay unquantized, as in the reference
(optimizations/quantization.py:108-110).  Weights are random (N(0, 0.02)); there are no
checkpoints in this package.
"""

from dataclasses import dataclass
import math

import torch
from torch import nn
import torch.nn.functional as F


@dataclass(frozen=True)
class GemmaConfig:
    width: int
    mlp_dim: int
    depth: int = 18
    num_heads: int = 8
    num_kv_heads: int = 1
    head_dim: int = 256
    rms_eps: float = 1e-6
    rope_theta: float = 10000.0
    adarms_cond_dim: int | None = None


def gemma_2b():
    return GemmaConfig(width=2048, mlp_dim=16384)


def gemma_300m():
    return GemmaConfig(width=1024, mlp_dim=4096, adarms_cond_dim=1024)


class GemmaRMSNorm(nn.Module):
    """fp32 statistics; plain: x * inv * (1 + w); adaptive: x * inv * (1 + scale) + shift, gate.

    With `fused_bits` set (see `fuse_norm_quantize`) the norm, the modulation and the row quantizer
    of the integer linears that follow run as ONE kernel and the result is a packed-activation
    carrier instead of a bf16 tensor (the fusion the reference leaves open for Gemma:
    models/pi05/modeling_gemma.py:62-106 is a chain of torch ops in front of every quantizer)."""

    def __init__(self, dim, eps, cond_dim=None):
        super().__init__()
        self.eps = eps
        self.fused_bits = None
        self.fused_fp4 = None  # "global" / "block": hand NVFP4 packs (with / without a per-tensor scale) to the linears
        self.projection_cache = None  # a ConstantProjectionCache over `modulation` (see ActionExpert)
        if cond_dim is None:
            self.weight = nn.Parameter(torch.zeros(dim, dtype=torch.bfloat16))
            self.dense = None
        else:
            self.dense = nn.Linear(cond_dim, dim * 3, bias=True).float()  # stays fp32: never quantized

    def modulation(self, cond):
        """dense(cond) split into everything a forward needs: fp32 (scale, shift) [B, 1, K] for the
        unfused arithmetic, the bf16 gate [B, 1, K], and contiguous bf16 (scale, shift) [B, K] for
        the fused norm -> quantize kernel.  A function of `cond` alone, hence cacheable."""
        scale, shift, gate = self.dense(cond.float()).chunk(3, dim=-1)
        return (scale.unsqueeze(1), shift.unsqueeze(1), gate.unsqueeze(1).to(torch.bfloat16),
                scale.to(torch.bfloat16).contiguous(), shift.to(torch.bfloat16).contiguous())

    def forward(self, x, cond=None, pending=None):
        """Returns (normalized, gate, residual stream).  `pending` = (branch, gate) is a residual update
        that has not been applied yet: the stream becomes x + branch (* gate).  In the fused path the
        update, the norm, the modulation and the row quantizer are one kernel."""
        fused = self.fused_bits is not None and x.is_cuda and x.dtype == torch.bfloat16
        if self.dense is not None:
            project = self.projection_cache if self.projection_cache is not None else self.modulation
            scale, shift, gate, scale_bf16, shift_bf16 = project(cond)
        branch, branch_gate = pending if pending is not None else (None, None)
        if fused:
            from .modulation import prepare_rmsnorm

            x = x if x.is_contiguous() else x.contiguous()
            if branch is not None:
                branch = branch if branch.is_contiguous() else branch.contiguous()
            tokens = x.shape[1] if self.dense is not None else 0
            gate_rows = None
            if branch_gate is not None:
                if self.dense is None:  # a gate needs per-batch rows; apply it outside the kernel
                    branch, branch_gate = branch * branch_gate, None
                else:
                    gate_rows = branch_gate.reshape(-1, x.shape[-1])
            weight = self.weight.detach() if self.dense is None else scale_bf16
            result = prepare_rmsnorm(x, weight, self.fused_bits, eps=self.eps, residual=branch, gate=gate_rows,
                                     shift=None if self.dense is None else shift_bf16, tokens=tokens,
                                     return_sum=branch is not None)
            packed, stream = result if branch is not None else (result, x)
            return packed, (None if self.dense is None else gate), stream
        if self.fused_fp4 is not None and self.dense is None and x.is_cuda and x.dtype == torch.bfloat16:
            from .fp4_linear import gemma_rms_norm_pack_nvfp4

            if branch is not None and branch_gate is not None:
                branch = branch * branch_gate
            x = x if x.is_contiguous() else x.contiguous()
            if branch is not None and not branch.is_contiguous():
                branch = branch.contiguous()
            packed, stream = gemma_rms_norm_pack_nvfp4(x, self.weight.detach(), self.eps, residual=branch,
                                                       global_scale=self.fused_fp4 == "global")
            return packed, None, stream
        if branch is not None:
            x = x + branch if branch_gate is None else x + branch * branch_gate
        xf = x.float()
        normed = xf * torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + self.eps)
        if self.dense is None:
            return (normed * (1.0 + self.weight.float())).to(x.dtype), None, x
        return (normed * (1.0 + scale) + shift).to(x.dtype), gate.to(x.dtype), x


def _leading_shape(x):
    """Shape without the feature axis, for a tensor or a packed-activation carrier."""
    if getattr(x, "_robotics_packed_input", False):
        leading = getattr(x, "leading_shape", None)
        return tuple(leading) if leading is not None else tuple(next(iter(x.packs.values())).shape)
    return tuple(x.shape[:-1])


def rotate_half(x):
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def rope_tables(positions, head_dim, theta, dtype):
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=positions.device, dtype=torch.float32) / head_dim))
    angles = positions.float()[..., None] * inv_freq
    emb = torch.cat((angles, angles), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rope_cache_update(q, k, v, cos, sin, k_all, v_all, prefix, heads, kv_heads, head_dim, token_major=False,
                      vt_all=None):
    """One kernel for rotary embedding + cache append (`rk_rope_cache_update`).  q, k, v: bf16
    [B, t, heads * d] / [B, t, kv_heads * d] whose rows are dense (slices of one projection output
    are fine); cos, sin [B, t, d]; k_all, v_all [B, kv_heads, rows, d] already holding `prefix`
    rows.  Returns the rotated queries as [B, heads, t, d]; with `token_major` that tensor is a
    transposed view of [B, t, heads, d] storage, the layout fused attention reads without a copy.
    `vt_all` [B, kv_heads, d, pitch]: the fresh values are also written transposed (`attention_prefix`)."""
    from . import _lib

    b, t = q.shape[0], q.shape[1]
    for name, tensor in (("q", q), ("k", k), ("v", v)):
        if tensor.dtype != torch.bfloat16 or tensor.stride(-1) != 1 or tensor.stride(0) != t * tensor.stride(1):
            raise ValueError(f"{name} must be bf16 rows of one [B * t, width] matrix")
    cos, sin = cos.contiguous(), sin.contiguous()
    if not (k_all.is_contiguous() and v_all.is_contiguous()):
        raise ValueError("cache buffers must be contiguous")
    shape = (b, t, heads, head_dim) if token_major else (b, heads, t, head_dim)
    q_out = torch.empty(shape, dtype=torch.bfloat16, device=q.device)
    args = (_lib.ptr(q), q.stride(1), _lib.ptr(k), k.stride(1), _lib.ptr(v), v.stride(1), _lib.ptr(cos), _lib.ptr(sin),
            b, t, heads, kv_heads, head_dim, _lib.ptr(q_out), 1 if token_major else 0, _lib.ptr(k_all), _lib.ptr(v_all),
            k_all.shape[2], prefix)
    if vt_all is None:
        code = _lib.load().rk_rope_cache_update(*args, _lib.stream_ptr(q.device))
    else:
        if not vt_all.is_contiguous():
            raise ValueError("the transposed value cache must be contiguous")
        code = _lib.load().rk_rope_cache_update_vt(*args, _lib.ptr(vt_all), vt_all.shape[-1], _lib.stream_ptr(q.device))
    _lib.check(code, "rk_rope_cache_update")
    return q_out.transpose(1, 2) if token_major else q_out


def attention_prefix(q, k_all, vt_all, kv_len, scaling=None):
    """Fresh query tokens over cached keys / values in one kernel (`rk_attention_prefix`): the arithmetic
    of the reference's eager attention (models/pi05/modeling_gemma.py:247-274).  q bf16 [B, t, heads, 256]
    contiguous (token major); k_all [B, kv_heads, rows, 256]; vt_all [B, kv_heads, 256, pitch] (values
    transposed, finite beyond `kv_len`).  Returns bf16 [B, t, heads * 256]."""
    from . import _lib

    b, t, heads, d = q.shape
    if q.dtype != torch.bfloat16 or not (q.is_contiguous() and k_all.is_contiguous() and vt_all.is_contiguous()):
        raise ValueError("attention_prefix takes contiguous bf16 tensors")
    out = torch.empty((b, t, heads * d), dtype=torch.bfloat16, device=q.device)
    with torch.cuda.device(q.device):
        ws = _lib.workspace(q.device, _lib.WORKSPACE_HEADER)
        code = _lib.load().rk_attention_prefix(
            _lib.ptr(q), _lib.ptr(k_all), _lib.ptr(vt_all), _lib.ptr(out), b, t, heads, k_all.shape[1], d, k_all.shape[2],
            vt_all.shape[-1], kv_len, float(d ** -0.5 if scaling is None else scaling), _lib.ptr(ws), ws.numel(),
            _lib.stream_ptr(q.device))
    _lib.check(code, "rk_attention_prefix")
    return out


class GemmaAttention(nn.Module):
    fused_rope = False  # set on an instance (or the class) to route rope + cache append through one kernel
    fused_attention = False  # with fused_rope and a transposed value cache: attention as one tcgen05 kernel

    def __init__(self, cfg):
        super().__init__()
        self.cfg = cfg
        self.q_proj = nn.Linear(cfg.width, cfg.num_heads * cfg.head_dim, bias=False)
        self.k_proj = nn.Linear(cfg.width, cfg.num_kv_heads * cfg.head_dim, bias=False)
        self.v_proj = nn.Linear(cfg.width, cfg.num_kv_heads * cfg.head_dim, bias=False)
        self.o_proj = nn.Linear(cfg.num_heads * cfg.head_dim, cfg.width, bias=False)

    def _project_out(self, out, residual):
        """o_proj; with `residual` = (stream, gate) its epilogue returns stream + o (* gate) (integer layers only)."""
        if residual is None:
            return self.o_proj(out)
        return self.o_proj(out, residual=residual[0], gate=residual[1])

    def forward(self, x, cos, sin, past_kv=None, residual=None):
        b, t = _leading_shape(x)
        cfg = self.cfg
        if self.fused_rope and past_kv is not None and len(past_kv) >= 3 and cos.is_cuda:
            k_all, v_all, prefix = past_kv[:3]
            vt_all = past_kv[3] if len(past_kv) > 3 and self.fused_attention and cfg.head_dim == 256 else None
            q = rope_cache_update(self.q_proj(x), self.k_proj(x), self.v_proj(x), cos, sin, k_all, v_all, prefix,
                                  cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, token_major=True, vt_all=vt_all)
            if vt_all is not None:
                # q is a transposed view of token-major storage: hand the storage to the kernel
                out = attention_prefix(q.transpose(1, 2), k_all, vt_all, prefix + t)
                return self._project_out(out, residual), (k_all, v_all)
            out = F.scaled_dot_product_attention(q, k_all, v_all, is_causal=False, enable_gqa=True)
            out = out.transpose(1, 2).reshape(b, t, -1).contiguous()
            return self._project_out(out, residual), (k_all, v_all)
        q = self.q_proj(x).view(b, t, cfg.num_heads, cfg.head_dim).transpose(1, 2)
        k = self.k_proj(x).view(b, t, cfg.num_kv_heads, cfg.head_dim).transpose(1, 2)
        v = self.v_proj(x).view(b, t, cfg.num_kv_heads, cfg.head_dim).transpose(1, 2)
        q = q * cos[:, None] + rotate_half(q) * sin[:, None]
        k = k * cos[:, None] + rotate_half(k) * sin[:, None]
        if past_kv is not None and len(past_kv) >= 3:
            # preallocated [B, kv_heads, prefix + t, head_dim] buffers whose first `prefix` rows already
            # hold the cached keys / values: only the t new rows are written (ActionExpert.forward)
            k_all, v_all, prefix = past_kv[:3]
            k_all[:, :, prefix:prefix + t] = k
            v_all[:, :, prefix:prefix + t] = v
            k, v = k_all, v_all
        elif past_kv is not None:
            k = torch.cat([past_kv[0], k], dim=2)
            v = torch.cat([past_kv[1], v], dim=2)
        present = (k, v)
        # full (non-causal) visibility: prefix tokens see each other; suffix tokens see the whole
        # prefix and each other (models/pi05/modeling_pi05.py:649,662,713).  Grouped-query attention
        # goes through the fused kernel, which reads each key/value head once instead of
        # materialising one copy per query head.
        out = F.scaled_dot_product_attention(q, k, v, is_causal=False, enable_gqa=True)
        out = out.transpose(1, 2).reshape(b, t, -1).contiguous()
        return self._project_out(out, residual), present


class GemmaMLP(nn.Module):
    fused_gate_up = None  # an `Fp4GateUpGelu` built from gate_proj / up_proj (see `build_fused_gate_up_fp4`), or None

    def __init__(self, cfg):
        super().__init__()
        self.gate_proj = nn.Linear(cfg.width, cfg.mlp_dim, bias=False)
        self.up_proj = nn.Linear(cfg.width, cfg.mlp_dim, bias=False)
        self.down_proj = nn.Linear(cfg.mlp_dim, cfg.width, bias=False)

    def forward(self, x, residual=None):
        """`residual` = (stream, gate): the down projection's epilogue returns stream + mlp (* gate)."""
        if self.fused_gate_up is not None and residual is None:
            return self.fused_gate_up.forward_into(self.down_proj, x)  # one GEMM for gate and up, GELU * up in its epilogue
        gate, up = self.gate_proj(x), self.up_proj(x)
        fused = getattr(self.down_proj, "forward_gelu", None)
        if residual is not None:
            return fused(gate, up, residual=residual[0], gate=residual[1])
        if fused is not None:  # quantized down_proj: GELU(gate) * up fused into its row quantizer
            return fused(gate, up)
        return self.down_proj(F.gelu(gate, approximate="tanh") * up)


class GemmaLayer(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.self_attn = GemmaAttention(cfg)
        self.mlp = GemmaMLP(cfg)
        self.input_layernorm = GemmaRMSNorm(cfg.width, cfg.rms_eps, cfg.adarms_cond_dim)
        self.post_attention_layernorm = GemmaRMSNorm(cfg.width, cfg.rms_eps, cfg.adarms_cond_dim)

    def forward(self, x, cos, sin, past_kv=None, cond=None, pending=None):
        """`pending`: the previous layer's MLP branch and gate, not yet added to the stream.  Returns the
        stream BEFORE this layer's own MLP update plus that update as the new `pending`, so that the
        next norm can apply it inside its kernel (a norm without the fused path applies it eagerly;
        the arithmetic - bf16(x + bf16(branch * gate)) - is the same either way)."""
        if self.residual_epilogue and x.is_cuda and self._integer_out_projections():
            # the o_proj and down_proj GEMMs write the updated stream themselves (`rk_gemm_int_residual`):
            # nothing is pending between layers and the norms read one tensor
            h, gate, x = self.input_layernorm(x, cond, pending)
            x, present = self.self_attn(h, cos, sin, past_kv, residual=(x, gate))
            h, gate2, x = self.post_attention_layernorm(x, cond, None)
            return self.mlp(h, residual=(x, gate2)), present, None
        h, gate, x = self.input_layernorm(x, cond, pending)
        h, present = self.self_attn(h, cos, sin, past_kv)
        h, gate2, x = self.post_attention_layernorm(x, cond, (h, gate))
        h = self.mlp(h)
        return x, present, (h, gate2)

    # set on an instance (or the class): apply the residual updates in the epilogues of the integer o_proj / down_proj
    # GEMMs instead of inside the next norm kernel (the same arithmetic; the reference's torch ops either way)
    residual_epilogue = False

    def _integer_out_projections(self):
        from .integer import IntegerLinear

        return all(isinstance(m, IntegerLinear) and m.out_features == m.packed_weight.shape[0]
                   for m in (self.self_attn.o_proj, self.mlp.down_proj))


class GemmaStack(nn.Module):
    """`depth` decoder layers plus the final norm; layer names end in ``layers.<i>.<...>``."""

    def __init__(self, cfg):
        super().__init__()
        self.cfg = cfg
        self.layers = nn.ModuleList([GemmaLayer(cfg) for _ in range(cfg.depth)])
        self.norm = GemmaRMSNorm(cfg.width, cfg.rms_eps, cfg.adarms_cond_dim)

    @torch.no_grad()
    def init_random(self, seed=0, std=0.02):
        gen = torch.Generator(device="cpu").manual_seed(seed)
        for param in self.parameters():
            if param.dim() >= 2:
                param.copy_((torch.randn(param.shape, generator=gen) * std).to(param.dtype))
        return self

    def forward(self, x, positions, past=None, cond=None):
        cos, sin = rope_tables(positions, self.cfg.head_dim, self.cfg.rope_theta, x.dtype)
        presents = []
        pending = None
        for index, layer in enumerate(self.layers):
            x, present, pending = layer(x, cos, sin, None if past is None else past[index], cond, pending)
            presents.append(present)
        x, _, _ = self.norm(x, cond, pending)
        return x, presents


def build_prefix_model(device, seed=0):
    """The 2B VLM backbone of the prefix pass: embeddings [B, 816, 2048] in, hidden states and KV out."""
    model = GemmaStack(gemma_2b()).to(torch.bfloat16).init_random(seed)
    return model.to(device).eval()


def sinusoidal_time_embedding(time, dimension, min_period=4e-3, max_period=4.0):
    fraction = torch.linspace(0.0, 1.0, dimension // 2, dtype=torch.float64, device=time.device)
    period = min_period * (max_period / min_period) ** fraction
    angles = (1.0 / period * 2 * math.pi)[None, :] * time.double()[:, None]
    return torch.cat([torch.sin(angles), torch.cos(angles)], dim=1)


class ActionExpert(nn.Module):
    """Flow-matching action expert: `steps` Euler steps of an 18-layer Gemma stack over `chunk`
    action tokens that attend to a cached prefix KV (models/pi05/modeling_pi05.py:793-889)."""

    def __init__(self, cfg=None, chunk=50, action_dim=32, steps=10):
        super().__init__()
        self.cfg = cfg or gemma_300m()
        self.chunk, self.action_dim, self.steps = chunk, action_dim, steps
        self.stack = GemmaStack(self.cfg).to(torch.bfloat16)
        for layer in list(self.stack.layers) + [self.stack]:
            for norm in (getattr(layer, "input_layernorm", None), getattr(layer, "post_attention_layernorm", None),
                         getattr(layer, "norm", None)):
                if norm is not None and norm.dense is not None:
                    norm.dense.float()
        width = self.cfg.width
        self.action_in_proj = nn.Linear(action_dim, width).float()
        self.time_mlp_in = nn.Linear(width, width).float()
        self.time_mlp_out = nn.Linear(width, width).float()
        self.action_out_proj = nn.Linear(width, action_dim).float()
        self._conditions = None  # (steps, step, batch, device) -> condition, see enable_condition_caches

    @torch.no_grad()
    def init_random(self, seed=0, std=0.02):
        gen = torch.Generator(device="cpu").manual_seed(seed)
        for param in self.parameters():
            if param.dim() >= 2:
                param.copy_((torch.randn(param.shape, generator=gen) * std).to(param.dtype))
        return self

    def adaptive_norms(self):
        return [m for m in self.stack.modules() if isinstance(m, GemmaRMSNorm) and m.dense is not None]

    def enable_condition_caches(self, projections=True):
        """The reference's `condition_cache` / `condition_projection_cache` switches
        (optimizations/pi05.py:273-333): the timestep condition of step i of an n-step schedule
        depends on nothing but (n, i), so it is computed once per (schedule, step, batch, device)
        and - with `projections` - every adaptive norm's dense(condition) is computed once per such
        condition.  Later calls, CUDA-graph captures included, read them as constants."""
        from .optimizations.constant_projection import ConstantProjectionCache

        self._conditions = {}
        eligible = lambda cond: any(cond is kept for kept in self._conditions.values())
        for norm in self.adaptive_norms():
            norm.projection_cache = ConstantProjectionCache(norm.modulation, eligible) if projections else None
        return self

    def disable_condition_caches(self):
        self._conditions = None
        for norm in self.adaptive_norms():
            norm.projection_cache = None

    def retained_tensors(self):
        kept = list((self._conditions or {}).values())
        for norm in self.adaptive_norms():
            if norm.projection_cache is not None:
                kept.extend(norm.projection_cache.retained_tensors())
        return tuple(kept)

    def condition(self, time, step=None):
        compute = lambda: F.silu(self.time_mlp_out(F.silu(self.time_mlp_in(
            sinusoidal_time_embedding(time, self.cfg.width).float()))))
        if self._conditions is None or step is None:
            return compute()
        key = (self.steps, step, time.shape[0], time.device)
        if key not in self._conditions:
            self._conditions[key] = compute()
        return self._conditions[key]

    def denoise_step(self, x_t, time, prefix_kv, prefix_len, step=None):
        b = x_t.shape[0]
        cond = self.condition(time, step)
        tokens = self.action_in_proj(x_t).to(torch.bfloat16)
        positions = prefix_len + torch.arange(self.chunk, device=x_t.device)[None, :].expand(b, -1)
        hidden, _ = self.stack(tokens, positions, past=prefix_kv, cond=cond)
        return self.action_out_proj(hidden.float())

    def forward(self, noise, prefix_k, prefix_v):
        """noise [B, chunk, action_dim] fp32; prefix_k / prefix_v [depth, B, kv_heads, T, head_dim] bf16."""
        b = noise.shape[0]
        depth, _, kv_heads, prefix_len, head_dim = prefix_k.shape
        # one key and one value buffer per layer for the whole chunk: the prefix rows are copied in
        # once, every denoise step then overwrites only its `chunk` suffix rows (instead of
        # concatenating prefix and suffix anew in every layer of every step)
        shape = (depth, b, kv_heads, prefix_len + self.chunk, head_dim)
        k_all = torch.empty(shape, dtype=prefix_k.dtype, device=prefix_k.device)
        v_all = torch.empty(shape, dtype=prefix_v.dtype, device=prefix_v.device)
        k_all[:, :, :, :prefix_len] = prefix_k
        v_all[:, :, :, :prefix_len] = prefix_v
        if GemmaAttention.fused_attention and GemmaAttention.fused_rope and noise.is_cuda and head_dim == 256:
            # the attention kernel reads the values transposed (keys contiguous): the prefix is
            # transposed once per chunk, every step appends its rows as columns
            pitch = (prefix_len + self.chunk + 7) // 8 * 8
            vt_all = torch.zeros((depth, b, kv_heads, head_dim, pitch), dtype=prefix_v.dtype, device=prefix_v.device)
            vt_all[..., :prefix_len] = prefix_v.transpose(-1, -2)
            prefix_kv = [(k_all[i], v_all[i], prefix_len, vt_all[i]) for i in range(depth)]
        else:
            prefix_kv = [(k_all[i], v_all[i], prefix_len) for i in range(depth)]
        dt = -1.0 / self.steps
        x_t = noise
        for step in range(self.steps):
            time = torch.full((b,), 1.0 + step * dt, device=noise.device, dtype=torch.float32)
            x_t = x_t + dt * self.denoise_step(x_t, time, prefix_kv, prefix_len, step)
        return x_t


def fuse_norm_quantize(stack, bits=8):
    """Turns on the one-kernel norm -> quantize path for every layer norm whose consumers are all
    integer linears of `bits` (call it inside the `quantize_linears` context; returns the norms it
    switched so that the caller can switch them back with `unfuse_norm_quantize`)."""
    from .integer import IntegerLinear, IntegerProjectionSlice

    def integer(module):
        return isinstance(module, (IntegerLinear, IntegerProjectionSlice)) and getattr(module, "bits", bits) == bits

    switched = []
    for layer in stack.layers:
        attn, mlp = layer.self_attn, layer.mlp
        if all(integer(m) for m in (attn.q_proj, attn.k_proj, attn.v_proj)):
            layer.input_layernorm.fused_bits = bits
            switched.append(layer.input_layernorm)
        if all(integer(m) for m in (mlp.gate_proj, mlp.up_proj)):
            layer.post_attention_layernorm.fused_bits = bits
            switched.append(layer.post_attention_layernorm)
    return switched


def unfuse_norm_quantize(norms):
    for norm in norms:
        norm.fused_bits = None
        norm.fused_fp4 = None


def build_fused_gate_up_fp4(stack, global_scale=True):
    """One `Fp4GateUpGelu` per layer from the bf16 gate / up linears (call it BEFORE `quantize_linears` swaps them).
    Returns the modules; `enable_fused_gate_up` switches a stack over to them, `disable_fused_gate_up` back."""
    from .fp4_linear import Fp4GateUpGelu

    return [Fp4GateUpGelu.from_linears(layer.mlp.gate_proj, layer.mlp.up_proj, global_scale=global_scale)
            for layer in stack.layers]


def enable_fused_gate_up(stack, fused_modules):
    from .fp4_linear import Fp4CutlassLinear

    for layer, fused in zip(stack.layers, fused_modules):
        if not isinstance(layer.mlp.down_proj, Fp4CutlassLinear):
            raise ValueError("the fused gate/up projection feeds an NVFP4 down projection: quantize the stack first")
        layer.mlp.fused_gate_up = fused


def disable_fused_gate_up(stack):
    for layer in stack.layers:
        layer.mlp.fused_gate_up = None


def fuse_norm_pack_fp4(stack):
    """The NVFP4 counterpart of `fuse_norm_quantize`: every plain (non-adaptive) layer norm whose
    consumers are all `Fp4CutlassLinear` layers with the same per-tensor-scale setting hands them
    one packed activation (add + norm + amax in one kernel, then the block packer).  Call it inside
    the `quantize_linears` context; undo with `unfuse_norm_quantize`."""
    from .fp4_linear import Fp4CutlassLinear

    def mode(modules):
        if not all(isinstance(m, Fp4CutlassLinear) for m in modules):
            return None
        kinds = {m.weight_global_scale is None for m in modules}
        return None if len(kinds) != 1 else ("block" if kinds.pop() else "global")

    switched = []
    for layer in stack.layers:
        attn, mlp = layer.self_attn, layer.mlp
        for norm, consumers in ((layer.input_layernorm, (attn.q_proj, attn.k_proj, attn.v_proj)),
                                (layer.post_attention_layernorm, (mlp.gate_proj, mlp.up_proj))):
            kind = mode(consumers)
            if kind is not None and norm.dense is None:
                norm.fused_fp4 = kind
                switched.append(norm)
    return switched


def expert_scope(name):
    """Selector for `quantize_linears`: the bf16 linears of the decoder layers are "expert"."""
    return "expert" if ".layers." in name and ".dense" not in name else None


def prefix_scope(name):
    return "text" if name.startswith("layers.") or ".layers." in name else None
