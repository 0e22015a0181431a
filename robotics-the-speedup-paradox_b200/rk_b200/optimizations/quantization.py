"""Model-specific selection above the precision backends: which ``nn.Linear`` modules are swapped
for quantized ones, how sibling projections share one activation pack or one GEMM, and how every
change is undone on exit.

Reference: optimizations/quantization.py:7-189.  Precisions ``int8`` / ``int4`` / ``fp8`` / ``fp4``
are the reference's; ``mxfp8`` and ``w4a16`` are added because this package ships those operators
as first-class Linear modules (the reference reaches them only through environment switches).
"""

from contextlib import contextmanager

from .patching import Patches

PRECISIONS = ("int8", "int4", "fp8", "fp4", "mxfp8", "w4a16")
SCOPES = ("text", "expert", "vision", "projector", "dit")


class ActivationCache:
    """Share one prepared activation among the `fanout` sibling projections that consume it."""

    def __init__(self, prepare, fanout):
        self.prepare = prepare
        self.fanout = fanout
        self.input = None
        self.packed = None
        self.remaining = 0

    def get(self, x):
        if self.remaining == 0 or self.input is not x:
            self.input, self.packed, self.remaining = x, self.prepare(x), self.fanout
        packed = self.packed
        self.remaining -= 1
        if self.remaining == 0:
            self.input = self.packed = None
        return packed


_PI05_MARKERS = (
    (".vision_model.encoder.layers.", "vision"),
    (".paligemma.model.language_model.layers.", "text"),
    (".gemma_expert.model.layers.", "expert"),
    (".multi_modal_projector.", "projector"),
)


def pi05_scope(name):
    """Scope of a pi0.5 module name, or None for modules that are never quantized (heads, action
    projections)."""
    for marker, scope in _PI05_MARKERS:
        if marker in name:
            return scope
    return None


def _factory(precision, *, tactic, pack_reuse, biasless_epilogue, site_bits, fp4_global_scale=False):
    if precision in ("int8", "int4"):
        from ..integer import IntegerLinear

        default_bits = 8 if precision == "int8" else 4

        def make(module, name):
            bits = site_bits[name] if site_bits is not None else default_bits
            return IntegerLinear.from_linear(module, bits=bits, tactic=tactic, pack_reuse=pack_reuse,
                                             biasless_epilogue=biasless_epilogue)
        return make
    if precision == "w4a16":
        from ..w4a16_linear import W4A16Linear

        return lambda module, name: W4A16Linear.from_linear(module, tactic=tactic)
    if precision in ("fp8", "mxfp8"):
        from ..fp8_linear import Fp8CutlassLinear

        mode = "per_tensor" if precision == "fp8" else "mxfp8"
        return lambda module, name: Fp8CutlassLinear.from_linear(module, role="linear", target_name=name, mode=mode)
    from ..fp4_linear import Fp4CutlassLinear

    return lambda module, name: Fp4CutlassLinear.from_linear(module, role="linear", target_name=name,
                                                             global_scale=fp4_global_scale)


def _backend_of(module):
    for attr in ("backend", "fp8_backend", "fp4_backend"):
        value = getattr(module, attr, None)
        if value is not None:
            return value
    return "unknown"


@contextmanager
def quantize_linears(model, precision, *, scopes=("text",), shared_quant=False, tactic=0, selector=pi05_scope,
                     grouped=False, pack_reuse=False, site_bits=None, group_qkv=False, group_gate_up=False,
                     group_views=False, biasless_epilogue=False, fp4_global_scale=False):
    """Swap every BF16 ``nn.Linear`` whose `selector(name)` is in `scopes`; yield a report; undo on exit.

    `fp4_global_scale` (precision "fp4" only): pack weights and activations with the fp32 per-tensor
    scale amax / (6 * 448) in front of the block scales; off reproduces the reference's format."""
    import torch

    if precision not in PRECISIONS:
        raise ValueError("Unknown low-precision backend")
    if not scopes or any(s not in SCOPES for s in scopes):
        raise ValueError("Explicit supported module scopes are required")
    if fp4_global_scale and precision != "fp4":
        raise ValueError("fp4_global_scale applies to the fp4 precision only")
    make = _factory(precision, tactic=tactic, pack_reuse=pack_reuse, biasless_epilogue=biasless_epilogue,
                    site_bits=site_bits, fp4_global_scale=fp4_global_scale)
    patches = Patches()
    report = {
        "precision": precision, "scopes": list(scopes), "modules": {}, "skipped": {}, "shared_quant": shared_quant,
        "tactic": tactic, "grouped": {}, "pack_reuse": pack_reuse, "biasless_epilogue": biasless_epilogue,
        "fp4_global_scale": fp4_global_scale,
    }
    try:
        swapped = 0
        for name, module in list(model.named_modules()):
            if not isinstance(module, torch.nn.Linear) or selector(name) not in scopes:
                continue
            if module.weight.dtype != torch.bfloat16:
                report["skipped"][name] = "Original parameter dtype is not BF16"
                continue
            parent_name, _, attr = name.rpartition(".")
            replacement = make(module, name)
            patches.set(model.get_submodule(parent_name), attr, replacement)
            report["modules"][name] = {"backend": _backend_of(replacement), "in_features": module.in_features,
                                       "out_features": module.out_features}
            swapped += 1
        if not swapped:
            raise ValueError("No eligible Linear modules in the selected scope")
        if grouped or group_qkv or group_gate_up:
            if not precision.startswith("int"):
                raise ValueError("Grouped projections currently support integer backends")
        if shared_quant or grouped or group_qkv or group_gate_up:
            if precision.startswith("int"):
                _share_siblings(model, patches, report, shared_quant=shared_quant, grouped=grouped, group_qkv=group_qkv,
                                group_gate_up=group_gate_up, group_views=group_views)
            elif precision in ("fp8", "mxfp8", "fp4"):
                _share_float_packs(model, patches, report)
            else:
                raise ValueError("Shared preparation supports the integer, fp8, mxfp8 and fp4 backends")
        yield report
    finally:
        patches.restore()


def _share_float_packs(model, patches, report):
    """fp8 / mxfp8 / fp4: the q/k/v and the gate/up projections of one parent read the same activation,
    so it is quantized (scale, codes, scale factors) once and the siblings run `forward_packed` on the
    shared result.  (The reference shares packs for its integer backends only; the operators are the
    same, this saves two of three packer launches per attention block and one of two per MLP.)"""
    from ..fp4_linear import Fp4CutlassLinear
    from ..fp8_linear import Fp8CutlassLinear

    shared = 0
    for module_name, module in list(model.named_modules()):
        for names in (("q_proj", "k_proj", "v_proj"), ("gate_proj", "up_proj")):
            members = [getattr(module, attr, None) for attr in names]
            members = [m for m in members if isinstance(m, (Fp4CutlassLinear, Fp8CutlassLinear))]
            if len(members) < 2 or len({(type(m), m.in_features, getattr(m, "mode", None)) for m in members}) != 1:
                continue
            if isinstance(members[0], Fp4CutlassLinear) and len({m.weight_global_scale is None for m in members}) != 1:
                continue
            cache = ActivationCache(members[0].pack_input, len(members))
            for layer in members:
                patches.bind(layer, "forward",
                             lambda self, x, cache=cache: self.forward_packed(*cache.get(x), shape=x.shape[:-1]))
            shared += 1
    report["shared_float_packs"] = shared


def _share_siblings(model, patches, report, *, shared_quant, grouped, group_qkv, group_gate_up, group_views):
    """Among the q/k/v and gate/up projections of one parent: fuse them into one GEMM (grouping
    switches) or let them share one activation pack (`shared_quant`)."""
    from ..integer import IntegerLinear, IntegerProjectionGroup, IntegerProjectionSlice

    for module_name, module in list(model.named_modules()):
        attention = ("q_proj", "k_proj", "v_proj") if getattr(module, "is_selfattn", True) else ("k_proj", "v_proj")
        for family, (names, fuse) in enumerate(((attention, grouped or group_qkv),
                                                (("gate_proj", "up_proj"), grouped or group_gate_up))):
            by_format = {}
            for attr in names:
                member = getattr(module, attr, None)
                if isinstance(member, IntegerLinear):
                    by_format.setdefault((member.bits, member.in_features), []).append((attr, member))
            for (bits, _), members in by_format.items():
                if len(members) < 2:
                    continue
                siblings = [layer for _, layer in members]
                if fuse:
                    group = IntegerProjectionGroup(siblings, contiguous_outputs=not group_views)
                    key = f"_robotics_integer_group_{family}_{bits}"
                    patches.set(module, key, group)
                    for index, (attr, _) in enumerate(members):
                        patches.set(module, attr, IntegerProjectionSlice(group, index))
                    report["grouped"][f"{module_name}.{key}"] = {
                        "members": [attr for attr, _ in members], "bits": bits,
                        "in_features": group.linear.in_features, "out_features": list(group.sizes),
                        "contiguous_outputs": not group_views,
                    }
                elif shared_quant:
                    cache = ActivationCache(siblings[0].pack_input, len(siblings))
                    for layer in siblings:
                        patches.bind(layer, "forward", lambda self, x, cache=cache: self.forward_packed(cache.get(x)))
