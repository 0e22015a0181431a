"""Optimization switches and measured-comparison helpers (CPU only).

Reference: optimizations/config.py:73-264.  `OptimizationConfig` keeps the same fields, switch
vocabulary and cross-switch rules; the integer tactic ids are those of
ampere_ada/tactics.py:4-13 (0..7), which the B200 kernels accept and ignore for results.
"""

from dataclasses import dataclass
import math
import re
from statistics import median

TACTIC_IDS = tuple(range(8))
CONVOLUTION_TACTICS = tuple(range(8))
SCOPES = ("text", "expert", "vision", "projector", "dit")
PRECISIONS = ("bf16", "int8", "int4", "fp8", "fp4")

ATTENTION_SWITCHES = {
    "attention_sdpa_flash": "sdpa_flash",
    "attention_sdpa_efficient": "sdpa_efficient",
    "attention_sdpa_math": "sdpa_math",
    "attention_flash_attn": "flash_attn",
}
CONVOLUTION_SWITCHES = {f"conv_cutlass_{t}": t for t in CONVOLUTION_TACTICS}
CONVOLUTION_SWITCHES.update({f"conv_cutlass_c96_{t}": t for t in CONVOLUTION_TACTICS})
CONVOLUTION_SWITCHES["conv_cutlass_c96"] = 0

# switches of the Cosmos pipeline that pi0.5 does not accept
COSMOS_ONLY_SWITCHES = (
    *ATTENTION_SWITCHES, *CONVOLUTION_SWITCHES, "vae_norm_fusion", "vae_silu_fusion", "vae_spatial_padding",
    "vae_condition_prefix", "cross_kv_cache", "modulation", "modulation_quant", "norm_modulation_quant",
    "residual_norm_modulation_quant",
)

# switches that only make sense together with an integer precision
PRECISION_SWITCHES = frozenset({
    "residual_norm_modulation_quant", "norm_modulation_quant", "modulation_quant", "shared_quant",
    "activation_quant_fusion", "integer_grouped", "integer_pack_reuse", "integer_qkv", "integer_gate_up",
    "integer_group_views", "integer_biasless",
})
GROUPING_SWITCHES = frozenset({"integer_grouped", "integer_qkv", "integer_gate_up"})

SWITCHES = (
    *ATTENTION_SWITCHES, *CONVOLUTION_SWITCHES,
    "vae_norm_fusion", "vae_silu_fusion", "vae_spatial_padding", "vae_condition_prefix", "cross_kv_cache",
    "residual_norm_modulation_quant", "norm_modulation_quant", "modulation_quant", "flow_loop", "mask_cache",
    "condition_cache", "condition_projection_cache", "empty_image_cache", "rope", "gated_residual", "gelu_mul",
    "norm", "projection_fusion", "cuda_graph", "shared_quant", "modulation", "activation_quant_fusion",
    "integer_grouped", "integer_pack_reuse", "integer_qkv", "integer_gate_up", "integer_group_views",
    "integer_biasless",
)


def _requires(switches, name, needed, message):
    if name in switches and not set(needed) <= switches:
        raise ValueError(message)


@dataclass(frozen=True)
class OptimizationConfig:
    switches: tuple = ()
    precision: str = "bf16"
    scopes: tuple = ("text",)
    tactic: int = 0
    quant_tier: int | None = None

    def __post_init__(self):
        if not isinstance(self.switches, tuple):
            raise ValueError("switches must be a tuple of names")
        if any(not isinstance(s, str) or s not in SWITCHES for s in self.switches):
            raise ValueError("Unknown optimization switch")
        on = set(self.switches)
        if len(on) != len(self.switches):
            raise ValueError("Duplicate optimization switch")
        _requires(on, "residual_norm_modulation_quant", ("norm_modulation_quant", "gated_residual"),
                  "residual_norm_modulation_quant requires norm_modulation_quant and gated_residual")
        if "norm_modulation_quant" in on and (
            not {"modulation", "modulation_quant"} <= on or self.precision not in ("int4", "int8")
            or self.scopes != ("dit",)
        ):
            raise ValueError(
                "norm_modulation_quant requires modulation, modulation_quant, INT4/INT8 and the Cosmos dit scope")
        if len(on & ATTENTION_SWITCHES.keys()) > 1:
            raise ValueError("Choose one attention backend per configuration")
        if len(on & CONVOLUTION_SWITCHES.keys()) > 1:
            raise ValueError("Choose one convolution tactic per configuration")
        _requires(on, "vae_silu_fusion", ("vae_norm_fusion",), "vae_silu_fusion requires vae_norm_fusion")
        if not self.scopes or any(s not in SCOPES for s in self.scopes):
            raise ValueError("Unknown quantization scope")
        if type(self.tactic) is not int or self.tactic not in TACTIC_IDS:
            raise ValueError("Unknown integer tactic")
        if self.precision not in PRECISIONS:
            raise ValueError("Unknown precision")
        _requires(on, "condition_projection_cache", ("condition_cache", "flow_loop"),
                  "condition_projection_cache requires condition_cache and flow_loop")
        if "integer_group_views" in on and not on & GROUPING_SWITCHES:
            raise ValueError("integer_group_views requires an integer projection grouping switch")
        if self.quant_tier is not None and (
            type(self.quant_tier) is not int or not 0 <= self.quant_tier <= 10 or self.precision != "int8"
            or self.scopes != ("dit",)
        ):
            raise ValueError("Progressive tiers require INT8 base precision and the Cosmos dit scope")

    @property
    def enabled(self):
        return self.switches

    @property
    def precision_label(self):
        return f"w4-t{self.quant_tier}" if self.quant_tier else self.precision

    def to_dict(self):
        data = {"switches": list(self.switches), "precision": self.precision, "scopes": list(self.scopes),
                "tactic": self.tactic}
        if self.quant_tier is not None:
            data["quant_tier"] = self.quant_tier
        return data


def from_dict(data):
    """Inverse of `OptimizationConfig.to_dict` (reference: optimizations/entry.py `from_dict`)."""
    allowed = {"switches", "precision", "scopes", "tactic", "quant_tier"}
    if not isinstance(data, dict) or set(data) - allowed:
        raise ValueError("Unknown optimization configuration fields")
    return OptimizationConfig(
        tuple(data.get("switches", ())), data.get("precision", "bf16"), tuple(data.get("scopes", ("text",))),
        data.get("tactic", 0), data.get("quant_tier"),
    )


def _shared(config):
    return tuple(s for s in config.switches if s not in PRECISION_SWITCHES)


def measurement_configurations(config, variants=None, *, allow_shared_variants=False):
    """The cohort measured together: the untouched model, the BF16 model with the same shared
    switches as each candidate, and the candidates themselves."""
    rows = [("original", OptimizationConfig())]
    shared = _shared(config)
    if variants is not None or config.precision != "bf16":
        rows.append(("optimized-bf16", OptimizationConfig(shared, "bf16", config.scopes, config.tactic)))
    if variants is None:
        rows.append(("candidate", config))
        return rows
    if not isinstance(variants, list) or not variants:
        raise ValueError("Variants must be a nonempty list")
    taken = {name for name, _ in rows}
    references = {frozenset(shared)}
    for data in variants:
        if not isinstance(data, dict) or set(data) - {"id", "switches", "precision", "scopes", "tactic", "quant_tier"}:
            raise ValueError("Unknown variant fields")
        name = data.get("id")
        if (not isinstance(name, str) or not re.fullmatch(r"[A-Za-z0-9][A-Za-z0-9_-]*", name) or name in taken
                or name.startswith("optimized-bf16-")):
            raise ValueError("Variant IDs must be unique, safe filenames and not reference IDs")
        current = OptimizationConfig(
            tuple(data.get("switches", config.switches)), data.get("precision", config.precision),
            tuple(data.get("scopes", config.scopes)), data.get("tactic", config.tactic),
            data.get("quant_tier", config.quant_tier),
        )
        current_shared = _shared(current)
        if set(current_shared) != set(shared) and not allow_shared_variants:
            raise ValueError(
                "Variants must use the same shared optimization switches as their matched BF16 reference")
        if set(current.switches) & PRECISION_SWITCHES and not current.precision.startswith("int"):
            raise ValueError("Integer switches require integer precision")
        if frozenset(current_shared) not in references:
            reference_id = f"optimized-bf16-{len(references) + 1}"
            rows.append((reference_id, OptimizationConfig(current_shared, "bf16", current.scopes, current.tactic)))
            taken.add(reference_id)
            references.add(frozenset(current_shared))
        taken.add(name)
        rows.append((name, current))
    return rows


def _checked_samples(values):
    values = list(values)
    if not values or any(
        isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or v <= 0 for v in values
    ):
        raise ValueError("Timing samples must be nonempty finite positive numbers")
    return values


def compare_samples(baseline, candidate, *, exact, max_abs):
    """Median-to-median comparison that keeps the raw samples and the numerical verdict."""
    baseline, candidate = _checked_samples(baseline), _checked_samples(candidate)
    if type(exact) is not bool or not math.isfinite(max_abs) or max_abs < 0:
        raise ValueError("Invalid numerical comparison")
    if exact and max_abs != 0:
        raise ValueError("Exact comparison must have zero error")
    before, after = median(baseline), median(candidate)
    return {
        "statistic": "median", "baseline_samples_ms": baseline, "candidate_samples_ms": candidate,
        "baseline_ms": before, "candidate_ms": after, "speedup_vs_baseline": before / after,
        "saved_ms": before - after, "exact": exact, "max_abs": max_abs,
    }
