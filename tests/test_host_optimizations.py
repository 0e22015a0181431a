"""Host-side plugin surface (no GPU): switches, instance patching, activation-pack sharing, scope
selection, the progressive tier map and the CUDA-graph helper's bookkeeping.  The contracts are
those the reference's own CPU tests pin (tests/test_optimization_config.py,
test_optimization_patching.py, test_quantization_selection.py, test_progressive_quantization.py,
test_graph_lifecycle_cpu.py)."""

import argparse
import math

import pytest

from rk_b200.optimizations import (ActivationCache, OptimizationConfig, Patches, compare_samples,
                                   cosmos_candidate_sites, cosmos_precision_map, cosmos_tier_variants,
                                   measurement_configurations, pi05_scope)
from rk_b200.optimizations import entry
from rk_b200.optimizations.config import from_dict


# ---------------------------------------------------------------- configuration
def test_defaults_keep_the_original_path():
    config = OptimizationConfig()
    assert config.enabled == () and config.precision == "bf16" and config.to_dict()["switches"] == []


def test_norm_pack_switch_needs_integer_dit_and_keeps_a_bf16_reference():
    switches = ("modulation", "modulation_quant", "norm_modulation_quant")
    rows = dict(measurement_configurations(OptimizationConfig(switches, "int4", ("dit",))))
    assert rows["optimized-bf16"].enabled == ("modulation",)
    combined = OptimizationConfig((*switches, "gated_residual", "residual_norm_modulation_quant"), "int4", ("dit",))
    assert dict(measurement_configurations(combined))["optimized-bf16"].enabled == ("modulation", "gated_residual")
    with pytest.raises(ValueError, match="residual_norm_modulation_quant requires"):
        OptimizationConfig(("residual_norm_modulation_quant",), "int4", ("dit",))
    for options in (dict(switches=switches, precision="bf16", scopes=("dit",)),
                    dict(switches=switches, precision="int4", scopes=("text",)),
                    dict(switches=("norm_modulation_quant",), precision="int4", scopes=("dit",))):
        with pytest.raises(ValueError, match="norm_modulation_quant requires"):
            OptimizationConfig(**options)


def test_tactics_and_tier_round_trip():
    config = OptimizationConfig(precision="int8", scopes=("dit",), tactic=7, quant_tier=3)
    assert from_dict(config.to_dict()) == config and config.precision_label == "w4-t3"
    with pytest.raises(ValueError):
        OptimizationConfig(quant_tier=1)  # tiers need int8 + dit
    with pytest.raises(ValueError):
        OptimizationConfig(tactic=8)


def test_unknown_and_duplicate_switches():
    assert OptimizationConfig(switches=("flow_loop", "rope")).enabled == ("flow_loop", "rope")
    with pytest.raises(ValueError, match="Unknown"):
        OptimizationConfig(switches=("made_up",))
    with pytest.raises(ValueError, match="Duplicate"):
        OptimizationConfig(switches=("rope", "rope"))
    with pytest.raises(ValueError, match="grouping"):
        OptimizationConfig(switches=("integer_group_views",), precision="int8")


def test_comparison_keeps_samples_and_quality_verdict():
    result = compare_samples([100, 110, 90], [50, 55, 45], exact=False, max_abs=0.1)
    assert result["speedup_vs_baseline"] == 2 and result["saved_ms"] == 50 and result["exact"] is False
    assert result["baseline_samples_ms"] == [100, 110, 90]
    for bad in ([], [0], [-1], [math.nan], [math.inf], [True]):
        with pytest.raises(ValueError):
            compare_samples([1], bad, exact=True, max_abs=0)


def test_command_line_flags():
    parser = argparse.ArgumentParser()
    entry.add_arguments(parser)
    args = parser.parse_args(["--precision", "int8", "--quant-scope", "expert", "--enable", "flow_loop", "--enable",
                              "cuda_graph", "--enable", "shared_quant", "--integer-tactic", "3"])
    config = entry.configuration(args, "pi05")
    assert config.scopes == ("expert",) and config.tactic == 3 and "cuda_graph" in config.enabled
    with pytest.raises(ValueError, match="flow_loop"):
        entry.configuration(parser.parse_args(["--enable", "cuda_graph"]), "pi05")
    with pytest.raises(ValueError, match="int8 or int4"):
        entry.configuration(parser.parse_args(["--enable", "shared_quant"]), "pi05")
    with pytest.raises(ValueError, match="dit"):
        entry.configuration(parser.parse_args(["--precision", "int8", "--quant-scope", "text"]), "cosmos")
    cosmos = entry.configuration(parser.parse_args(["--precision", "int8", "--quant-tier", "4"]), "cosmos")
    assert cosmos.scopes == ("dit",) and cosmos.quant_tier == 4


# ---------------------------------------------------------------- patching
def _value():
    return "original"


class _Model:
    def forward(self):
        return _value()


def test_instance_patch_leaves_module_globals_and_other_instances_alone():
    one, two = _Model(), _Model()
    patches = Patches()
    patches.globals(one, "forward", {"_value": lambda: "optimized"})
    assert one.forward() == "optimized" and two.forward() == "original" and _value() == "original"
    patches.restore()
    assert "forward" not in vars(one) and one.forward() == "original"
    with pytest.raises(ValueError, match="missing global"):
        patches.globals(one, "forward", {"not_there": 1})


def test_patch_restores_attributes_kept_in_a_module_registry():
    class Registry:
        def __init__(self):
            object.__setattr__(self, "_modules", {"layer": "original"})

        def __getattr__(self, name):
            return self._modules[name]

        def __setattr__(self, name, value):
            self._modules[name] = value

        def __delattr__(self, name):
            del self._modules[name]

    module = Registry()
    patches = Patches()
    patches.set(module, "layer", "optimized")
    assert module.layer == "optimized"
    patches.restore()
    assert module.layer == "original"


# ---------------------------------------------------------------- selection
def test_pack_is_shared_only_inside_one_projection_group():
    calls = []

    def prepare(x):
        calls.append(object())
        return calls[-1]

    cache = ActivationCache(prepare, 3)
    x, other = object(), object()
    first = cache.get(x)
    assert cache.get(x) is first and cache.get(x) is first
    assert cache.get(x) is not first          # fan-out exhausted: prepared again
    assert cache.get(other) is not calls[-2]  # a new input never reuses the old pack
    assert len(calls) == 3


def test_scope_skips_language_head_and_action_projections():
    assert pi05_scope("paligemma_with_expert.paligemma.model.language_model.layers.0.mlp.up_proj") == "text"
    assert pi05_scope("paligemma_with_expert.gemma_expert.model.layers.0.self_attn.q_proj") == "expert"
    assert pi05_scope("paligemma_with_expert.paligemma.lm_head") is None
    assert pi05_scope("action_out_proj") is None


def test_quantize_linears_rejects_bad_requests_before_touching_the_model():
    from rk_b200.optimizations import quantize_linears

    with pytest.raises(ValueError, match="Unknown low-precision"):
        with quantize_linears(object(), "int2"):
            pass
    with pytest.raises(ValueError, match="scopes"):
        with quantize_linears(object(), "int8", scopes=("everything",)):
            pass


def test_quantize_linears_skips_non_bf16_and_restores_on_exit():
    import torch

    from rk_b200.optimizations import quantize_linears

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj = torch.nn.Linear(8, 8).float()  # fp32: reported as skipped

    model = torch.nn.ModuleDict({"layers": torch.nn.ModuleList([Block()])})
    original = model["layers"][0].q_proj
    with pytest.raises(ValueError, match="No eligible"):
        with quantize_linears(model, "int8", scopes=("dit",), selector=lambda name: "dit"):
            pass
    assert model["layers"][0].q_proj is original


# ---------------------------------------------------------------- progressive tiers
def test_tier_ladder_counts_are_cumulative(golden):
    names = cosmos_candidate_sites()
    assert len(names) == 280
    previous = set()
    for tier, expected in enumerate((0, 8, 18, 28, 36, 46, 56, 84, 168, 224, 280)):
        mapping = cosmos_precision_map(names, tier)
        selected = {name for name, bits in mapping.items() if bits == 4}
        assert len(selected) == expected and previous <= selected and set(mapping.values()) <= {4, 8}
        previous = selected
    assert cosmos_precision_map(names, 1)["blocks.20.cross_attn.output_proj"] == 4
    assert cosmos_precision_map(names, 1)["blocks.19.cross_attn.output_proj"] == 8
    # identical to the reference's own map (fixture generated from its code)
    tier5 = cosmos_precision_map(names, 5)
    assert [tier5[n] for n in names] == golden["tier5_bits"].tolist()
    assert golden["tier_w4_counts"].tolist() == [0, 8, 18, 28, 36, 46, 56, 84, 168, 224, 280]


def test_tier_ladder_rejects_other_architectures_and_bad_tiers():
    names = cosmos_candidate_sites()
    for tier in (-1, 11, True):
        with pytest.raises(ValueError):
            cosmos_precision_map(names, tier)
    with pytest.raises(ValueError, match="candidate"):
        cosmos_precision_map(names[:-1], 1)
    with pytest.raises(ValueError, match="candidate"):
        cosmos_precision_map(names + [names[0]], 1)
    wrapped = [n.replace("blocks.3.", "blocks.3._checkpoint_wrapped_module.") for n in names]
    assert sum(v == 4 for v in cosmos_precision_map(wrapped, 2).values()) == 18


def test_progressive_sweep_variants_from_one_template():
    template = OptimizationConfig(("modulation", "cuda_graph"), scopes=("dit",), tactic=1)
    variants = cosmos_tier_variants(template, [0, 3, 10])
    rows = measurement_configurations(template, variants)
    assert [name for name, _ in rows] == ["original", "optimized-bf16", "w8a8", "w4-t3", "w4-t10"]
    assert [c.quant_tier for _, c in rows[2:]] == [0, 3, 10]
    assert all(c.precision == "int8" and c.tactic == 1 for _, c in rows[2:])
    with pytest.raises(ValueError):
        cosmos_tier_variants(template, [1, 1])


def test_condition_caches_leave_the_flow_loop_output_unchanged():
    """`condition_cache` / `condition_projection_cache` of the reference's pi0.5 optimizations
    (optimizations/pi05.py:273-333): the per-step timestep condition and every adaptive norm's
    dense(condition) are constants of the schedule; caching them changes no bit of the result,
    fills once, and exposes the tensors a CUDA-graph owner has to keep alive."""
    import torch

    from rk_b200.gemma_stack import ActionExpert, GemmaConfig
    from rk_b200.optimizations import ConstantProjectionCache

    cfg = GemmaConfig(width=64, mlp_dim=128, depth=2, num_heads=2, num_kv_heads=1, head_dim=32, adarms_cond_dim=64)
    expert = ActionExpert(cfg, chunk=6, action_dim=8, steps=3).init_random(1).eval()
    gen = torch.Generator().manual_seed(0)
    noise = torch.randn(2, 6, 8, generator=gen)
    pk = torch.randn(2, 2, 1, 10, 32, generator=gen).to(torch.bfloat16)
    pv = torch.randn(2, 2, 1, 10, 32, generator=gen).to(torch.bfloat16)
    with torch.no_grad():
        plain = expert(noise, pk, pv)
        expert.enable_condition_caches()
        first = expert(noise, pk, pv)
        norms = expert.adaptive_norms()
        assert len(norms) == 2 * 2 + 1  # two per layer and the final norm
        assert len(expert._conditions) == 3 and all(len(n.projection_cache) == 3 for n in norms)
        kept = expert.retained_tensors()
        assert len(kept) == 3 + len(norms) * 3 * 5
        second = expert(noise * 2, pk, pv)  # other inputs, same schedule: nothing is added
        assert len(expert._conditions) == 3 and all(len(n.projection_cache) == 3 for n in norms)
        assert torch.equal(first, plain)
        expert.disable_condition_caches()
        assert torch.equal(expert(noise * 2, pk, pv), second)
        assert all(n.projection_cache is None for n in norms) and expert.retained_tensors() == ()
    # an input that was not registered is never cached
    calls = []
    cache = ConstantProjectionCache(lambda v: (calls.append(1), v + 1)[1], lambda v: False)
    t = torch.zeros(2)
    assert torch.equal(cache(t), t + 1) and torch.equal(cache(t), t + 1) and len(calls) == 2 and len(cache) == 0


def test_fp8_prefill_scale_state_measures_every_nth_multirow_call(monkeypatch):
    """Periodic reuse of the dynamic FP8 activation scale (reference: blackwell/fp8_linear.py:147-239),
    with the two quantizer entry points replaced by recorders."""
    import torch

    from rk_b200 import fp8_linear as P8

    calls = []
    monkeypatch.setattr(P8, "quantize_bf16", lambda t: (calls.append("measure") or "codes", torch.tensor([float(len(calls))])))
    monkeypatch.setattr(P8, "quantize_bf16_with_scale", lambda t, s: calls.append(("reuse", float(s))) or "codes")
    state = P8.Fp8PrefillScaleState(3)
    x = torch.zeros(4, 8)
    scales = [float(state.quantize(x)[1]) for _ in range(7)]
    assert calls == ["measure", ("reuse", 1.0), ("reuse", 1.0), "measure", ("reuse", 4.0), ("reuse", 4.0), "measure"]
    assert scales == [1.0, 1.0, 1.0, 4.0, 4.0, 4.0, 7.0]
    assert state.to_dict() == {"eligible": True, "interval": 3, "prefill_calls": 7, "refreshes": 3, "reuses": 4,
                               "operator_fallbacks": 0}
    # single-row (decode) calls always measure and do not advance the schedule
    calls.clear()
    state.quantize(torch.zeros(1, 8))
    assert calls == ["measure"] and state.prefill_calls == 7
    # ineligible roles and interval 1 never reuse; "static" measures once
    assert P8.Fp8PrefillScaleState(5, eligible=False).interval == 1
    assert P8.resolve_fp8_prefill_scale_refresh_interval("static") == 2 ** 31 - 1
    monkeypatch.setenv(P8.PREFILL_SCALE_REFRESH_INTERVAL_ENV, "4")
    assert P8.Fp8PrefillScaleState().interval == 4
    for bad in ("0", "-2", "soon"):
        with pytest.raises(ValueError):
            P8.resolve_fp8_prefill_scale_refresh_interval(bad)


def test_fp8_prefill_scale_refresh_is_configured_per_model():
    import torch

    from rk_b200 import fp8_linear as P8

    class Layer(torch.nn.Module):
        def __init__(self, eligible):
            super().__init__()
            self._prefill_scale_state = P8.Fp8PrefillScaleState(eligible=eligible)

    model = torch.nn.Sequential(Layer(True), Layer(True), Layer(False))
    assert P8.configure_fp8_prefill_scale_refresh(model, 8) == {"interval": 8, "states": 2}
    stats = P8.fp8_prefill_scale_refresh_stats(model)
    assert stats["states"] == 2 and stats["intervals"] == [8] and stats["reuses"] == 0
    assert P8.configure_fp8_prefill_scale_refresh(torch.nn.Sequential(Layer(False))) == {"interval": 1, "states": 0}


def _fake_fp4(in_features, out_features, global_scale):
    import torch

    from rk_b200.fp4_linear import Fp4CutlassLinear

    return Fp4CutlassLinear(torch.zeros(out_features, in_features // 2, dtype=torch.uint8), torch.zeros(16, dtype=torch.uint8),
                            torch.ones(1) if global_scale else None, None, in_features, out_features, "linear", "probe")


def test_fused_fp4_norms_need_uniform_fp4_consumers_and_plain_weights():
    """`fuse_norm_pack_fp4` switches a norm only when every linear that reads it is an NVFP4 layer with the
    same per-tensor-scale setting, never an adaptive norm; `unfuse_norm_quantize` switches them back."""
    from rk_b200.gemma_stack import GemmaConfig, GemmaStack, fuse_norm_pack_fp4, unfuse_norm_quantize

    cfg = GemmaConfig(width=128, mlp_dim=256, depth=3, num_heads=2, num_kv_heads=1, head_dim=64)
    stack = GemmaStack(cfg)
    qd, kvd = cfg.num_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
    # layer 0: everything NVFP4 with per-tensor scales; layer 1: q/k/v mixed scale settings, gate/up block-only;
    # layer 2: one bf16 projection left in each group
    l0, l1, l2 = stack.layers
    l0.self_attn.q_proj, l0.self_attn.k_proj, l0.self_attn.v_proj = (_fake_fp4(128, qd, True), _fake_fp4(128, kvd, True),
                                                                      _fake_fp4(128, kvd, True))
    l0.mlp.gate_proj, l0.mlp.up_proj = _fake_fp4(128, 256, True), _fake_fp4(128, 256, True)
    l1.self_attn.q_proj, l1.self_attn.k_proj, l1.self_attn.v_proj = (_fake_fp4(128, qd, True), _fake_fp4(128, kvd, False),
                                                                      _fake_fp4(128, kvd, True))
    l1.mlp.gate_proj, l1.mlp.up_proj = _fake_fp4(128, 256, False), _fake_fp4(128, 256, False)
    l2.self_attn.q_proj = _fake_fp4(128, qd, True)
    l2.mlp.gate_proj = _fake_fp4(128, 256, True)
    norms = fuse_norm_pack_fp4(stack)
    assert norms == [l0.input_layernorm, l0.post_attention_layernorm, l1.post_attention_layernorm]
    assert [n.fused_fp4 for n in norms] == ["global", "global", "block"]
    assert l1.input_layernorm.fused_fp4 is None and l2.input_layernorm.fused_fp4 is None
    assert stack.norm.fused_fp4 is None  # the final norm feeds no linear
    unfuse_norm_quantize(norms)
    assert all(n.fused_fp4 is None for n in norms)
    adaptive = GemmaStack(GemmaConfig(width=128, mlp_dim=256, depth=1, num_heads=2, num_kv_heads=1, head_dim=64,
                                      adarms_cond_dim=128))
    layer = adaptive.layers[0]
    layer.self_attn.q_proj, layer.self_attn.k_proj, layer.self_attn.v_proj = (_fake_fp4(128, qd, True), _fake_fp4(128, kvd, True),
                                                                                _fake_fp4(128, kvd, True))
    assert fuse_norm_pack_fp4(adaptive) == []


def test_packed_nvfp4_activation_carrier():
    import torch

    from rk_b200.fp4_linear import PackedNvfp4Activation
    from rk_b200.gemma_stack import _leading_shape

    carrier = PackedNvfp4Activation(torch.zeros(6, 64, dtype=torch.uint8), torch.zeros(512, dtype=torch.uint8), torch.ones(1),
                                    (2, 3), 128)
    assert carrier.shape == (2, 3, 128) and carrier.shape[:-1] == (2, 3) and _leading_shape(carrier) == (2, 3)
    layer = _fake_fp4(128, 64, True)
    q, sf, ga = layer.pack_input(carrier)
    assert q is carrier.codes and sf is carrier.scale_factors and ga is carrier.global_scale
    with pytest.raises(ValueError):
        _fake_fp4(256, 64, True).pack_input(carrier)      # feature count
    with pytest.raises(ValueError):
        _fake_fp4(128, 64, False).pack_input(carrier)     # a per-tensor scale the layer does not expect
