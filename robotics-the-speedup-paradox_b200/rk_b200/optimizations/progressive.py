"""Progressive W8A8 -> W4A4 site selection for the Cosmos DiT (28 blocks x 10 linears).

Reference: optimizations/progressive.py:4-86.  A tier is a cumulative list of rules; a site is
4-bit at tier t when any rule with threshold <= t matches it.  Tier 0 is all-int8, tier 10 all-int4;
the number of 4-bit sites per tier is 0, 8, 18, 28, 36, 46, 56, 84, 168, 224, 280.
"""

BLOCKS = 28
ATTENTION_FAMILIES = ("self_attn", "cross_attn")
PROJECTIONS = ("q_proj", "k_proj", "v_proj", "output_proj")
MLP_ROLES = ("layer1", "layer2")
WRAPPER = "._checkpoint_wrapped_module"


def cosmos_candidate_sites():
    per_block = [f"{family}.{role}" for family in ATTENTION_FAMILIES for role in PROJECTIONS]
    per_block += [f"mlp.{role}" for role in MLP_ROLES]
    return [f"blocks.{block}.{site}" for block in range(BLOCKS) for site in per_block]


def _first_low_tier(block, family, role):
    """Smallest tier at which this site drops to 4 bits."""
    early, late = block < 10, block >= 20
    if family == "cross_attn" and role == "output_proj":
        return 1 if late else (3 if early else 6)
    if family == "mlp" and role == "layer1":
        return 2 if early else (4 if late else 5)
    if family == "mlp" and role == "layer2":
        return 7
    if family == "self_attn" and role != "v_proj":
        return 8
    if (family == "self_attn" and role == "v_proj") or (family == "cross_attn" and role == "q_proj"):
        return 9
    return 10


def cosmos_precision_map(names, tier):
    if type(tier) is not int or not 0 <= tier <= 10:
        raise ValueError("Cosmos quantization tier must be an integer from 0 to 10")
    names = list(names)
    canonical = [name.replace(WRAPPER, "") for name in names]
    expected = cosmos_candidate_sites()
    if len(canonical) != len(expected) or set(canonical) != set(expected):
        raise ValueError("Cosmos tier protocol requires the exact 280 candidate sites in 28 blocks")
    bits = {}
    for original, name in zip(names, canonical):
        _, block, family, role = name.split(".")
        bits[original] = 4 if tier >= 1 and _first_low_tier(int(block), family, role) <= tier else 8
    return bits


def cosmos_tier_variants(template, tiers=None):
    """Variant dictionaries for a W8A8-to-W4A4 sweep that share one workload template."""
    tiers = list(range(11)) if tiers is None else list(tiers)
    if template.scopes != ("dit",) or template.precision not in ("bf16", "int8") or template.quant_tier is not None:
        raise ValueError("A progressive sweep requires a BF16/INT8 Cosmos dit template without a single tier")
    if not tiers or len(set(tiers)) != len(tiers) or any(type(t) is not int or not 0 <= t <= 10 for t in tiers):
        raise ValueError("Select unique integer tiers from 0 to 10")
    switches = list(template.enabled)
    switches += [s for s in ("shared_quant", "activation_quant_fusion", "integer_pack_reuse") if s not in switches]
    return [
        {"id": f"w4-t{tier}" if tier else "w8a8", "precision": "int8", "switches": switches, "scopes": ["dit"],
         "tactic": template.tactic, "quant_tier": tier}
        for tier in tiers
    ]
