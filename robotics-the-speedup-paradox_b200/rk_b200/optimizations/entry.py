"""Command-line flags of the optimization layer and their validation (CPU only).

Reference: optimizations/entry.py:14-111 (``add_arguments``, ``configuration``, ``from_dict``).
"""

from .config import (COSMOS_ONLY_SWITCHES, PRECISION_SWITCHES, PRECISIONS, SCOPES, SWITCHES, TACTIC_IDS,
                     OptimizationConfig, from_dict)  # noqa: F401

COSMOS_SWITCHES = frozenset({
    *COSMOS_ONLY_SWITCHES, "gated_residual", "cuda_graph", "shared_quant", "activation_quant_fusion",
    "integer_grouped", "integer_pack_reuse", "integer_qkv", "integer_group_views", "integer_biasless",
})


def add_arguments(parser):
    parser.add_argument("--model-runtime", choices=("owned", "native"), default="owned")
    parser.add_argument("--enable", action="append", choices=SWITCHES, default=[],
                        help="Enable one independent optimization (repeatable)")
    parser.add_argument("--precision", choices=PRECISIONS, default="bf16")
    parser.add_argument("--quant-scope", action="append", choices=SCOPES)
    parser.add_argument("--integer-tactic", type=int, choices=TACTIC_IDS, default=0)
    parser.add_argument("--quant-tier", type=int, choices=range(11),
                        help="Cosmos appendix tier: 0=W8A8, 1..10 progressively W4A4")


def configuration(args, model="pi05"):
    """Parsed flags -> a validated OptimizationConfig for `model` ("pi05" or "cosmos")."""
    default_scope = ("text",) if model == "pi05" else ("dit",)
    config = OptimizationConfig(tuple(args.enable), args.precision, tuple(args.quant_scope or default_scope),
                                args.integer_tactic, getattr(args, "quant_tier", None))
    on = set(config.switches)
    if on & PRECISION_SWITCHES and not config.precision.startswith("int"):
        raise ValueError("Integer preparation switches require int8 or int4 precision")
    allowed = set(SWITCHES) - set(COSMOS_ONLY_SWITCHES) if model == "pi05" else COSMOS_SWITCHES
    if on - allowed:
        raise ValueError(f"Unsupported {model} optimization switch")
    if model == "pi05" and "condition_cache" in on and "flow_loop" not in on:
        raise ValueError("condition_cache requires flow_loop")
    if "empty_image_cache" in on and "cuda_graph" not in on:
        raise ValueError("empty_image_cache requires cuda_graph")
    if args.model_runtime == "native" and (on or config.precision != "bf16"):
        raise ValueError("Local optimizations require --model-runtime owned")
    if model == "pi05" and "cuda_graph" in on and "flow_loop" not in on:
        raise ValueError("PI0.5 cuda_graph requires flow_loop")
    if model == "cosmos" and config.scopes != ("dit",):
        raise ValueError("Cosmos quantization scope must be dit")
    if model == "pi05" and "dit" in config.scopes:
        raise ValueError("PI0.5 does not support the dit quantization scope")
    return config
