"""Plugin surface of the quantized-linear path: switches, instance patching, module selection
and the progressive W8A8 -> W4A4 tier map.  Mirrors ``src/robotics_bench/optimizations`` of the
reference for the parts that concern quantized linears (config.py, patching.py, quantization.py,
progressive.py, entry.py); the other hot spots that package tunes (attention, VAE, convolution)
are accepted as switch names so existing configurations still parse, and are not acted on here.
"""

from .constant_projection import ConstantProjectionCache  # noqa: F401
from .config import OptimizationConfig, compare_samples, measurement_configurations  # noqa: F401
from .patching import Patches  # noqa: F401
from .progressive import cosmos_candidate_sites, cosmos_precision_map, cosmos_tier_variants  # noqa: F401
from .quantization import ActivationCache, pi05_scope, quantize_linears  # noqa: F401
