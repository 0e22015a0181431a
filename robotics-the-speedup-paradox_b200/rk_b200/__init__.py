"""B200-native quantized-linear operators behind the reference's operator surface.

The kernels live in ``librk_b200.so`` (C ABI: ``include/rk_b200.h``); the modules here mirror
``src/robotics_kernels`` of the reference: ``IntegerLinear`` / ``prepare_activation`` /
``PackedActivation`` (integer path), ``W4A16Linear`` (int4 group-128 weights), and the loaders'
status helpers.  Importing this package does not load the library; the first operator call does,
and raises when the library is missing.
"""

from ._lib import backend_status, library_path  # noqa: F401
