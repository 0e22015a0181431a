"""Import-path mirror of the reference's ``src/robotics_kernels/blackwell/cute_mxfp8_swiglu.py``: the fused
MXFP8 gate/up GEMM + SwiGLU + MXFP8 output lives in `rk_b200.mxfp8_swiglu`."""

from .mxfp8_swiglu import cutlass_swiglu_mxfp8_packed  # noqa: F401
