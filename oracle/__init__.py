"""CPU oracle for the quantized-linear hot path.

TEST INFRASTRUCTURE ONLY.  This package restates, on the CPU with numpy, the
arithmetic of the reference's quantized-linear operators.  It is the checker the
CUDA kernels are compared against; nothing in the shipped package imports it.
Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import it.

Parity status per family (what the restatement is pinned against):

* integer (W8A8 / W4A4 row quantizer, weight quantizer, GEMM epilogue, AdaLN
  modulation pack): PINNED.  Golden fixtures in ``tests/golden/`` were produced
  by running the reference's own Triton kernels (interpreter mode, CPU) and its
  own torch weight-packing code, and by evaluating the known-answer formula of
  ``tests/gpu/test_integer_linear.py:30-37``.
* number formats (E4M3, UE4M3, UE8M0, E2M1) and the scale-factor layout: PINNED
  against the conversion routines the reference itself calls - the host paths
  of its vendored CUTLASS 4.4.2 types, the toolkit's FP8 conversion, and its own
  ``scale_offset`` - compiled from the reference checkout by
  ``oracle/build_ref.py`` (``oracle/ref_formats.cpp`` -> ``oracle/_ref``), and
  cross-checked against torch's float8 casts.
* per-tensor FP8, MXFP8, NVFP4 packers and GEMMs: PARITY UNPINNED by any
  reference test or runnable reference code (they are CUDA-only and the
  reference has no numerical test for them); the restatement follows the
  source line by line and is anchored only on the pinned number formats.
* W4A16 int4 group-128: defined by the benchmark configuration, not by the
  reference; PARITY UNPINNED (conventions follow the reference's int4 packing).
"""
