#!/usr/bin/env python3
"""Generate golden fixtures for the integer path by running the REFERENCE's own code on the CPU.

Needs a checkout of the reference (``--reference``, default: a directory named ``reference`` beside
this repository); run once where that checkout exists:

    python tests/golden/make_golden.py [--reference PATH]

What runs:

* the reference's Triton kernels ``_prepare`` (ampere_ada/integer.py:75-119) and
  ``_prepare_modulation`` / ``_prepare_norm_modulation`` / ``_prepare_residual_norm_modulation``
  (ampere_ada/modulation.py:52-146) in Triton's interpreter mode (``TRITON_INTERPRET=1``), which
  executes the kernel bodies with numpy.  Two primitives of the interpreter are substituted so
  that it computes what the compiled kernel computes on a GPU: the CUDA-only
  ``libdevice.nearbyint`` becomes ``numpy.rint`` (both round half to even), and the
  interpreter's float32 -> bfloat16 conversion, which truncates, becomes round-to-nearest-even
  (the compiled ``.to(bfloat16)`` is ``cvt.rn.bf16.f32``), done with torch's own conversion.
  The kernel sources themselves run unchanged.
* the torch ops of ``IntegerLinear.from_linear`` (ampere_ada/integer.py:236-281) on CPU tensors,
  with the CUDA check satisfied by a stand-in weight wrapper and the extension loader stubbed.
* the known-answer formula of the reference's GPU test (tests/gpu/test_integer_linear.py:30-37).
* ``cosmos_precision_map`` (src/robotics_bench/optimizations/progressive.py:14-52) tier counts.

Output: ``tests/golden/integer_golden.npz`` (bf16 tensors stored as uint16 bit patterns).
"""

import argparse
import os
import sys
from pathlib import Path
from types import SimpleNamespace

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch


def bits16(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main():
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--reference", default=str(Path(__file__).resolve().parents[3] / "reference"))
    parser.add_argument("--output", default=str(Path(__file__).with_name("integer_golden.npz")))
    args = parser.parse_args()
    sys.path.insert(0, str(Path(args.reference) / "src"))

    import triton
    import triton.language as tl
    from triton.runtime.interpreter import TensorHandle

    from robotics_kernels.ampere_ada import integer as ref_integer
    from robotics_kernels.ampere_ada import modulation as ref_modulation
    from robotics_bench.optimizations.progressive import cosmos_candidate_sites, cosmos_precision_map

    def nearbyint(x):
        return tl.tensor(TensorHandle(np.rint(x.handle.data), x.handle.dtype), x.type)

    ref_integer.libdevice = SimpleNamespace(nearbyint=nearbyint)
    ref_modulation.libdevice = SimpleNamespace(nearbyint=nearbyint)

    from triton.runtime import interpreter as interp

    truncating_convert = interp._convert_float

    def convert_float(data, src_type, dst_type, rounding_mode):
        if src_type == tl.float32 and dst_type == tl.bfloat16:
            values = torch.from_numpy(np.ascontiguousarray(data, dtype=np.float32))
            return values.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16).reshape(data.shape)
        return truncating_convert(data, src_type, dst_type, rounding_mode)

    interp._convert_float = convert_float

    out = {}
    gen = torch.Generator().manual_seed(20240611)

    def randn(*shape, std=1.0):
        return (torch.randn(*shape, generator=gen) * std).to(torch.bfloat16)

    # ---- row quantizer: plain / GELU table / GELU table * up, both nibble-packing code paths
    lut = torch.nn.functional.gelu(
        torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16), approximate="tanh"
    )
    out["gelu_tanh_lut"] = bits16(lut)
    cases = [(3, 130), (17, 256), (4, 2048), (2, 1)]
    for ci, (rows, k) in enumerate(cases):
        x = randn(rows, k)
        if ci == 1:
            x[5] = 0  # an all-zero row: scale must be 1.0
        up = randn(rows, k)
        out[f"rows{ci}_x"] = bits16(x)
        out[f"rows{ci}_up"] = bits16(up)
        pad = triton.cdiv(k, 128) * 128
        for bits in (8, 4):
            for mode in (0, 1, 2):
                for reuse in (False, True):
                    if bits == 8 and reuse:
                        continue
                    data = torch.zeros(
                        (rows, pad if bits == 8 else pad // 2), dtype=torch.int8 if bits == 8 else torch.uint8
                    )
                    scales = torch.zeros(rows, dtype=torch.float32)
                    ref_integer._prepare[(rows,)](
                        x, up, lut if mode else x, data, scales, k, pad, bits, mode,
                        triton.next_power_of_2(pad), reuse, x.stride(0), up.stride(0),
                    )
                    tag = f"rows{ci}_b{bits}_m{mode}_r{int(reuse)}"
                    out[tag + "_q"] = data.numpy().view(np.uint8).copy()
                    out[tag + "_s"] = scales.numpy().copy()

    # ---- weight quantizer (from_linear torch ops)
    class CudaLookalike:
        """Wraps a CPU tensor; reports is_cuda so the reference's guard lets the torch ops run."""

        def __init__(self, t):
            self._t = t
            self.is_cuda = True
            self.dtype = t.dtype

        def detach(self):
            return self._t

    ref_integer.load_integer_extension = lambda: None
    for wi, (n, k) in enumerate([(37, 130), (80, 256), (8, 128)]):
        w = randn(n, k, std=0.02)
        if wi == 1:
            w[3] = 0
        bias = randn(n, std=0.01)
        out[f"w{wi}_w"] = bits16(w)
        out[f"w{wi}_bias"] = bits16(bias)
        for bits in (8, 4):
            layer = ref_integer.IntegerLinear.from_linear(
                SimpleNamespace(weight=CudaLookalike(w), bias=bias), bits=bits
            )
            out[f"w{wi}_b{bits}_q"] = layer.packed_weight.numpy().view(np.uint8).copy()
            out[f"w{wi}_b{bits}_s"] = layer.weight_scale.numpy().copy()
            out[f"w{wi}_b{bits}_bias"] = bits16(layer.bias)

    # ---- known-answer formula of the reference GPU test
    for ki, (m, n, k) in enumerate([(1, 37, 130), (50, 80, 256)]):
        lin = torch.nn.Linear(k, n, dtype=torch.bfloat16)
        with torch.no_grad():
            lin.weight.copy_(randn(n, k, std=0.05))
            lin.bias.copy_(randn(n, std=0.05))
        x = randn(m, k)
        out[f"ka{ki}_x"] = bits16(x)
        out[f"ka{ki}_w"] = bits16(lin.weight.detach())
        out[f"ka{ki}_bias"] = bits16(lin.bias.detach())
        for bits in (8, 4):
            limit = 2 ** (bits - 1) - 1
            ws = lin.weight.float().abs().amax(dim=1).clamp_min(1e-30) / limit
            xs = x.float().abs().amax(dim=1).clamp_min(1e-30) / limit
            qw = torch.round(lin.weight.float() / ws[:, None]).clamp(-limit, limit)
            qx = torch.round(x.float() / xs[:, None]).clamp(-limit, limit)
            ref = ((qx @ qw.T) * xs[:, None] * ws[None, :] + lin.bias.float()).to(x.dtype)
            out[f"ka{ki}_b{bits}_out"] = bits16(ref.detach())

    # ---- AdaLN modulation packs
    for mi, (b, tokens, k) in enumerate([(2, 5, 130), (1, 7, 256)]):
        x = randn(b, tokens, k)
        y = randn(b, tokens, k)
        scale = randn(b, 1, k, std=0.3)
        shift = randn(b, 1, k, std=0.3)
        gate = randn(b, 1, k, std=0.5)
        for name, t in (("x", x), ("y", y), ("scale", scale), ("shift", shift), ("gate", gate)):
            out[f"mod{mi}_{name}"] = bits16(t)
        rows, pad = b * tokens, triton.cdiv(k, 128) * 128
        for bits in (8, 4):
            for variant in ("plain", "norm", "residual"):
                data = torch.zeros(
                    (rows, pad if bits == 8 else pad // 2), dtype=torch.int8 if bits == 8 else torch.uint8
                )
                scales = torch.zeros(rows, dtype=torch.float32)
                common = (x, scale.contiguous(), shift.contiguous(), data, scales, k, pad, tokens, bits,
                          triton.next_power_of_2(pad))
                tag = f"mod{mi}_b{bits}_{variant}"
                if variant == "plain":
                    ref_modulation._prepare_modulation[(rows,)](*common)
                elif variant == "norm":
                    ref_modulation._prepare_norm_modulation[(rows,)](*common, EPS=1e-6)
                else:
                    residual = torch.zeros_like(x)
                    ref_modulation._prepare_residual_norm_modulation[(rows,)](
                        *common, EPS=1e-6, Y=y, GATE=gate.contiguous(), RESIDUAL=residual
                    )
                    out[tag + "_residual"] = bits16(residual)
                out[tag + "_q"] = data.numpy().view(np.uint8).copy()
                out[tag + "_s"] = scales.numpy().copy()

    # ---- progressive tiers: number of 4-bit sites per tier
    sites = cosmos_candidate_sites()
    out["tier_w4_counts"] = np.array(
        [sum(1 for v in cosmos_precision_map(sites, tier).values() if v == 4) for tier in range(11)], dtype=np.int64
    )
    tier5 = cosmos_precision_map(sites, 5)
    out["tier5_bits"] = np.array([tier5[s] for s in sites], dtype=np.int8)

    np.savez_compressed(args.output, **out)
    print(args.output, os.path.getsize(args.output), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
