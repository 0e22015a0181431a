#!/usr/bin/env python3
"""Per-shape timing of the quantized GEMM and quantizer entry points, through the C ABI.

    python robotics-the-speedup-paradox_b200/rk_b200/microbench.py [w4a16] [w8a8] [fp8] [mxfp8] [nvfp4] [quant]
    python robotics-the-speedup-paradox_b200/rk_b200/microbench.py w8a8:400x8192x1024 quant:16384x2048   # explicit shapes
    python robotics-the-speedup-paradox_b200/rk_b200/microbench.py layer    # per-kernel device time of one expert layer
    python robotics-the-speedup-paradox_b200/rk_b200/microbench.py prefix_layer   # the same for one NVFP4 prefix layer

Each shape is timed as a CUDA graph of back-to-back launches that rotate through enough independent
weight copies to exceed the 126 MB L2 (so a launch streams its weights from HBM), between two CUDA
events on the launching stream.  Shapes are the ones the reference's benchmark configurations name:
the Gemma-2B MLP gate/up GEMM at decode batch sizes (W4A16), the Cosmos cross-attention projection
(W8A8, M = 64), the action-expert and prefix linears of the pi0.5 stack (W8A8, M = 400 / 1764) and
the 816-token prefix GEMMs (FP8 / MXFP8 / NVFP4).  One line per shape: time, algorithmic GB/s and
its share of the measured copy bandwidth, T(FL)OPS, and the device status word (0 = no wait gave up).
"""

import json
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import torch

from rk_b200 import _lib as L


def _hbm_peak():
    path = HERE.parent.parent / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text())["hbm_gbs"], "measured"
    return 6650.0, "fallback"


class Bench:
    def __init__(self):
        if not torch.cuda.is_available():
            raise SystemExit("microbench needs a CUDA device")
        self.lib = L.load()
        self.dev = torch.device("cuda:0")
        torch.cuda.set_device(0)
        self.hbm, self.hbm_src = _hbm_peak()

    def time_us(self, calls, reps=3):
        """calls: one callable(stream_ptr) per rotating copy; average microseconds per launch."""
        stream = torch.cuda.current_stream()
        for f in calls:
            f(L.stream_ptr(self.dev))
        torch.cuda.synchronize()
        graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        side.wait_stream(stream)
        inner = len(calls) * 3
        with torch.cuda.graph(graph, stream=side):
            sp = L.stream_ptr(self.dev)
            for i in range(inner):
                calls[i % len(calls)](sp)
        stream.wait_stream(side)
        graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / (reps * inner) * 1e3

    @staticmethod
    def copies(nbytes):
        return max(2, int(300e6 // nbytes) + 1)

    def report(self, name, m, n, k, tactic, us, nbytes, ops, unit, ws):
        print(f"{name:6s} m{m:5d} n{n:6d} k{k:6d} t{tactic}: {us:8.2f} us  {nbytes / us / 1e3:8.1f} GB/s "
              f"({nbytes / us / 1e3 / self.hbm * 100:5.1f}% of {self.hbm_src} copy bw)  {ops / us / 1e6:8.1f} {unit}  "
              f"status={L.read_status(ws)}", flush=True)

    def w8a8(self, m, n, k, tactic=0):
        dev, lib = self.dev, self.lib
        a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=dev)
        sa, sb = torch.rand(m, device=dev), torch.rand(n, device=dev)
        bs = [torch.randint(-127, 128, (n, k), dtype=torch.int8, device=dev) for _ in range(self.copies(n * k))]
        out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
        ws = L.gemm_workspace(L.OP_W8A8, dev, m, n, k)
        calls = [(lambda sp, b=b: lib.rk_gemm_int(L.ptr(a), L.ptr(sa), L.ptr(b), L.ptr(sb), None, L.ptr(out), m, n, k, 8,
                                                  tactic, L.ptr(ws), ws.numel(), sp)) for b in bs]
        self.report("w8a8", m, n, k, tactic, self.time_us(calls), m * k + n * k + 2 * m * n + 4 * (m + n), 2 * m * n * k,
                    "TOPS", ws)

    def float8(self, kind, m, n, k, tactic=0):
        dev, lib = self.dev, self.lib
        a = torch.randint(0, 120, (m, k), dtype=torch.uint8, device=dev)
        bs = [torch.randint(0, 120, (n, k), dtype=torch.uint8, device=dev) for _ in range(self.copies(n * k))]
        out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
        one = torch.ones(1, device=dev)
        if kind == "fp8":
            ws = L.gemm_workspace(L.OP_FP8, dev, m, n, k)
            calls = [(lambda sp, b=b: lib.rk_gemm_fp8(L.ptr(a), L.ptr(one), L.ptr(b), L.ptr(one), None, L.ptr(out), m, n, k,
                                                      tactic, L.ptr(ws), ws.numel(), sp)) for b in bs]
            nbytes = m * k + n * k + 2 * m * n
        elif kind == "mxfp8":
            ws = L.gemm_workspace(L.OP_MXFP8, dev, m, n, k)
            sfa = torch.full((lib.rk_sf_bytes(m, k // 32),), 127, dtype=torch.uint8, device=dev)
            sfb = torch.full((lib.rk_sf_bytes(n, k // 32),), 127, dtype=torch.uint8, device=dev)
            calls = [(lambda sp, b=b: lib.rk_gemm_mxfp8(L.ptr(a), L.ptr(sfa), L.ptr(b), L.ptr(sfb), None, L.ptr(out), m, n,
                                                        k, tactic, L.ptr(ws), ws.numel(), sp)) for b in bs]
            nbytes = m * k + n * k + 2 * m * n + (m + n) * k // 32
        elif kind == "nvfp4sw":  # gate/up GEMM (n = 2 * inter, interleaved rows) with SwiGLU + NVFP4 re-pack in the epilogue
            ws = L.gemm_workspace(L.OP_NVFP4, dev, m, n, k)
            a = a[:, :k // 2].contiguous()
            bs = [b[:, :k // 2].contiguous() for b in bs]
            sfa = torch.full((lib.rk_sf_bytes(m, k // 16),), 0x38, dtype=torch.uint8, device=dev)
            sfb = torch.full((lib.rk_sf_bytes(n, k // 16),), 0x38, dtype=torch.uint8, device=dev)
            q = torch.empty((m, n // 4), dtype=torch.uint8, device=dev)
            sfo = torch.empty(lib.rk_sf_bytes(m, n // 32), dtype=torch.uint8, device=dev)
            calls = [(lambda sp, b=b: lib.rk_gemm_nvfp4_swiglu(L.ptr(a), L.ptr(sfa), None, L.ptr(b), L.ptr(sfb), None, L.ptr(q),
                                                                L.ptr(sfo), m, n, k, tactic, L.ptr(ws), ws.numel(), sp)) for b in bs]
            nbytes = (m * k + n * k) // 2 + m * n // 4 + (m + n) * k // 16 + m * n // 32
        elif kind == "mxfp8sw":  # MXFP8 gate/up GEMM with the table-SiLU SwiGLU producer + MXFP8 re-pack in the epilogue
            ws = L.gemm_workspace(L.OP_MXFP8, dev, m, n, k)
            sfa = torch.full((lib.rk_sf_bytes(m, k // 32),), 127, dtype=torch.uint8, device=dev)
            sfb = torch.full((lib.rk_sf_bytes(n, k // 32),), 127, dtype=torch.uint8, device=dev)
            raw = torch.arange(65536, device=dev, dtype=torch.int32).to(torch.uint16)
            table = torch.nn.functional.silu(raw.view(torch.bfloat16)).contiguous()
            q = torch.empty((m, n // 2), dtype=torch.uint8, device=dev)
            sfo = torch.empty(lib.rk_sf_bytes(m, n // 64), dtype=torch.uint8, device=dev)
            calls = [(lambda sp, b=b: lib.rk_gemm_mxfp8_swiglu(L.ptr(a), L.ptr(sfa), L.ptr(b), L.ptr(sfb), L.ptr(table), L.ptr(q),
                                                                L.ptr(sfo), m, n, k, tactic, L.ptr(ws), ws.numel(), sp)) for b in bs]
            nbytes = m * k + n * k + m * n // 2 + (m + n) * k // 32 + m * n // 64
        elif kind == "fp8p":  # bf16 activations converted inside the kernel
            ws = L.gemm_workspace(L.OP_FP8, dev, m, n, k)
            x = torch.randn(m, k, device=dev).to(torch.bfloat16)
            calls = [(lambda sp, b=b: lib.rk_gemm_fp8_producer(L.ptr(x), L.ptr(b), L.ptr(one), None, L.ptr(out), m, n, k,
                                                               tactic, L.ptr(ws), ws.numel(), sp)) for b in bs]
            nbytes = 2 * m * k + n * k + 2 * m * n
        elif kind == "w4a8":  # MXFP4 weights expanded inside the kernel, MXFP8 activations
            ws = L.gemm_workspace(L.OP_MXFP8, dev, m, n, k)
            bs = [b[:, :k // 2].contiguous() for b in bs]
            sfa = torch.full((lib.rk_sf_bytes(m, k // 32),), 127, dtype=torch.uint8, device=dev)
            sfb = torch.full((lib.rk_sf_bytes(n, k // 32),), 127, dtype=torch.uint8, device=dev)
            calls = [(lambda sp, b=b: lib.rk_gemm_w4a8_mx(L.ptr(a), L.ptr(sfa), L.ptr(b), L.ptr(sfb), None, L.ptr(out), m, n,
                                                          k, tactic, L.ptr(ws), ws.numel(), sp)) for b in bs]
            nbytes = m * k + n * k // 2 + 2 * m * n + (m + n) * k // 32
        elif kind == "w4a4":  # both operands packed int4, widened inside the kernel
            ws = L.gemm_workspace(L.OP_W8A8, dev, m, n, k)
            a4 = a[:, :k // 2].contiguous()
            bs = [b[:, :k // 2].contiguous() for b in bs]
            sa, sb = torch.rand(m, device=dev), torch.rand(n, device=dev)
            calls = [(lambda sp, b=b: lib.rk_gemm_int(L.ptr(a4), L.ptr(sa), L.ptr(b), L.ptr(sb), None, L.ptr(out), m, n, k, 4,
                                                      tactic, L.ptr(ws), ws.numel(), sp)) for b in bs]
            nbytes = (m * k + n * k) // 2 + 2 * m * n
        else:
            ws = L.gemm_workspace(L.OP_NVFP4, dev, m, n, k)
            a = a[:, :k // 2].contiguous()
            bs = [b[:, :k // 2].contiguous() for b in bs]
            sfa = torch.full((lib.rk_sf_bytes(m, k // 16),), 0x38, dtype=torch.uint8, device=dev)
            sfb = torch.full((lib.rk_sf_bytes(n, k // 16),), 0x38, dtype=torch.uint8, device=dev)
            calls = [(lambda sp, b=b: lib.rk_gemm_nvfp4(L.ptr(a), L.ptr(sfa), None, L.ptr(b), L.ptr(sfb), None, None,
                                                        L.ptr(out), m, n, k, tactic, L.ptr(ws), ws.numel(), sp)) for b in bs]
            nbytes = (m * k + n * k) // 2 + 2 * m * n + (m + n) * k // 16
        self.report(kind, m, n, k, tactic, self.time_us(calls), nbytes, 2 * m * n * k, "TFLOPS", ws)

    def w4a16(self, m, n, k, tactic=0):
        dev, lib = self.dev, self.lib
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        qs = [torch.randint(0, 255, (n, k // 2), dtype=torch.uint8, device=dev) for _ in range(self.copies(n * k // 2))]
        sc = torch.rand(k // 128, n, device=dev).to(torch.bfloat16)
        out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
        ws = L.gemm_workspace(L.OP_W4A16, dev, m, n, k)
        calls = [(lambda sp, q=q: lib.rk_gemm_w4a16_g128(L.ptr(x), L.ptr(q), L.ptr(sc), None, L.ptr(out), m, n, k, tactic,
                                                         L.ptr(ws), ws.numel(), sp)) for q in qs]
        nbytes = n * k // 2 + k // 128 * n * 2 + 2 * m * k + 2 * m * n
        self.report("w4a16", m, n, k, tactic, self.time_us(calls), nbytes, 2 * m * n * k, "TFLOPS", ws)

    def quant_rows(self, rows, k, bits=8):
        dev, lib = self.dev, self.lib
        xs = [torch.randn(rows, k, device=dev).to(torch.bfloat16) for _ in range(self.copies(rows * k * 2))]
        kp = (k + 127) // 128 * 128
        q = torch.empty((rows, kp), dtype=torch.uint8, device=dev)
        s = torch.empty(rows, device=dev)
        calls = [(lambda sp, x=x: lib.rk_quant_rows(L.ptr(x), rows, k, k, None, 0, None, 0, bits, L.ptr(q), L.ptr(s), sp))
                 for x in xs]
        us = self.time_us(calls)
        nbytes = rows * k * 3
        print(f"quant  rows{rows:6d} k{k:6d} int{bits}: {us:8.2f} us  {nbytes / us / 1e3:8.1f} GB/s "
              f"({nbytes / us / 1e3 / self.hbm * 100:5.1f}% of {self.hbm_src} copy bw)", flush=True)


def swiglu_pack(bench, rows, inter, interleaved=1):
    """SwiGLU -> NVFP4 pack of a bf16 [rows, 2 * inter] gate/up tensor (the second launch of the two-launch MLP path)."""
    dev, lib = bench.dev, bench.lib
    xs = [torch.randn(rows, 2 * inter, device=dev).to(torch.bfloat16) for _ in range(bench.copies(rows * inter * 4))]
    q = torch.empty((rows, inter // 2), dtype=torch.uint8, device=dev)
    sf = torch.empty(lib.rk_sf_bytes(rows, inter // 16), dtype=torch.uint8, device=dev)
    calls = [(lambda sp, x=x: lib.rk_swiglu_pack_nvfp4_layout(L.ptr(x), rows, inter, interleaved, L.ptr(q), L.ptr(sf), sp)) for x in xs]
    us = bench.time_us(calls)
    nbytes = rows * inter * 4 + rows * inter // 2 + rows * inter // 16
    print(f"swiglu_pack rows{rows:6d} inter{inter:6d}: {us:8.2f} us  {nbytes / us / 1e3:8.1f} GB/s "
          f"({nbytes / us / 1e3 / bench.hbm * 100:5.1f}% of {bench.hbm_src} copy bw)", flush=True)


def layer_breakdown(envs=8, prefix=816, repeats=5):
    """Device time per kernel of ONE decoder layer of the action expert (width 1024, MLP 4096, 50
    action tokens x `envs` environments attending to `prefix` cached tokens), eager launches under
    the torch profiler: the bf16 layer, then the W8A8 layer with every option the benchmark's
    chunk loop uses (grouped projections as views, fused gated-residual + adaRMSNorm + quantizer,
    rotary embedding + cache append kernel, cached condition projections)."""
    from torch.profiler import ProfilerActivity, profile

    from rk_b200.gemma_stack import (ActionExpert, GemmaAttention, expert_scope, fuse_norm_quantize, rope_tables,
                                     unfuse_norm_quantize)
    from rk_b200.optimizations import quantize_linears

    dev = torch.device("cuda:0")
    expert = ActionExpert().init_random(0).to(dev).eval()
    cfg = expert.cfg
    gen = torch.Generator().manual_seed(7)
    x = torch.randn(envs, expert.chunk, cfg.width, generator=gen).to(torch.bfloat16).to(dev)
    branch = torch.randn(envs, expert.chunk, cfg.width, generator=gen).to(torch.bfloat16).to(dev)
    cond = torch.randn(envs, cfg.width, generator=gen).to(dev)
    k_all = torch.randn(envs, cfg.num_kv_heads, prefix + expert.chunk, cfg.head_dim, generator=gen).to(torch.bfloat16).to(dev)
    v_all = torch.randn(k_all.shape, generator=gen).to(torch.bfloat16).to(dev)
    positions = prefix + torch.arange(expert.chunk, device=dev)[None].expand(envs, -1)
    layer = expert.stack.layers[1]
    expert.enable_condition_caches()
    expert._conditions[("probe",)] = cond  # registers the condition, so that its projections are cached
    GemmaAttention.fused_rope = True

    pitch = (prefix + expert.chunk + 7) // 8 * 8
    vt_all = torch.zeros((envs, cfg.num_kv_heads, cfg.head_dim, pitch), dtype=torch.bfloat16, device=dev)
    vt_all[..., :prefix + expert.chunk] = v_all.transpose(-1, -2)

    def run(tag):
        with torch.no_grad():
            cos, sin = rope_tables(positions, cfg.head_dim, cfg.rope_theta, x.dtype)
            gate = layer.input_layernorm.modulation(cond)[2]
            step = lambda: layer(x, cos, sin, (k_all, v_all, prefix, vt_all), cond, (branch, gate))
            for _ in range(3):
                step()
            torch.cuda.synchronize()
            with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
                for _ in range(repeats):
                    step()
                torch.cuda.synchronize()
        rows = [(e.key, e.count, e.device_time_total) for e in prof.key_averages()
                if e.device_time_total > 0 and e.device_type == torch.autograd.DeviceType.CUDA]
        rows.sort(key=lambda r: -r[2])
        total = sum(r[2] for r in rows)
        print(f"--- {tag}: {total / repeats:.1f} us of device time per layer ({envs} x {expert.chunk} tokens, prefix {prefix})")
        for key, count, t in rows:
            print(f"{t / repeats:8.1f} us  x{count / repeats:4.1f}  {key[:120]}")

    try:
        run("bf16 linears")
        with quantize_linears(expert, "int8", scopes=("expert",), selector=expert_scope, shared_quant=True, grouped=True,
                              group_views=True):
            norms = fuse_norm_quantize(expert.stack)
            run("W8A8 linears, grouped, fused norm / residual / rope, torch SDPA")
            GemmaAttention.fused_attention = True
            run("W8A8 linears, grouped, fused norm / residual / rope, rk_attn_prefix_kernel")
            unfuse_norm_quantize(norms)
    finally:
        GemmaAttention.fused_rope = False
        GemmaAttention.fused_attention = False


def prefix_layer_breakdown(tokens=816, depth=2, repeats=5):
    """Per-kernel device time of one layer of the cfg4 prefix stack (Gemma-2B widths, every linear NVFP4
    with the fp32 per-tensor scale, shared packs): tensor-op elementwise work against the fused form
    (norm + amax kernel, GELU * up + amax kernel, rotary embedding into preallocated caches)."""
    from dataclasses import replace

    from torch.profiler import ProfilerActivity, profile

    from rk_b200.gemma_stack import GemmaStack, fuse_norm_pack_fp4, gemma_2b, prefix_scope, unfuse_norm_quantize
    from rk_b200.optimizations import quantize_linears

    dev = torch.device("cuda:0")
    cfg = replace(gemma_2b(), depth=depth)
    model = GemmaStack(cfg).to(torch.bfloat16).init_random(1).to(dev).eval()
    x = torch.randn(1, tokens, cfg.width, device=dev).to(torch.bfloat16)
    pos = torch.arange(tokens, device=dev)[None]
    caches = [tuple(torch.zeros(1, cfg.num_kv_heads, tokens, cfg.head_dim, dtype=torch.bfloat16, device=dev)
                    for _ in range(2)) + (0,) for _ in range(depth)]

    def run(tag, past):
        with torch.no_grad():
            for _ in range(3):
                model(x, pos, past=past)
            torch.cuda.synchronize()
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                for _ in range(repeats):
                    model(x, pos, past=past)
                torch.cuda.synchronize()
        rows = [(e.device_time_total / repeats / depth, e.count / repeats / depth, e.key) for e in prof.key_averages()
                if e.device_time_total > 0]
        rows.sort(reverse=True)
        print(f"--- {tag}: {sum(r[0] for r in rows):.1f} us of device time per layer ({tokens} tokens)")
        for t, count, key in rows[:16]:
            print(f"{t:8.1f} us  x{count:4.1f}  {key[:120]}")

    with quantize_linears(model, "fp4", scopes=("text",), selector=prefix_scope, fp4_global_scale=True, shared_quant=True):
        downs = [layer.mlp.down_proj for layer in model.layers]
        for m in downs:  # tensor-op GELU * up in front of the down projection, as the reference's harness runs it
            m.forward_gelu = lambda gate, up, m=m: m(torch.nn.functional.gelu(gate, approximate="tanh") * up)
        run("NVFP4 linears, tensor-op norms / GELU / rotary embedding", None)
        for m in downs:
            del m.forward_gelu
        norms = fuse_norm_pack_fp4(model)
        for layer in model.layers:
            layer.self_attn.fused_rope = True
        run("NVFP4 linears, fused norm + amax, GELU * up + amax, rotary embedding into caches", caches)
        unfuse_norm_quantize(norms)


def main(argv):
    which = argv or ["w4a16", "w8a8", "fp8", "mxfp8", "nvfp4", "quant"]
    b = Bench()
    # one explicit shape: "w8a8:400x8192x1024", "w4a16:8x16384x2048", "fp8:...", "quant:16384x2048"
    for spec in [a for a in which if ":" in a]:
        kind, dims = spec.split(":")
        dims = [int(d) for d in dims.split("x")]
        if kind == "quant":
            b.quant_rows(*dims)
        elif kind == "swiglu_pack":
            swiglu_pack(b, *dims)
        elif kind == "w4a16":
            b.w4a16(*dims)
        elif kind == "w8a8":
            b.w8a8(*dims)
        else:
            b.float8(kind, *dims)
    which = [a for a in which if ":" not in a]
    if "layer" in which:
        layer_breakdown()
        return
    if "prefix_layer" in which:
        prefix_layer_breakdown()
        return
    if "w4a16" in which:
        for m in (1, 8, 50, 128, 256):
            b.w4a16(m, 16384, 2048)
    if "w8a8" in which:
        for shape in ((64, 2048, 2048), (400, 2560, 1024), (400, 1024, 2048), (400, 8192, 1024), (400, 1024, 4096),
                      (1764, 2048, 2048), (1764, 8192, 2048), (1764, 2048, 8192), (1764, 6144, 2048), (4096, 8192, 8192)):
            b.w8a8(*shape)
    for kind in ("fp8", "mxfp8", "nvfp4"):
        if kind in which:
            for shape in ((50, 16384, 2048), (256, 16384, 2048), (816, 16384, 2048), (816, 2048, 16384), (816, 2048, 2048),
                          (4096, 8192, 8192)):
                b.float8(kind, *shape)
    if "quant" in which:
        for rows, k in ((64, 2048), (400, 1024), (400, 4096), (1764, 2048), (1764, 8192), (16384, 2048)):
            b.quant_rows(rows, k)


if __name__ == "__main__":
    main(sys.argv[1:])
