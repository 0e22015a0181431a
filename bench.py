#!/usr/bin/env python3
"""Throughput benchmark of the quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload ``cfg2_w4a16_g128``: the W4A16 group-wise int4 GEMM of the Gemma-2B MLP gate/up
shape (N=16384, K=2048, group 128) at M in {1, 8, 50, 256}.  One step = one pass over the four
activation batches (four GEMM launches).  Weights rotate through enough independent copies that
the working set exceeds the 126 MB L2, so a launch streams its weights from HBM.

Prints ONE JSON line (rank 0).  ``value`` is whole-job TOPS with inputs resident in HBM; ``e2e``
is the same metric through the public Linear module with host activations (H2D copy, GEMM, D2H
copy inside the timed region); ``roofline`` describes the dominant kernel; ``cpu_baseline`` is
the CPU oracle port of the same operator timed on the host cores over a bounded sample.

``--impl reference`` times the CPU implementation only (the reference's quantized path has no
CPU build of its own; the oracle port stands in), on rank 0.
"""

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "robotics-the-speedup-paradox_b200"))

import numpy as np
import torch

L2_BYTES = 126 * 1024 * 1024
N, K, GROUP = 16384, 2048, 128
M_LIST = (1, 8, 50, 256)


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def algorithmic_bytes(m):
    """Bytes one W4A16 launch must move: packed weights + group scales + activations + output."""
    return N * K // 2 + (K // GROUP) * N * 2 + m * K * 2 + m * N * 2


# DRAM bytes (read + write) of one launch, from an ncu capture of this workload's four launches
# (dram__bytes_read.sum + dram__bytes_write.sum; the outputs stay in L2, so writes were zero).
NCU_DRAM_TRAFFIC = {1: 17330432, 8: 17373952, 50: 17549312, 256: 18384896}


def algorithmic_ops(m):
    return 2 * m * N * K


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        mhz, reasons, mx = [], set(), None
        for s in self.samples:
            try:
                mhz.append(float(s[0]))
                mx = float(s[1])
            except ValueError:
                continue
            for name, flag in zip(names, s[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(mhz)) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


def make_inputs(device, copies, seed):
    """Seeded synthetic weights (N(0, 0.02)) and activations (N(0, 1)); weights packed on the GPU."""
    from rk_b200.w4a16_linear import pack_weight

    gen = torch.Generator(device="cpu").manual_seed(seed)
    weights = []
    for _ in range(copies):
        w = (torch.randn(N, K, generator=gen) * 0.02).to(torch.bfloat16).to(device)
        weights.append(pack_weight(w))
        del w
    xs = {m: torch.randn(m, K, generator=gen).to(torch.bfloat16).to(device) for m in M_LIST}
    return weights, xs


def cpu_port_once(x, packed, scales):
    """The oracle port on host cores: dequantize (int4 codes x bf16 group scales) then fp32 matmul."""
    from oracle import w4a16 as OW

    w = torch.from_numpy(OW.dequantize(packed, scales))
    return (torch.from_numpy(x) @ w.T).to(torch.bfloat16)


def time_cpu_baseline(budget_s=12.0):
    """Bounded sample: full-size weights, every M of the workload, as many passes as fit the budget."""
    from oracle import w4a16 as OW
    from oracle.formats import bf16_round

    torch.set_num_threads(os.cpu_count() or 1)
    rng = np.random.default_rng(42)
    w = bf16_round((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    packed, scales, _ = OW.pack_weight(w)
    xs = {m: bf16_round(rng.standard_normal((m, K)).astype(np.float32)) for m in M_LIST}
    cpu_port_once(xs[1], packed, scales)  # warm-up
    ops, elapsed, passes = 0, 0.0, 0
    while elapsed < budget_s and passes < 8:
        t0 = time.perf_counter()
        for m in M_LIST:
            cpu_port_once(xs[m], packed, scales)
        elapsed += time.perf_counter() - t0
        ops += sum(algorithmic_ops(m) for m in M_LIST)
        passes += 1
    return {"value": ops / elapsed / 1e12, "unit": "TOPS", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{passes} full passes of the workload (dequantize + fp32 matmul per launch), "
                      f"{elapsed:.1f} s of CPU time"}, elapsed / passes


def run_reference(args, rank, budget_s=150.0):
    """CPU arm: the oracle port on the host cores.  A step is one pass over the four activation
    batches against a SAMPLE of the weight matrix - the first `rows` output channels - sized so that
    warm-up plus timed steps fit `budget_s`; throughput counts only the operations actually done."""
    if rank != 0:
        return
    from oracle import w4a16 as OW
    from oracle.formats import bf16_round

    _, full_pass_s = time_cpu_baseline(budget_s=4.0)  # warms caches and the thread pool, times a full pass
    total_steps = args.warmup + args.steps
    frac = min(1.0, budget_s / (total_steps * full_pass_s))
    rows = int(min(N, max(GROUP, round(N * frac / GROUP) * GROUP)))
    rng = np.random.default_rng(42)
    w = bf16_round((rng.standard_normal((rows, K)) * 0.02).astype(np.float32))
    packed, scales, _ = OW.pack_weight(w)
    xs = {m: bf16_round(rng.standard_normal((m, K)).astype(np.float32)) for m in M_LIST}
    steps_t = []
    for i in range(total_steps):
        t0 = time.perf_counter()
        for m in M_LIST:
            cpu_port_once(xs[m], packed, scales)
        if i >= args.warmup:
            steps_t.append(time.perf_counter() - t0)
    total = sum(steps_t)
    ops = sum(2 * m * rows * K for m in M_LIST) * args.steps
    value = ops / total / 1e12
    sample = (f"each step covers the first {rows} of {N} output channels at every M "
              f"({100.0 * rows / N:.1f}% of the workload's operations), {total:.1f} s of CPU time in {args.steps} steps")
    line = {
        "impl": "reference", "metric": "quantized_gemm_tops", "value": value, "unit": "TOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int4xbf16->f32",
        "data": "synthetic", "config": workload_config(default_copies()),
        "cpu_baseline": {"value": value, "unit": "TOPS", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def default_copies():
    """Independent weight copies the GPU arm rotates through: working set comfortably above L2."""
    return L2_BYTES // (N * K // 2 + (K // GROUP) * N * 2) + 5


def chunk_latency(device, reps=13, warmups=5, envs=8, prefix_len=816):
    """p50 wall-clock latency of one action chunk: the 10-step flow-matching loop of a random-init
    18-layer Gemma-architecture expert (width 1024, MLP 4096), all bf16 linears swapped for W8A8,
    the whole loop replayed from one CUDA graph, `envs` independent environments per GPU attending
    to a cached bf16 prefix KV of `prefix_len` tokens."""
    from rk_b200.gemma_stack import (ActionExpert, GemmaAttention, expert_scope, fuse_norm_quantize,
                                     unfuse_norm_quantize)
    from rk_b200.graph import CudaGraphCall
    from rk_b200.optimizations import quantize_linears

    expert = ActionExpert().init_random(0).to(device).eval()
    # the reference's condition_cache / condition_projection_cache switches, in both arms: the
    # timestep conditions of the fixed 10-step schedule and the adaptive norms' dense(condition)
    # are computed during the eager warm-up calls and are constants of the captured graph
    expert.enable_condition_caches()
    GemmaAttention.fused_rope = True  # rotary embedding + cache append as one kernel, in both arms
    cfg = expert.cfg
    gen = torch.Generator().manual_seed(7)
    noise = torch.randn(envs, expert.chunk, expert.action_dim, generator=gen).to(device)
    shape = (cfg.depth, envs, cfg.num_kv_heads, prefix_len, cfg.head_dim)
    pk = torch.randn(shape, generator=gen).to(torch.bfloat16).to(device)
    pv = torch.randn(shape, generator=gen).to(torch.bfloat16).to(device)

    def measure(fn):
        with torch.no_grad():
            call = CudaGraphCall(fn, retained_tensors=expert.retained_tensors)
            for _ in range(warmups):
                call(noise, pk, pv)
            torch.cuda.synchronize(device)
            samples = []
            for _ in range(reps):
                t0 = time.perf_counter()
                call(noise, pk, pv)
                torch.cuda.synchronize(device)
                samples.append((time.perf_counter() - t0) * 1e3)
        return float(np.median(samples)), samples

    bf16_ms, _ = measure(lambda n, k, v: expert(n, k, v))
    # group_views: the slices of a grouped projection stay views of its output (the rope kernel and
    # the GELU*up quantizer take row-strided inputs), instead of one copy per slice
    with quantize_linears(expert, "int8", scopes=("expert",), selector=expert_scope, shared_quant=True,
                          grouped=True, group_views=True) as report:
        norms = fuse_norm_quantize(expert.stack)  # adaRMSNorm + modulation + row quantizer as one kernel
        int8_ms, samples = measure(lambda n, k, v: expert(n, k, v))
        unfuse_norm_quantize(norms)
        swapped = len(report["modules"])
        groups = len(report["grouped"])
    GemmaAttention.fused_rope = False
    return {"p50_ms": int8_ms, "bf16_p50_ms": bf16_ms, "chunks_per_s": envs / (int8_ms * 1e-3), "envs": envs,
            "steps": expert.steps, "prefix_len": prefix_len, "linears_w8a8": swapped, "projection_groups": groups, "fused_norm_quantizers": len(norms),
            "fused_rope_cache_update": True, "cached_conditions": len(expert._conditions),
            "cached_condition_projections": sum(len(n.projection_cache) for n in expert.adaptive_norms()), "reps": reps,
            "timing": "wall clock around CudaGraphCall (input copy, graph replay, output clone), synchronised"}


def column_parallel_leg(info, device, reps=30):
    """Auxiliary multi-GPU figure (only under a multi-rank launch): the widest projection of the
    prefix pass (FP8, M=816, N=16384, K=2048) split along N over the ranks, each rank computing its
    [M, N/G] slab, then one NCCL all-gather.  Reported beside the same GEMM on one GPU."""
    from rk_b200 import replicas
    from rk_b200.fp8_linear import Fp8CutlassLinear

    m, n, k = 816, 16384, 2048
    gen = torch.Generator().manual_seed(3)  # the same layer on every rank
    full = torch.nn.Linear(k, n, bias=False, dtype=torch.bfloat16)
    with torch.no_grad():
        full.weight.copy_((torch.randn(n, k, generator=gen) * 0.02).to(torch.bfloat16))
    full = full.to(device).requires_grad_(False)
    x = torch.randn(m, k, generator=gen).to(torch.bfloat16).to(device)
    make = lambda lin: Fp8CutlassLinear.from_linear(lin, "linear", "gate_up")
    sharded = replicas.ColumnParallelLinear(full, info, make)
    single = make(full)

    def timed(fn):
        for _ in range(3):
            fn()
        replicas.barrier(info, device)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize(device)
        return a.elapsed_time(b) / reps * 1e3

    with torch.no_grad():
        us_sharded = timed(lambda: sharded(x))
        us_single = timed(lambda: single(x))
        a, b = sharded(x).float(), single(x).float()
        rel = float((a - b).norm() / b.norm())  # slabs carry their own per-tensor weight scale
    us_sharded, us_single = replicas.max_over_ranks([us_sharded, us_single], info, device)
    return {"op": "fp8 linear (dynamic activation scale) M=816 N=16384 K=2048", "ranks": info.world,
            "us_column_parallel_with_all_gather": us_sharded, "us_one_gpu": us_single,
            "rel_frobenius_vs_one_gpu": rel, "collective": "nccl all_gather_into_tensor of bf16 slabs"}


def workload_config(copies):
    return {"workload": "cfg2_w4a16_g128", "N": N, "K": K, "group": GROUP, "M": list(M_LIST),
            "launches_per_step": len(M_LIST), "timing": "CUDA events around CUDA-graph replays",
            "l2": f"inputs larger than L2: weights rotate through {copies} copies "
                  f"({copies * (N * K // 2 + (K // GROUP) * N * 2) / 1e6:.0f} MB > 126 MB)"}


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=6000)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="cfg2_w4a16_g128", choices=["cfg2_w4a16_g128"])
    parser.add_argument("--skip-cpu", action="store_true", help="omit the cpu_baseline leg")
    parser.add_argument("--skip-chunk", action="store_true", help="omit the action-chunk latency leg")
    parser.add_argument("--no-graphs", action="store_true",
                        help="launch the timed steps directly instead of replaying CUDA graphs (for profilers; "
                             "host launch cost then sits inside the timed region)")
    args = parser.parse_args()
    if args.warmup < 3:
        args.warmup = 3

    from rk_b200 import replicas

    info = replicas.rank_info()
    rank, world, local_rank = info.rank, info.world, info.local_rank

    if args.impl == "reference":
        run_reference(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    from rk_b200 import _lib
    from rk_b200.w4a16_linear import W4A16Linear, linear_w4a16

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    replicas.init(info, device)

    copies = default_copies()
    weights, xs = make_inputs(device, copies, seed=42 + rank)
    outs = {m: torch.empty((m, N), device=device, dtype=torch.bfloat16) for m in M_LIST}
    lib = _lib.load()
    ws = _lib.gemm_workspace(_lib.OP_W4A16, device, max(M_LIST), N, K)
    stream = torch.cuda.current_stream(device)
    sp = _lib.stream_ptr(device)
    launches = 0

    def launch(m, copy):
        nonlocal launches
        q, s = weights[copy]
        code = lib.rk_gemm_w4a16_g128(_lib.ptr(xs[m]), _lib.ptr(q), _lib.ptr(s), None, _lib.ptr(outs[m]), m, N, K, 0,
                                      _lib.ptr(ws), ws.numel(), sp)
        if code != 0:
            raise RuntimeError(_lib.last_error())
        launches += 1

    def step(i):
        for j, m in enumerate(M_LIST):
            launch(m, (i * len(M_LIST) + j) % copies)

    def barrier():
        replicas.barrier(info, device)

    def capture(first_step, count):
        """One CUDA graph holding `count` consecutive steps (host launch cost stays out of the timing)."""
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(device)
        side.wait_stream(stream)
        with torch.cuda.graph(graph, stream=side):
            sp_side = _lib.stream_ptr(device)
            for i in range(count):
                for j, m in enumerate(M_LIST):
                    q, s = weights[((first_step + i) * len(M_LIST) + j) % copies]
                    code = lib.rk_gemm_w4a16_g128(_lib.ptr(xs[m]), _lib.ptr(q), _lib.ptr(s), None, _lib.ptr(outs[m]),
                                                  m, N, K, 0, _lib.ptr(ws), ws.numel(), sp_side)
                    if code != 0:
                        raise RuntimeError(_lib.last_error())
        stream.wait_stream(side)
        return graph

    for i in range(args.warmup):
        step(i)
    barrier()
    # the timed region replays graphs of `copies` steps (one full rotation of the weight copies)
    # plus one graph with the remainder, so that exactly args.steps steps run
    full, rest = divmod(args.steps, copies)
    cycle = tail = None
    if not args.no_graphs:
        cycle = capture(0, copies)
        tail = capture(0, rest) if rest else None
        cycle.replay()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        deadline = time.perf_counter() + 3.0  # the first sample marks that sampling is live
        while not sampler.samples and time.perf_counter() < deadline:
            time.sleep(0.02)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record(stream)
    if args.no_graphs:
        for i in range(args.steps):
            step(i)
    else:
        for _ in range(full):
            cycle.replay()
        if tail is not None:
            tail.replay()
    stop.record(stream)
    barrier()
    elapsed_ms = start.elapsed_time(stop)
    timed_launches = args.steps * len(M_LIST)
    status = _lib.read_status(ws)

    # per-kernel launch durations, measured live: a graph of `inner` back-to-back launches of one
    # shape (rotating weights) between two events on the launching stream
    inner = copies * 4
    per_m_ms = {}
    for m in M_LIST:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if args.no_graphs:
            torch.cuda.synchronize(device)
            a.record(stream)
            for c in range(inner):
                launch(m, c % copies)
            b.record(stream)
            torch.cuda.synchronize(device)
            per_m_ms[m] = a.elapsed_time(b) / inner
            continue
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(device)
        side.wait_stream(stream)
        with torch.cuda.graph(graph, stream=side):
            sp_side = _lib.stream_ptr(device)
            for c in range(inner):
                q, s = weights[c % copies]
                lib.rk_gemm_w4a16_g128(_lib.ptr(xs[m]), _lib.ptr(q), _lib.ptr(s), None, _lib.ptr(outs[m]), m, N, K, 0,
                                       _lib.ptr(ws), ws.numel(), sp_side)
        stream.wait_stream(side)
        graph.replay()
        torch.cuda.synchronize(device)
        a.record(stream)
        for _ in range(3):
            graph.replay()
        b.record(stream)
        torch.cuda.synchronize(device)
        per_m_ms[m] = a.elapsed_time(b) / (3 * inner)

    # end to end through the public module: pinned host activations in, host result out
    layers = [W4A16Linear(q, s, None, K, N) for (q, s) in weights]
    host_x = {m: xs[m].cpu().pin_memory() for m in M_LIST}
    host_out = {m: torch.empty((m, N), dtype=torch.bfloat16).pin_memory() for m in M_LIST}
    dev_x = {m: torch.empty_like(xs[m]) for m in M_LIST}

    def e2e_step(i):
        for j, m in enumerate(M_LIST):
            dev_x[m].copy_(host_x[m], non_blocking=True)
            y = layers[(i * len(M_LIST) + j) % copies](dev_x[m])
            host_out[m].copy_(y, non_blocking=True)
        torch.cuda.synchronize(device)

    e2e_steps = max(10, min(args.steps, 100))
    for i in range(3):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    barrier()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None

    # second half of the headline metric: p50 action-chunk latency of the W8A8 expert loop
    chunk = None
    if not args.skip_chunk:
        chunk = chunk_latency(device)
        if world > 1:
            (worst,) = replicas.max_over_ranks([chunk["p50_ms"]], info, device)
            chunk["p50_ms_max_over_ranks"] = worst
            chunk["box_chunks_per_s"] = replicas.whole_job_rate(chunk["envs"], info, worst)

    elapsed_ms, e2e_ms = replicas.max_over_ranks([elapsed_ms, e2e_s * 1e3], info, device)
    column_parallel = column_parallel_leg(info, device) if world > 1 else None

    step_ops = sum(algorithmic_ops(m) for m in M_LIST)
    value = replicas.whole_job_rate(step_ops * args.steps, info, elapsed_ms) / 1e12
    e2e_value = replicas.whole_job_rate(step_ops * e2e_steps, info, e2e_ms) / 1e12

    if rank == 0:
        peaks = load_peaks()
        dominant = max(M_LIST, key=lambda m: per_m_ms[m])
        per_case = {}
        for m in M_LIST:
            t = per_m_ms[m] * 1e-3
            per_case[f"M{m}"] = {
                "us": per_m_ms[m] * 1e3, "tops": algorithmic_ops(m) / t / 1e12,
                "gbs": algorithmic_bytes(m) / t / 1e9, "hbm_frac": algorithmic_bytes(m) / t / 1e9 / peaks["hbm_gbs"],
                "bf16_frac": algorithmic_ops(m) / t / 1e12 / peaks["bf16_tflops"],
            }
        d = per_case[f"M{dominant}"]
        hbm_bound = d["hbm_frac"] >= d["bf16_frac"]
        roofline = {
            "kernel": f"{'rk_gemm_w4a16_fold_kernel' if dominant > 64 else 'rk_gemm_w4a16_kernel'} (M={dominant})",
            "bound": "hbm" if hbm_bound else "tensor",
            "achieved": d["gbs"] if hbm_bound else d["tops"],
            "peak": peaks["hbm_gbs"] if hbm_bound else peaks["bf16_tflops"],
            "unit": "GB/s" if hbm_bound else "TFLOP/s",
            "frac": d["hbm_frac"] if hbm_bound else d["bf16_frac"],
            "traffic": NCU_DRAM_TRAFFIC.get(dominant),
            "peak_source": peaks["source"],
            "algorithmic_per_launch": algorithmic_bytes(dominant) if hbm_bound else algorithmic_ops(dominant),
        }
        cpu_baseline = None
        if not args.skip_cpu:
            cpu_baseline, _ = time_cpu_baseline()
        line = {
            "metric": "quantized_gemm_tops", "value": value, "unit": "TOPS", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int4xbf16->f32", "data": "synthetic",
            "config": workload_config(copies), "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "TOPS",
                    "h2d_bytes_per_step": sum(m * K * 2 for m in M_LIST),
                    "d2h_bytes_per_step": sum(m * N * 2 for m in M_LIST), "steps": e2e_steps},
            "gpu_launches": timed_launches, "roofline": roofline, "per_case": per_case,
            "cpu_baseline": cpu_baseline, "device_status": status, "action_chunk": chunk,
            "column_parallel": column_parallel,
        }
        print(json.dumps(line))
    replicas.finish()


if __name__ == "__main__":
    main()
