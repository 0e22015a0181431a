"""GPU tests of the Gemma-architecture harness around the quantized linears: per-linear parity of
the W8A8 path inside the action-expert loop, CUDA-graph replay of the whole loop, NVFP4 prefix."""

import numpy as np
import pytest
import torch

from oracle import formats as F
from oracle import integer as OI

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def H():
    import gpu_helpers

    return gpu_helpers


def small_expert(device):
    from rk_b200.gemma_stack import ActionExpert, GemmaConfig

    cfg = GemmaConfig(width=256, mlp_dim=512, depth=2, num_heads=2, num_kv_heads=1, head_dim=128, adarms_cond_dim=256)
    return ActionExpert(cfg, chunk=50, action_dim=32, steps=3).init_random(1).to(device).eval()


def test_expert_loop_w8a8_linears_match_oracle_and_graph_replays(H):
    from rk_b200.gemma_stack import expert_scope
    from rk_b200.graph import CudaGraphCall
    from rk_b200.integer import IntegerLinear
    from rk_b200.optimizations import quantize_linears

    expert = small_expert(H.DEVICE)
    b, t = 8, 96
    gen = torch.Generator().manual_seed(3)
    noise = torch.randn(b, 50, 32, generator=gen).to(H.DEVICE)
    pk = torch.randn(2, b, 1, t, 128, generator=gen).to(torch.bfloat16).to(H.DEVICE)
    pv = torch.randn(2, b, 1, t, 128, generator=gen).to(torch.bfloat16).to(H.DEVICE)
    with torch.no_grad():
        reference = expert(noise, pk, pv)
        with quantize_linears(expert, "int8", scopes=("expert",), selector=expert_scope) as report:
            assert len(report["modules"]) == 2 * 7 and not report["skipped"]
            # every swapped linear reproduces the oracle bit for bit on the activations it sees
            seen = {}
            hooks = [m.register_forward_hook(lambda mod, args, out, name=n: seen.__setitem__(name, (args[0], out)))
                     for n, m in expert.named_modules() if isinstance(m, IntegerLinear)]
            quantized = expert(noise, pk, pv)
            for hook in hooks:
                hook.remove()
            # down_proj runs through forward_gelu (fused GELU*up pack), which bypasses module hooks
            assert len(seen) == 12
            for name, (x, y) in seen.items():
                if getattr(x, "_robotics_packed_input", False):
                    continue
                layer = expert.get_submodule(name)
                xs = H.to_np(x).reshape(-1, layer.in_features)
                a, sa, _ = OI.quantize_rows(xs, 8)
                want, _ = OI.gemm(a, sa, layer.packed_weight.cpu().numpy(), layer.weight_scale.cpu().numpy(), None, 8)
                assert np.array_equal(H.bits(y).reshape(-1, layer.out_features), F.bf16_bits(want)), name
            # the whole loop under a captured graph equals eager execution, also after new inputs
            call = CudaGraphCall(lambda n_, k_, v_: expert(n_, k_, v_))
            assert torch.equal(call(noise, pk, pv), quantized)
            noise2 = torch.randn(b, 50, 32, generator=gen).to(H.DEVICE)
            assert torch.equal(call(noise2, pk, pv), expert(noise2, pk, pv))
            assert call.captures == 1 and call.replays == 2
    rel = (quantized - reference).norm() / reference.norm()
    assert rel < 0.1


def test_full_size_expert_every_linear_matches_oracle(H):
    """The benchmark's own expert - 18 layers, width 1024, MLP 4096, 8 heads of 256 over one KV head,
    8 environments x 50 action tokens against an 816-token prefix - for one denoising step: each of
    the 18 x 6 hooked W8A8 linears (q, k, v, o, gate, up) is held to the oracle bit for bit on the
    activations it actually saw (M = 400; N = 256 ... 4096; K = 1024 or 2048)."""
    from rk_b200.gemma_stack import ActionExpert, expert_scope
    from rk_b200.integer import IntegerLinear
    from rk_b200.optimizations import quantize_linears

    expert = ActionExpert(steps=1).init_random(2).to(H.DEVICE).eval()
    cfg = expert.cfg
    assert (cfg.depth, cfg.width, cfg.mlp_dim, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim) == (18, 1024, 4096, 8, 1, 256)
    envs, prefix = 8, 816
    gen = torch.Generator().manual_seed(5)
    noise = torch.randn(envs, expert.chunk, expert.action_dim, generator=gen).to(H.DEVICE)
    shape = (cfg.depth, envs, cfg.num_kv_heads, prefix, cfg.head_dim)
    pk = torch.randn(shape, generator=gen).to(torch.bfloat16).to(H.DEVICE)
    pv = torch.randn(shape, generator=gen).to(torch.bfloat16).to(H.DEVICE)
    with torch.no_grad():
        with quantize_linears(expert, "int8", scopes=("expert",), selector=expert_scope) as report:
            assert len(report["modules"]) == cfg.depth * 7 and not report["skipped"]
            seen = {}
            hooks = [m.register_forward_hook(lambda mod, args, out, name=n: seen.__setitem__(name, (args[0], out)))
                     for n, m in expert.named_modules() if isinstance(m, IntegerLinear)]
            out = expert(noise, pk, pv)
            for hook in hooks:
                hook.remove()
            torch.cuda.synchronize()
            assert torch.isfinite(out).all()
            checked = 0
            for name, (x, y) in seen.items():
                if getattr(x, "_robotics_packed_input", False):
                    continue
                layer = expert.get_submodule(name)
                xs = H.to_np(x).reshape(-1, layer.in_features)
                assert xs.shape[0] == envs * expert.chunk
                a, sa, _ = OI.quantize_rows(xs, 8)
                want, _ = OI.gemm(a, sa, layer.packed_weight.cpu().numpy(), layer.weight_scale.cpu().numpy(), None, 8)
                assert np.array_equal(H.bits(y).reshape(-1, layer.out_features), F.bf16_bits(want)), name
                checked += 1
            assert checked == cfg.depth * 6


def test_grouped_projections_and_fused_norm_quantizer_keep_the_loop_output(H):
    """Grouping q/k/v and gate/up into one GEMM each is exact; fusing adaRMSNorm + modulation + row
    quantizer into one kernel changes only the rounding of the normalized activations."""
    from rk_b200.gemma_stack import expert_scope, fuse_norm_quantize, unfuse_norm_quantize
    from rk_b200.optimizations import quantize_linears

    expert = small_expert(H.DEVICE)
    b, t = 4, 64
    gen = torch.Generator().manual_seed(5)
    noise = torch.randn(b, 50, 32, generator=gen).to(H.DEVICE)
    pk = torch.randn(2, b, 1, t, 128, generator=gen).to(torch.bfloat16).to(H.DEVICE)
    pv = torch.randn(2, b, 1, t, 128, generator=gen).to(torch.bfloat16).to(H.DEVICE)
    with torch.no_grad():
        with quantize_linears(expert, "int8", scopes=("expert",), selector=expert_scope, shared_quant=True) as _:
            plain = expert(noise, pk, pv)
        with quantize_linears(expert, "int8", scopes=("expert",), selector=expert_scope, shared_quant=True,
                              grouped=True) as report:
            assert len(report["grouped"]) == 2 * 2
            grouped = expert(noise, pk, pv)
            norms = fuse_norm_quantize(expert.stack)
            assert len(norms) == 2 * 2
            fused = expert(noise, pk, pv)
            unfuse_norm_quantize(norms)
            assert torch.equal(expert(noise, pk, pv), grouped)
    assert torch.equal(grouped, plain)  # same integer arithmetic, one GEMM instead of two or three
    rel = (fused - grouped).norm() / grouped.norm()
    assert rel < 2e-2


def test_residual_updates_in_the_gemm_epilogues_keep_the_loop_output(H):
    """The gated residual updates applied by the o_proj / down_proj epilogues (`rk_gemm_int_residual`)
    instead of inside the next norm kernel: the same three roundings, so the loop output is unchanged -
    with tensor-op norms and with the fused norm -> quantize kernels."""
    from rk_b200.gemma_stack import GemmaLayer, expert_scope, fuse_norm_quantize, unfuse_norm_quantize
    from rk_b200.optimizations import quantize_linears

    expert = small_expert(H.DEVICE)
    b, t = 4, 64
    gen = torch.Generator().manual_seed(6)
    noise = torch.randn(b, 50, 32, generator=gen).to(H.DEVICE)
    pk = torch.randn(2, b, 1, t, 128, generator=gen).to(torch.bfloat16).to(H.DEVICE)
    pv = torch.randn(2, b, 1, t, 128, generator=gen).to(torch.bfloat16).to(H.DEVICE)
    with torch.no_grad():
        with quantize_linears(expert, "int8", scopes=("expert",), selector=expert_scope, shared_quant=True, grouped=True):
            plain = expert(noise, pk, pv)
            norms = fuse_norm_quantize(expert.stack)
            fused = expert(noise, pk, pv)
            GemmaLayer.residual_epilogue = True
            try:
                assert torch.equal(expert(noise, pk, pv), fused)
                unfuse_norm_quantize(norms)
                assert torch.equal(expert(noise, pk, pv), plain)
            finally:
                GemmaLayer.residual_epilogue = False
                unfuse_norm_quantize(norms)
        GemmaLayer.residual_epilogue = True
        try:  # bf16 linears: the switch changes nothing
            assert torch.equal(expert(noise, pk, pv), expert(noise, pk, pv))
        finally:
            GemmaLayer.residual_epilogue = False


def test_condition_caches_and_chunk_buffers_under_graph_capture(H):
    """With the timestep conditions and their projections cached (filled by the eager warm-up
    calls) the captured loop reads them as constants: same output as the uncached eager loop, for
    the inputs of the capture and for new ones."""
    from rk_b200.gemma_stack import expert_scope, fuse_norm_quantize
    from rk_b200.graph import CudaGraphCall
    from rk_b200.optimizations import quantize_linears

    expert = small_expert(H.DEVICE)
    b, t = 4, 64
    gen = torch.Generator().manual_seed(11)
    noise = torch.randn(b, 50, 32, generator=gen).to(H.DEVICE)
    noise2 = torch.randn(b, 50, 32, generator=gen).to(H.DEVICE)
    pk = torch.randn(2, b, 1, t, 128, generator=gen).to(torch.bfloat16).to(H.DEVICE)
    pv = torch.randn(2, b, 1, t, 128, generator=gen).to(torch.bfloat16).to(H.DEVICE)
    with torch.no_grad():
        with quantize_linears(expert, "int8", scopes=("expert",), selector=expert_scope, shared_quant=True,
                              grouped=True) as _:
            fuse_norm_quantize(expert.stack)
            want, want2 = expert(noise, pk, pv), expert(noise2, pk, pv)
            expert.enable_condition_caches()
            call = CudaGraphCall(lambda n_, k_, v_: expert(n_, k_, v_), retained_tensors=expert.retained_tensors)
            assert torch.equal(call(noise, pk, pv), want)
            assert torch.equal(call(noise2, pk, pv), want2)
            assert call.captures == 1 and len(expert._conditions) == 3
            assert all(len(n.projection_cache) == 3 for n in expert.adaptive_norms())
            assert len(call._constants) == len(expert.retained_tensors()) > 0
            expert.disable_condition_caches()


@pytest.mark.parametrize("shape", [(2, 5, 3, 1, 32, 7), (8, 50, 8, 1, 256, 816), (1, 1, 2, 2, 128, 0), (3, 17, 4, 2, 512, 40)])
def test_rope_cache_update_kernel_matches_oracle_and_tensor_ops(H, shape):
    """One launch for rotary embedding + cache append: rotated queries and keys bit-identical to the
    oracle (and so to the bf16 tensor-op chain), values copied, every other cache row untouched;
    q, k, v given as slices of one projection output."""
    from oracle import rope as OR
    from rk_b200.gemma_stack import rope_cache_update, rope_tables

    b, t, heads, kv, d, prefix = shape
    gen = torch.Generator().manual_seed(13)
    width = (heads + 2 * kv) * d
    qkv = (torch.randn(b, t, width, generator=gen) * 2).to(torch.bfloat16).to(H.DEVICE)
    q, k, v = qkv[..., :heads * d], qkv[..., heads * d:(heads + kv) * d], qkv[..., (heads + kv) * d:]
    positions = prefix + torch.arange(t, device=H.DEVICE)[None].expand(b, -1)
    cos, sin = rope_tables(positions, d, 10000.0, torch.bfloat16)
    rows = prefix + t + 3
    k_all = torch.full((b, kv, rows, d), 5.0, dtype=torch.bfloat16, device=H.DEVICE)
    v_all = torch.full((b, kv, rows, d), 6.0, dtype=torch.bfloat16, device=H.DEVICE)
    q_out = rope_cache_update(q, k, v, cos, sin, k_all, v_all, prefix, heads, kv, d)
    kc, vc = np.full((b, kv, rows, d), 5.0, np.float32), np.full((b, kv, rows, d), 6.0, np.float32)
    want_q = OR.cache_update(H.to_np(q).reshape(b, t, heads, d), H.to_np(k).reshape(b, t, kv, d),
                             H.to_np(v).reshape(b, t, kv, d), H.to_np(cos), H.to_np(sin), kc, vc, prefix)
    assert np.array_equal(H.bits(q_out), F.bf16_bits(want_q))
    assert np.array_equal(H.bits(k_all), F.bf16_bits(kc))
    assert np.array_equal(H.bits(v_all), F.bf16_bits(vc))
    # and the tensor-op chain the harness runs without the kernel
    half = d // 2
    rot = lambda x: torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    q4 = q.reshape(b, t, heads, d).transpose(1, 2)
    assert torch.equal(q_out, q4 * cos[:, None] + rot(q4) * sin[:, None])
    # token-major storage: the same values as a transposed view of [B, t, heads, d]
    k2, v2 = torch.zeros_like(k_all), torch.zeros_like(v_all)
    q_tm = rope_cache_update(q, k, v, cos, sin, k2, v2, prefix, heads, kv, d, token_major=True)
    assert q_tm.shape == q_out.shape and q_tm.transpose(1, 2).is_contiguous() and torch.equal(q_tm, q_out)
    assert torch.equal(k2[:, :, prefix:prefix + t], k_all[:, :, prefix:prefix + t])


def test_rope_cache_update_refuses_bad_arguments(H):
    from rk_b200 import _lib

    lib = _lib.load()
    t = torch.zeros(4096, dtype=torch.bfloat16, device=H.DEVICE)
    p = _lib.ptr(t)
    call = lambda **kw: lib.rk_rope_cache_update(p, kw.get("qs", 64), p, 32, p, 32, p, p, 1, 2, 2, 1, kw.get("d", 32), p, 0, p,
                                                 p, kw.get("rows", 8), kw.get("prefix", 0), H.stream())
    assert call() == 0
    assert call(d=24) == _lib.RK_EINVAL       # head_dim not a multiple of 16
    assert call(qs=60) == _lib.RK_EINVAL      # row stride not a multiple of 8 elements
    assert call(qs=32) == _lib.RK_EINVAL      # row stride shorter than a row of two heads
    assert call(rows=8, prefix=7) == _lib.RK_EINVAL  # cache too short for prefix + tokens
    torch.cuda.synchronize()


def test_fused_rope_leaves_the_loop_output_unchanged(H):
    from rk_b200.gemma_stack import GemmaAttention, expert_scope
    from rk_b200.optimizations import quantize_linears

    expert = small_expert(H.DEVICE)
    b, t = 4, 64
    gen = torch.Generator().manual_seed(17)
    noise = torch.randn(b, 50, 32, generator=gen).to(H.DEVICE)
    pk = torch.randn(2, b, 1, t, 128, generator=gen).to(torch.bfloat16).to(H.DEVICE)
    pv = torch.randn(2, b, 1, t, 128, generator=gen).to(torch.bfloat16).to(H.DEVICE)
    with torch.no_grad():
        for grouped, views in ((False, False), (True, False), (True, True)):
            with quantize_linears(expert, "int8", scopes=("expert",), selector=expert_scope, shared_quant=True,
                                  grouped=grouped, group_views=views) as _:
                want = expert(noise, pk, pv)
                GemmaAttention.fused_rope = True
                try:
                    got = expert(noise, pk, pv)
                finally:
                    GemmaAttention.fused_rope = False
                assert torch.equal(got, want)
        bf16 = expert(noise, pk, pv)
        GemmaAttention.fused_rope = True
        try:
            assert torch.equal(expert(noise, pk, pv), bf16)
        finally:
            GemmaAttention.fused_rope = False


def test_prefix_stack_nvfp4_close_to_bf16(H):
    from rk_b200.gemma_stack import GemmaConfig, GemmaStack, prefix_scope
    from rk_b200.optimizations import quantize_linears

    cfg = GemmaConfig(width=256, mlp_dim=1024, depth=2, num_heads=2, num_kv_heads=1, head_dim=128)
    model = GemmaStack(cfg).to(torch.bfloat16).init_random(2).to(H.DEVICE).eval()
    x = H.randn_bf16((1, 816, 256), 1.0, 5).to(H.DEVICE)
    pos = torch.arange(816, device=H.DEVICE)[None]
    with torch.no_grad():
        ref, _ = model(x, pos)
        for precision, tol in (("fp4", 0.35), ("mxfp8", 0.08), ("fp8", 0.08), ("w4a16", 0.35)):
            with quantize_linears(model, precision, scopes=("text",), selector=prefix_scope) as report:
                assert len(report["modules"]) == 14
                out, kv = model(x, pos)
            rel = ((out.float() - ref.float()).norm() / ref.float().norm()).item()
            assert rel < tol, (precision, rel)
            assert kv[0][0].shape == (1, 1, 816, 128)


def test_full_width_prefix_layers_nvfp4_every_linear_matches_oracle(H):
    """Two layers of the benchmark's prefix model at its real widths (width 2048, MLP 16384, 8 heads of
    256 over one KV head; 816 tokens) with every linear in NVFP4 + the fp32 per-tensor scale on weights
    and activations: each of the 14 linears - shapes (816, 2048, 2048), (816, 256, 2048),
    (816, 16384, 2048) and (816, 2048, 16384) - is held to the oracle on the activations it saw: the
    per-tensor scale and the packed codes / scale factors bit for bit, the product within 1e-2."""
    from oracle import blockscale as OB
    from oracle import fp8 as OF
    from rk_b200.fp4_linear import Fp4CutlassLinear
    from rk_b200.gemma_stack import GemmaConfig, GemmaStack, prefix_scope
    from rk_b200.optimizations import quantize_linears

    cfg = GemmaConfig(width=2048, mlp_dim=16384, depth=2, num_heads=8, num_kv_heads=1, head_dim=256)
    model = GemmaStack(cfg).to(torch.bfloat16).init_random(4).to(H.DEVICE).eval()
    x = H.randn_bf16((1, 816, 2048), 1.0, 6).to(H.DEVICE)
    pos = torch.arange(816, device=H.DEVICE)[None]
    with torch.no_grad():
        with quantize_linears(model, "fp4", scopes=("text",), selector=prefix_scope, fp4_global_scale=True) as report:
            assert len(report["modules"]) == 14
            seen = {}
            hooks = [m.register_forward_hook(lambda mod, args, out, name=n: seen.__setitem__(name, (args[0], out)))
                     for n, m in model.named_modules() if isinstance(m, Fp4CutlassLinear)]
            # the down projections' fused GELU * up path bypasses module hooks (test_gpu_modules holds it to
            # these tensor ops bit for bit): route them through `forward` here so that they are seen too
            downs = [layer.mlp.down_proj for layer in model.layers]
            for m in downs:
                m.forward_gelu = lambda gate, up, m=m: m(torch.nn.functional.gelu(gate, approximate="tanh") * up)
            out, _ = model(x, pos)
            for hook in hooks:
                hook.remove()
            for m in downs:
                del m.forward_gelu
            torch.cuda.synchronize()
            assert torch.isfinite(out).all() and len(seen) == 14
            shapes = set()
            for name, (a, y) in seen.items():
                layer = model.get_submodule(name)
                flat = a.reshape(-1, layer.in_features)
                xs = H.to_np(flat)
                shapes.add((xs.shape[0], layer.out_features, layer.in_features))
                ga = OF.tensor_scale(xs, np.float32(6.0 * 448.0))
                pa, sa, swa = OB.pack_nvfp4(xs, ga)
                q, sf, g = layer.pack_input(flat)
                assert g.item() == ga, name
                assert np.array_equal(q.cpu().numpy(), pa) and np.array_equal(sf.cpu().numpy(), swa), name
                # the weight codes were packed by the kernel under test: unswizzle its scale factors for the oracle product
                gw = float(layer.weight_global_scale.item())
                sw = OB.unswizzle_sf(layer.weight_scale.cpu().numpy(), layer.out_features, layer.in_features // 16)
                _, want = OB.gemm_dequantized(OB.dequant_nvfp4(pa, sa, ga),
                                              OB.dequant_nvfp4(layer.packed_weight.cpu().numpy(), sw, gw))
                got = H.to_np(y.reshape(-1, layer.out_features))
                assert H.rel_frobenius(got, want) < 1e-2, name
            assert shapes == {(816, 2048, 2048), (816, 256, 2048), (816, 16384, 2048), (816, 2048, 16384)}


def test_shared_float_packs_leave_the_prefix_output_unchanged(H):
    """q/k/v and gate/up sharing one packed activation (fp8, mxfp8, fp4 with and without the per-tensor
    scale) give exactly the output of the unshared modules: the same codes reach the same GEMMs."""
    from rk_b200.gemma_stack import GemmaConfig, GemmaStack, prefix_scope
    from rk_b200.optimizations import quantize_linears

    cfg = GemmaConfig(width=256, mlp_dim=1024, depth=2, num_heads=2, num_kv_heads=1, head_dim=128)
    model = GemmaStack(cfg).to(torch.bfloat16).init_random(3).to(H.DEVICE).eval()
    x = H.randn_bf16((1, 200, 256), 1.0, 8).to(H.DEVICE)
    pos = torch.arange(200, device=H.DEVICE)[None]
    with torch.no_grad():
        for precision, extra in (("fp8", {}), ("mxfp8", {}), ("fp4", {}), ("fp4", {"fp4_global_scale": True})):
            with quantize_linears(model, precision, scopes=("text",), selector=prefix_scope, **extra):
                plain, _ = model(x, pos)
            with quantize_linears(model, precision, scopes=("text",), selector=prefix_scope, shared_quant=True, **extra) as report:
                assert report["shared_float_packs"] == 2 * cfg.depth
                shared, _ = model(x, pos)
            assert torch.equal(plain, shared), precision
    with pytest.raises(ValueError):
        with quantize_linears(model, "fp8", scopes=("text",), selector=prefix_scope, grouped=True):
            pass


def test_prefix_pass_with_fused_norm_packers_and_cache_writes(H):
    """The prefix pass as a serving stack runs it: norms that hand NVFP4 packs to q/k/v and gate/up,
    GELU * up fused in front of the down projection's packer, rotary embedding written straight into
    preallocated caches.  GELU and rope paths are bit-exact against tensor ops; the fused norm differs
    from the tensor-op norm by the summation order of mean(x^2) only (at most one bf16 ulp in front of
    the packer), so the pass stays within 2e-2 of the unfused one and the caches hold the keys / values."""
    from rk_b200.gemma_stack import (GemmaAttention, GemmaConfig, GemmaStack, fuse_norm_pack_fp4, prefix_scope,
                                     unfuse_norm_quantize)
    from rk_b200.optimizations import quantize_linears

    cfg = GemmaConfig(width=256, mlp_dim=1024, depth=2, num_heads=2, num_kv_heads=1, head_dim=128)
    model = GemmaStack(cfg).to(torch.bfloat16).init_random(3).to(H.DEVICE).eval()
    t = 200
    x = H.randn_bf16((1, t, 256), 1.0, 8).to(H.DEVICE)
    pos = torch.arange(t, device=H.DEVICE)[None]
    with torch.no_grad():
        for extra in ({"fp4_global_scale": True}, {}):
            with quantize_linears(model, "fp4", scopes=("text",), selector=prefix_scope, shared_quant=True, **extra):
                plain, kv = model(x, pos)
                caches = [(torch.zeros(1, 1, t, 128, dtype=torch.bfloat16, device=H.DEVICE),
                           torch.zeros(1, 1, t, 128, dtype=torch.bfloat16, device=H.DEVICE), 0) for _ in range(cfg.depth)]
                GemmaAttention.fused_rope = True
                try:
                    roped, kv2 = model(x, pos, past=caches)
                    assert torch.equal(roped, plain)
                    for (k0, v0), (k1, v1) in zip(kv, kv2):
                        assert torch.equal(k0, k1) and torch.equal(v0, v1)
                    norms = fuse_norm_pack_fp4(model)
                    assert len(norms) == 2 * cfg.depth
                    assert {n.fused_fp4 for n in norms} == {"global" if extra else "block"}
                    fused, kv3 = model(x, pos, past=caches)
                    unfuse_norm_quantize(norms)
                finally:
                    GemmaAttention.fused_rope = False
                rel = ((fused.float() - plain.float()).norm() / plain.float().norm()).item()
                assert rel < 2e-2, rel
                assert kv3[0][0].data_ptr() == caches[0][0].data_ptr()
    assert all(n.fused_fp4 is None for n in norms)


def test_prefix_pass_with_one_gemm_for_gate_and_up(H):
    """Gate and up as ONE NVFP4 GEMM with GELU * up in its epilogue (`Fp4GateUpGelu`): another quantization of the
    same two weights (one per-tensor scale for both halves), so the pass stays close to the one with separate
    projections; together with the fused norms it runs from packed activations end to end."""
    from rk_b200.gemma_stack import (GemmaConfig, GemmaStack, build_fused_gate_up_fp4, disable_fused_gate_up,
                                     enable_fused_gate_up, fuse_norm_pack_fp4, prefix_scope, unfuse_norm_quantize)
    from rk_b200.optimizations import quantize_linears

    cfg = GemmaConfig(width=256, mlp_dim=1024, depth=2, num_heads=2, num_kv_heads=1, head_dim=128)
    model = GemmaStack(cfg).to(torch.bfloat16).init_random(3).to(H.DEVICE).eval()
    x = H.randn_bf16((1, 200, 256), 1.0, 8).to(H.DEVICE)
    pos = torch.arange(200, device=H.DEVICE)[None]
    with torch.no_grad():
        for gs in (True, False):
            fused_modules = build_fused_gate_up_fp4(model, global_scale=gs)
            with quantize_linears(model, "fp4", scopes=("text",), selector=prefix_scope, shared_quant=True, fp4_global_scale=gs):
                plain, _ = model(x, pos)
                enable_fused_gate_up(model, fused_modules)
                try:
                    one_gemm, _ = model(x, pos)
                    norms = fuse_norm_pack_fp4(model)
                    with_norms, _ = model(x, pos)
                    unfuse_norm_quantize(norms)
                finally:
                    disable_fused_gate_up(model)
                assert torch.equal(model(x, pos)[0], plain)
            for out in (one_gemm, with_norms):
                rel = ((out.float() - plain.float()).norm() / plain.float().norm()).item()
                assert rel < 5e-2, rel
    with pytest.raises(ValueError):
        enable_fused_gate_up(model, fused_modules)  # bf16 down projections
