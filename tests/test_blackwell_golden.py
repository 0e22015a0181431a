"""Parity against the REFERENCE's own Blackwell kernels, through fixtures they produced on a B200.

`tests/golden/blackwell_golden.npz` holds what the reference's per-tensor FP8, MXFP8 and NVFP4
quantizers / packers and CUTLASS GEMMs returned for seeded inputs (`tests/golden/make_blackwell_golden.py`,
run with the extensions built by `oracle/build_ref_kernels.py`).  Small cases are stored in full;
full-size cases as SHA-256 digests plus the (few) positions where the reference's fast-math build
differs from IEEE arithmetic, with the reference's byte there, plus a fixed sample of each GEMM output.

CPU tests hold the numpy oracle to the fixtures; GPU tests hold the CUDA kernels to them, through
the C ABI.  A digest comparison means: our array, with the listed positions overwritten by the
reference's bytes, hashes to the reference's digest - so every other position is bit-identical.
"""

import hashlib
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import blockscale as OB
from oracle import fp8 as OF

GOLDEN = Path(__file__).resolve().parent / "golden"
FIXTURE = GOLDEN / "blackwell_golden.npz"
sys.path.insert(0, str(GOLDEN))
pytestmark = pytest.mark.skipif(not FIXTURE.exists(), reason="blackwell_golden.npz has not been generated")


@pytest.fixture(scope="module")
def G():
    return np.load(FIXTURE)


@pytest.fixture(scope="module")
def maker():
    import make_blackwell_golden

    return make_blackwell_golden


def sha(array):
    return hashlib.sha256(np.ascontiguousarray(array).tobytes()).hexdigest()


def patched_sha(G, key, ours):
    """Digest of `ours` after the listed differences to the reference are applied."""
    flat = np.ascontiguousarray(ours).view(np.uint8).reshape(-1).copy()
    count = int(G[key + "_diff_count"])
    pos = G[key + "_diff_pos"]
    assert count == pos.size, f"{key}: {count} differences, only {pos.size} listed"
    flat[pos] = G[key + "_diff_val"]
    return sha(flat), count


def cases(maker, names=None):
    return [c for c in maker.CASES if names is None or c[0] in names]


def valid_sf(buf, rows, groups):
    """Scale-factor buffer with everything but the valid (row, group) bytes zeroed."""
    out = np.zeros_like(np.asarray(buf, dtype=np.uint8).reshape(-1))
    idx = OB.sf_offsets(rows, groups).reshape(-1)
    out[idx] = np.asarray(buf, dtype=np.uint8).reshape(-1)[idx]
    return out


# ------------------------------------------------------------------ CPU: the oracle against the fixtures
@pytest.mark.parametrize("name", ["small", "cfg3_gate_up", "cfg4_q"])
def test_oracle_quantizers_match_reference_kernels(G, maker, name):
    (_, m, n, k), = cases(maker, (name,))
    x, w, _ = maker.case_inputs(name, m, n, k)
    xs = x.float().numpy()
    tensors = [("a", xs)]
    if name == "small":
        tensors.append(("w", w.float().numpy()))
    differing = {}
    for tag, t in tensors:
        rows, cols = t.shape
        # per-tensor FP8: the reference divides with fast-math, its scale may sit one ulp from amax / 448
        codes, scale = OF.quantize(t)
        ref_scale = np.float32(G[f"{name}_fp8_{tag}_scale"][0])
        assert abs(float(ref_scale) - float(scale)) <= float(np.spacing(np.float32(scale)))
        digest, differing[f"fp8_{tag}"] = patched_sha(G, f"{name}_fp8_{tag}_codes", codes)
        assert digest == str(G[f"{name}_fp8_{tag}_codes_sha"])
        # MXFP8: codes and swizzled UE8M0 scale buffer
        codes, _, sf_buf = OB.pack_mxfp8(t)
        digest, differing[f"mxfp8_{tag}"] = patched_sha(G, f"{name}_mxfp8_{tag}_codes", codes)
        assert digest == str(G[f"{name}_mxfp8_{tag}_codes_sha"])
        assert patched_sha(G, f"{name}_mxfp8_{tag}_sf", sf_buf)[0] == str(G[f"{name}_mxfp8_{tag}_sf_sha"])
        # NVFP4: packed E2M1 codes and swizzled UE4M3 scale buffer
        packed, _, sf_buf = OB.pack_nvfp4(t)
        digest, differing[f"nvfp4_{tag}"] = patched_sha(G, f"{name}_nvfp4_{tag}_codes", packed)
        assert digest == str(G[f"{name}_nvfp4_{tag}_codes_sha"])
        assert patched_sha(G, f"{name}_nvfp4_{tag}_sf", sf_buf)[0] == str(G[f"{name}_nvfp4_{tag}_sf_sha"])
    # Block formats: the reference's block arithmetic is exact enough that nothing differs.  Per-tensor
    # FP8: the reference divides amax / 448 and 1 / scale with fast-math; when its scale lands one ulp
    # from the IEEE quotient, values that sit on a rounding boundary of x / scale (under 1 %) flip.
    for key, count in differing.items():
        assert count <= (len(xs.reshape(-1)) // 100 if key.startswith("fp8") else 0), (key, count)


def test_small_case_arrays_are_stored_in_full(G):
    for key in ("small_fp8_a_codes", "small_mxfp8_a_sf", "small_nvfp4_w_codes", "small_fp8_out_t1", "small_nvfp4_out_t0"):
        assert key in G.files
        if not key.endswith(("_t1", "_t0")):
            assert sha(G[key]) == str(G[key + "_sha"])


def test_oracle_gemms_match_reference_outputs_small(G, maker):
    """The reference GEMM outputs of the small case against dequantize -> float64 matmul of the oracle,
    on the reference's own codes: equal up to the last bf16 digit (tolerance: relative Frobenius 2e-3)."""
    (_, m, n, k), = cases(maker, ("small",))
    _, _, bias = maker.case_inputs("small", m, n, k)
    b = bias.float().numpy()
    bits = lambda key: (G[key].astype(np.uint32) << 16).view(np.float32)
    want, _ = OF.gemm(G["small_fp8_a_codes"].reshape(m, k), G["small_fp8_a_scale"][0], G["small_fp8_w_codes"].reshape(n, k),
                      G["small_fp8_w_scale"][0], b)
    assert OB.rel_frobenius(bits("small_fp8_out_t1"), want) < 2e-3
    sa = OB.unswizzle_sf(G["small_mxfp8_a_sf"], m, k // 32)
    sb = OB.unswizzle_sf(G["small_mxfp8_w_sf"], n, k // 32)
    want, _ = OB.gemm_dequantized(OB.dequant_mxfp8(G["small_mxfp8_a_codes"].reshape(m, k), sa),
                                  OB.dequant_mxfp8(G["small_mxfp8_w_codes"].reshape(n, k), sb), b)
    assert OB.rel_frobenius(bits("small_mxfp8_out_t1"), want) < 2e-3
    sa = OB.unswizzle_sf(G["small_nvfp4_a_sf"], m, k // 16)
    sb = OB.unswizzle_sf(G["small_nvfp4_w_sf"], n, k // 16)
    want, _ = OB.gemm_dequantized(OB.dequant_nvfp4(G["small_nvfp4_a_codes"].reshape(m, k // 2), sa),
                                  OB.dequant_nvfp4(G["small_nvfp4_w_codes"].reshape(n, k // 2), sb), b)
    assert OB.rel_frobenius(bits("small_nvfp4_out_t0"), want) < 2e-3


# ------------------------------------------------------------------ GPU: the CUDA kernels against the fixtures
def _dev(t):
    return t.to(torch.device("cuda:0"))


def _apply(G, key, tensor):
    """Our device array with the reference's differing bytes written in: the reference's array."""
    flat = tensor.contiguous().view(torch.uint8).reshape(-1).clone()
    pos = torch.from_numpy(G[key + "_diff_pos"]).to(flat.device)
    if pos.numel():
        flat[pos] = torch.from_numpy(G[key + "_diff_val"]).to(flat.device)
    return flat.view(tensor.dtype).reshape(tensor.shape)


def _sample(maker, out):
    rows = torch.from_numpy(maker.sample_rows(out.shape[0])).to(out.device)
    return out[rows][:, ::maker.SAMPLE_COL_STEP].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def _close_to_reference(got_bits, ref_bits):
    """bf16 samples: at most one step apart, and not often (both kernels accumulate in fp32, in different orders)."""
    got = (got_bits.astype(np.uint32) << 16).view(np.float32)
    ref = (ref_bits.astype(np.uint32) << 16).view(np.float32)
    assert OB.rel_frobenius(got, ref) < 1e-3
    assert (got_bits != ref_bits).mean() < 0.02


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["small", "cfg3_gate_up", "cfg4_down", "cfg4_q", "cfg4_kv"])
def test_cuda_quantizers_and_gemms_match_reference_kernels(G, maker, name):
    from rk_b200 import fp4_linear as P4
    from rk_b200 import fp8_linear as P8

    (_, m, n, k), = cases(maker, (name,))
    x, w, bias = (_dev(t) for t in maker.case_inputs(name, m, n, k))
    report = {}
    # ---- per-tensor FP8
    qa, sa = P8.quantize_bf16(x)
    qb, sb = P8.quantize_bf16(w)
    for tag, q in (("a", qa), ("w", qb)):
        digest, report[f"fp8_{tag}"] = patched_sha(G, f"{name}_fp8_{tag}_codes", q.view(torch.uint8).cpu().numpy())
        assert digest == str(G[f"{name}_fp8_{tag}_codes_sha"])
    ra, rb = _apply(G, f"{name}_fp8_a_codes", qa), _apply(G, f"{name}_fp8_w_codes", qb)
    rsa = torch.from_numpy(G[f"{name}_fp8_a_scale"]).to(x.device)
    rsb = torch.from_numpy(G[f"{name}_fp8_w_scale"]).to(x.device)
    out = P8.linear_forward_packed(ra, rsa, rb, rsb, bias)
    assert np.array_equal(_sample(maker, out), G[f"{name}_fp8_out_ours_sample"])
    for tactic in (1, 6, 2):
        if f"{name}_fp8_out_t{tactic}_sample" in G.files:
            _close_to_reference(_sample(maker, out), G[f"{name}_fp8_out_t{tactic}_sample"])
    # ---- MXFP8
    qa, fa = P8.mxfp8_pack(x)
    qb, fb = P8.mxfp8_pack(w)
    for tag, q, f in (("a", qa, fa), ("w", qb, fb)):
        digest, report[f"mxfp8_{tag}"] = patched_sha(G, f"{name}_mxfp8_{tag}_codes", q.view(torch.uint8).cpu().numpy())
        assert digest == str(G[f"{name}_mxfp8_{tag}_codes_sha"])
        assert patched_sha(G, f"{name}_mxfp8_{tag}_sf", f.cpu().numpy())[0] == str(G[f"{name}_mxfp8_{tag}_sf_sha"])
    out = P8.mxfp8_linear(_apply(G, f"{name}_mxfp8_a_codes", qa), _apply(G, f"{name}_mxfp8_a_sf", fa),
                          _apply(G, f"{name}_mxfp8_w_codes", qb), _apply(G, f"{name}_mxfp8_w_sf", fb), bias)
    assert np.array_equal(_sample(maker, out), G[f"{name}_mxfp8_out_ours_sample"])
    for tactic in (1, 6, 102, 2, 4):
        if f"{name}_mxfp8_out_t{tactic}_sample" in G.files:
            _close_to_reference(_sample(maker, out), G[f"{name}_mxfp8_out_t{tactic}_sample"])
    # ---- NVFP4 (the reference's format: no per-tensor scale)
    qa, fa = P4.pack_nvfp4(x)
    qb, fb = P4.pack_nvfp4(w)
    for tag, q, f in (("a", qa, fa), ("w", qb, fb)):
        digest, report[f"nvfp4_{tag}"] = patched_sha(G, f"{name}_nvfp4_{tag}_codes", q.cpu().numpy())
        assert digest == str(G[f"{name}_nvfp4_{tag}_codes_sha"])
        assert patched_sha(G, f"{name}_nvfp4_{tag}_sf", f.cpu().numpy())[0] == str(G[f"{name}_nvfp4_{tag}_sf_sha"])
    out = P4.linear_forward_packed_gemm_bf16(_apply(G, f"{name}_nvfp4_a_codes", qa), _apply(G, f"{name}_nvfp4_a_sf", fa), None,
                                             _apply(G, f"{name}_nvfp4_w_codes", qb), _apply(G, f"{name}_nvfp4_w_sf", fb), None,
                                             bias, k)
    assert np.array_equal(_sample(maker, out), G[f"{name}_nvfp4_out_ours_sample"])
    if f"{name}_nvfp4_out_t0_sample" in G.files:
        _close_to_reference(_sample(maker, out), G[f"{name}_nvfp4_out_t0_sample"])
    # block formats are bit-identical; per-tensor FP8 may flip under 1 % of the codes when the
    # reference's fast-math scale sits one ulp from the IEEE quotient
    for key, count in report.items():
        assert count <= ((m if key.endswith("_a") else n) * k // 100 if key.startswith("fp8") else 0), (key, count)


@pytest.mark.gpu
def test_cuda_fused_producers_match_reference_kernels(G, maker):
    """RMSNorm(+residual) and SwiGLU producers in front of the FP8 / NVFP4 quantizers, small case in full."""
    from rk_b200 import fp4_linear as P4
    from rk_b200 import fp8_linear as P8

    if "prod_fp8_rms_codes" not in G.files:
        pytest.skip("the fixture holds no producer outputs")
    x, res, weight, gate_up, inter = (_dev(t) if torch.is_tensor(t) else t for t in maker.producer_inputs())
    s, nrm, q, scale = P8.add_rms_norm_quantize_bf16(x, res, weight, 1e-6)
    assert np.array_equal(s.view(torch.uint8).cpu().numpy().reshape(-1), G["prod_fp8_rms_sum"].reshape(-1))
    # the reference's rsqrt is the fast-math approximation: normalised values may differ in the last bf16 digit
    for key, ours in (("prod_fp8_rms_norm", nrm), ("prod_fp8_rms_codes", q)):
        count = int(G[key + "_diff_count"])
        assert patched_sha(G, key, ours.view(torch.uint8).cpu().numpy())[0] == str(G[key + "_sha"])
        assert count <= ours.numel() // 50, (key, count)
    q, scale = P8.quantize_swiglu_bf16(gate_up, inter)
    assert patched_sha(G, "prod_fp8_swiglu_codes", q.view(torch.uint8).cpu().numpy())[0] == str(G["prod_fp8_swiglu_codes_sha"])
    assert int(G["prod_fp8_swiglu_codes_diff_count"]) <= q.numel() // 50
    if "prod_nvfp4_rms_codes" in G.files:
        s, nrm, q, sf = P4.add_rms_norm_fp4_quant_bf16(x, res, weight, 1e-6, True)
        assert patched_sha(G, "prod_nvfp4_rms_codes", q.cpu().numpy())[0] == str(G["prod_nvfp4_rms_codes_sha"])
        assert int(G["prod_nvfp4_rms_codes_diff_count"]) <= q.numel() // 50


# ------------------------------------------------------------------ second fixture file: W4A8 MX, FP8 producer, SwiGLU chains
EXT = GOLDEN / "blackwell_golden_ext.npz"
needs_ext = pytest.mark.skipif(not EXT.exists(), reason="blackwell_golden_ext.npz has not been generated")


@pytest.fixture(scope="module")
def GX():
    return np.load(EXT)


@needs_ext
def test_oracle_w4a8_mx_packers_match_reference_kernels(GX, maker):
    """`pack_mxfp8_activation` / `pack_mxfp4_weight` of the reference (blackwell/csrc/fp4_mx_cutlass_linear.cu)
    against the oracle: small case in full, the 816 x 2048 activation of the full-size case by digest."""
    _, m, n, k = maker.EXT_CASES[0]
    x, w, bias = maker.case_inputs("small", m, n, k)
    ca, sa, swa = OB.pack_mxfp8_ceil(x.float().numpy())
    pb, sb, swb = OB.pack_mxfp4_ceil(w.float().numpy())
    assert np.array_equal(GX["small_w4a8_a_codes"].reshape(m, k), ca) and np.array_equal(GX["small_w4a8_a_sf"], swa)
    assert np.array_equal(GX["small_w4a8_w_codes"].reshape(n, k // 2), pb) and np.array_equal(GX["small_w4a8_w_sf"], swb)
    # the reference's GEMM output on those operands against dequantize -> float64 matmul
    want, _ = OB.gemm_dequantized(OB.dequant_mxfp8(ca, sa), OB.dequant_mxfp4(pb, sb), bias.float().numpy())
    got = (GX["small_w4a8_out"].astype(np.uint32) << 16).view(np.float32)
    assert OB.rel_frobenius(got, want) < 2e-3
    _, m, n, k = maker.EXT_CASES[1]
    x, _, _ = maker.case_inputs("w4a8_gate_up", m, n, k)
    ca, _, swa = OB.pack_mxfp8_ceil(x.float().numpy())
    assert patched_sha(GX, "w4a8_gate_up_w4a8_a_codes", ca) == (str(GX["w4a8_gate_up_w4a8_a_codes_sha"]), 0)
    assert patched_sha(GX, "w4a8_gate_up_w4a8_a_sf", swa) == (str(GX["w4a8_gate_up_w4a8_a_sf_sha"]), 0)


@needs_ext
def test_oracle_fp8_producer_matches_reference_output_small(GX, maker):
    """The reference's producer GEMM (bf16 activations converted in its main loop, unit scale) against
    the oracle: e4m3 of the clamped activations, reference weight codes and scale."""
    _, m, n, k = maker.EXT_CASES[0]
    x, _, bias = maker.case_inputs("small", m, n, k)
    codes = OF.quantize_with_scale(x.float().numpy(), np.float32(1.0))
    want, _ = OF.gemm(codes, np.float32(1.0), GX["small_fp8prod_w_codes"].reshape(n, k), GX["small_fp8prod_w_scale"][0],
                      bias.float().numpy())
    got = (GX["small_fp8prod_out"].astype(np.uint32) << 16).view(np.float32)
    assert OB.rel_frobenius(got, want) < 2e-3


@needs_ext
@pytest.mark.gpu
def test_cuda_w4a8_mx_and_producer_match_reference_kernels(GX, maker):
    from rk_b200 import fp4_mx_linear as PM
    from rk_b200 import fp8_linear as P8

    for name, m, n, k in maker.EXT_CASES:
        x, w, bias = (_dev(t) for t in maker.case_inputs(name, m, n, k))
        if name != "producer_kv":
            qa, fa = PM.pack_mxfp8_activation(x)
            qb, fb = PM.pack_mxfp4_weight(w)
            for tag, ours in (("a_codes", qa.view(torch.uint8)), ("a_sf", fa), ("w_codes", qb), ("w_sf", fb)):
                key = f"{name}_w4a8_{tag}"
                assert patched_sha(GX, key, ours.cpu().numpy()) == (str(GX[key + "_sha"]), 0), key  # bit-identical
            out = PM.linear_w4a8_packed(qa, fa, qb, fb, bias)
            assert np.array_equal(_sample(maker, out), GX[f"{name}_w4a8_out_ours_sample"])
            _close_to_reference(_sample(maker, out), GX[f"{name}_w4a8_out_sample"])
        if name != "w4a8_gate_up":
            wq, wscale = P8.quantize_bf16(w)
            if sha(wq.view(torch.uint8).cpu().numpy()) == str(GX[f"{name}_fp8prod_w_codes_sha"]):
                # same weight codes as the reference's quantizer produced: outputs are comparable directly
                ref_scale = torch.from_numpy(GX[f"{name}_fp8prod_w_scale"]).to(x.device)
                out = P8.linear_forward_producer(x, wq, ref_scale, bias)
                assert np.array_equal(_sample(maker, out), GX[f"{name}_fp8prod_out_ours_sample"])
                _close_to_reference(_sample(maker, out), GX[f"{name}_fp8prod_out_sample"])


@needs_ext
@pytest.mark.gpu
def test_cuda_swiglu_chains_match_reference_kernels(GX, maker):
    """SwiGLU -> pack -> down projection, both gate/up layouts, NVFP4 and W4A8-MX: the reference's final
    outputs (`linear_forward_swiglu_gemm_bf16`, `pack_swiglu_mxfp8` + `linear_w4a8_packed`)."""
    from rk_b200 import fp4_linear as P4
    from rk_b200 import fp4_mx_linear as PM

    x, res, weight, gate_up, inter = (_dev(t) if torch.is_tensor(t) else t for t in maker.producer_inputs())
    gen = torch.Generator().manual_seed(78)
    wd = (torch.randn(256, inter, generator=gen) * 0.02).to(torch.bfloat16)
    lin = torch.nn.Linear(inter, 256, bias=False, dtype=torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_(wd)
    lin = lin.to(gate_up.device).requires_grad_(False)
    bits = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)
    for interleaved in (False, True):
        # the fixtures' gate_up is read in the requested layout as it stands (same bytes, other meaning)
        if f"swiglu_nvfp4_out_{int(interleaved)}" in GX.files:
            out = P4.Fp4CutlassLinear.from_linear(lin, "linear", "down").forward_swiglu(gate_up, inter, interleaved)
            ref = GX[f"swiglu_nvfp4_out_{int(interleaved)}"]
            assert (bits(out) != ref).mean() < 0.02
        tag = f"swiglu_mxfp8_{int(interleaved)}"
        if tag + "_out" in GX.files:
            q, sf = PM.pack_swiglu_mxfp8(gate_up, inter, interleaved)
            assert patched_sha(GX, tag + "_codes", q.view(torch.uint8).cpu().numpy())[0] == str(GX[tag + "_codes_sha"])
            assert patched_sha(GX, tag + "_sf", sf.cpu().numpy())[0] == str(GX[tag + "_sf_sha"])
            out = PM.Fp4MxLinear.from_linear(lin, "linear", "down").forward_swiglu(gate_up, inter, interleaved)
            assert (bits(out) != GX[tag + "_out"]).mean() < 0.02


# ------------------------------------------------------------------ third fixture file: the table-SiLU SwiGLU producer for MXFP8
SILU = GOLDEN / "blackwell_golden_silu.npz"
needs_silu = pytest.mark.skipif(not SILU.exists(), reason="blackwell_golden_silu.npz has not been generated")


@pytest.fixture(scope="module")
def GS():
    return np.load(SILU)


@needs_silu
def test_oracle_silu_mul_pack_matches_reference_kernel(GS, maker):
    """`robotics_mxfp8_swiglu::silu_mul_pack` (blackwell/csrc/mxfp8_swiglu.cu) on a B200 against the numpy
    restatement, with the SiLU table the reference was given: codes and scale bytes, bit for bit."""
    from oracle.formats import bf16_from_bits

    table = bf16_from_bits(GS["silu_table_bits"])
    for name, rows, inter in maker.SILU_CASES:
        gate_up = maker.silu_inputs(name, rows, inter).float().numpy()
        codes, _, swizzled = OB.silu_mul_pack_mxfp8(gate_up, inter, table)
        tag = "silu_" + name
        assert int(GS[tag + "_codes_diff_count"]) == 0 and int(GS[tag + "_sf_diff_count"]) == 0
        assert sha(codes) == str(GS[tag + "_codes_sha"]), name
        assert sha(swizzled) == str(GS[tag + "_sf_sha"]), name
        if name == "small":
            assert np.array_equal(codes.reshape(-1), GS[tag + "_codes"].reshape(-1)) and np.array_equal(swizzled, GS[tag + "_sf"].reshape(-1))
            assert OB.unswizzle_sf(swizzled, rows, inter // 32)[3, 0] == 255  # the block with the infinity


@needs_silu
@pytest.mark.gpu
def test_cuda_silu_mul_pack_matches_reference_kernel(GS, maker):
    from rk_b200 import mxfp8_swiglu as MS

    table = MS.make_bf16_silu_table(torch.device("cuda:0"))
    assert np.array_equal(table.view(torch.int16).cpu().numpy().view(np.uint16), GS["silu_table_bits"])
    for name, rows, inter in maker.SILU_CASES:
        gate_up = _dev(maker.silu_inputs(name, rows, inter))
        q, sf = MS.silu_mul_pack_mxfp8(gate_up.reshape(1, rows, 2 * inter), inter, table)
        assert q.shape == (1, rows, inter) and q.dtype == torch.float8_e4m3fn
        tag = "silu_" + name
        assert sha(q.view(torch.uint8).cpu().numpy()) == str(GS[tag + "_codes_sha"]), name
        assert sha(sf.cpu().numpy()) == str(GS[tag + "_sf_sha"]), name
    with pytest.raises(ValueError):
        MS.silu_mul_pack_mxfp8(gate_up[:, :100], 50, table)
    with pytest.raises(ValueError):
        MS.silu_mul_pack_mxfp8(gate_up, inter, table[:100])
