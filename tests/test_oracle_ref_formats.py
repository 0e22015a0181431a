"""Pins the oracle's number formats and scale-factor layout on the reference's own conversion code.

`oracle/_ref/libref_formats.so` is compiled (by `oracle/build_ref.py`) from the headers of a
checkout of the reference: its vendored CUTLASS conversions, the toolkit's FP8 conversion it calls,
and its `scale_offset`.  The numpy restatement must agree with it bit for bit over exhaustive or
dense input sweeps.  Skipped when the helper has not been built (no reference checkout)."""

import ctypes
from pathlib import Path

import numpy as np
import pytest

from oracle import blockscale as OB
from oracle import formats as F

LIB = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "libref_formats.so"


@pytest.fixture(scope="module")
def ref():
    if not LIB.exists():
        pytest.skip("oracle/_ref/libref_formats.so not built (needs a checkout of the reference)")
    lib = ctypes.CDLL(str(LIB))
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    for name in ("ref_nv_e4m3", "ref_cutlass_e4m3", "ref_cutlass_ue8m0", "ref_cutlass_ue8m0_inverse",
                 "ref_cutlass_ue8m0_value", "ref_cutlass_e2m1", "ref_cutlass_e2m1_value", "ref_cutlass_ue4m3",
                 "ref_cutlass_ue4m3_value", "ref_cutlass_e4m3_value"):
        fn = getattr(lib, name)
        fn.argtypes = [vp, i64, vp]
        fn.restype = None
    lib.ref_scale_offset.argtypes = [i64, i64, i64]
    lib.ref_scale_offset.restype = i64
    lib.ref_scale_storage_size.argtypes = [i64, i64]
    lib.ref_scale_storage_size.restype = i64
    return lib


def _call(fn, src, out_dtype, count=None):
    src = np.ascontiguousarray(src)
    out = np.empty(src.size, dtype=out_dtype)
    fn(src.ctypes.data, src.size if count is None else count, out.ctypes.data)
    return out


def _sweep_f32(seed=0):
    """Every bf16 bit pattern widened to fp32 (all exponents, NaN/inf included) plus random fp32 in the
    ranges the packers produce, plus exact rounding ties of the small formats."""
    bf = (np.arange(1 << 16, dtype=np.uint32) << 16).view(np.float32)
    rng = np.random.default_rng(seed)
    rnd = np.concatenate([
        rng.standard_normal(200000).astype(np.float32) * s for s in (1e-3, 0.3, 4.0, 100.0, 600.0)
    ])
    ties = np.concatenate([np.arange(0, 1024, dtype=np.float32) / 64.0, np.arange(0, 1024, dtype=np.float32) / 2.0,
                           np.arange(0, 4096, dtype=np.float32) * np.float32(2.0 ** -13)])
    return np.concatenate([bf, rnd, ties, -ties]).astype(np.float32)


def _same_codes(got, want, nan_mask, nan_pred):
    """Codes must agree exactly where the input is a number; for NaN inputs both must be a NaN code."""
    assert np.array_equal(got[~nan_mask], want[~nan_mask])
    assert nan_pred(got[nan_mask]).all() and nan_pred(want[nan_mask]).all()


def test_e4m3_encode_matches_toolkit_and_cutlass_conversions(ref):
    x = _sweep_f32()
    ours = F.e4m3_encode(x)
    nan = np.isnan(x)
    is_nan_code = lambda c: (c & 0x7F) == 0x7F
    _same_codes(ours, _call(ref.ref_nv_e4m3, x, np.uint8), nan, is_nan_code)
    _same_codes(ours, _call(ref.ref_cutlass_e4m3, x, np.uint8), nan, is_nan_code)


def test_e4m3_ue4m3_e2m1_decode_match_cutlass(ref):
    codes = np.arange(256, dtype=np.uint8)
    want = _call(ref.ref_cutlass_e4m3_value, codes, np.float32)
    got = F.e4m3_decode(codes)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(got[~np.isnan(got)], want[~np.isnan(want)])
    want = _call(ref.ref_cutlass_ue4m3_value, codes[:127], np.float32)
    assert np.array_equal(F.ue4m3_decode(codes[:127]), want)
    nib = np.arange(16, dtype=np.uint8)
    assert np.array_equal(F.e2m1_decode(nib), _call(ref.ref_cutlass_e2m1_value, nib, np.float32))


def test_e2m1_encode_matches_cutlass_constructor(ref):
    x = _sweep_f32(1)
    x = x[~np.isnan(x)]
    assert np.array_equal(F.e2m1_encode(x), _call(ref.ref_cutlass_e2m1, x, np.uint8))


def test_ue4m3_encode_matches_cutlass_constructor(ref):
    x = np.abs(_sweep_f32(2))
    x = x[~np.isnan(x)]
    assert np.array_equal(F.ue4m3_encode(x), _call(ref.ref_cutlass_ue4m3, x, np.uint8))


def test_ue8m0_roundup_and_inverse_match_cutlass(ref):
    # every non-negative finite bf16 value, and fp32 values one ulp either side of each power of two
    bf = (np.arange(0, 0x7F80, dtype=np.uint32) << 16).view(np.float32)
    p2 = (np.arange(1, 255, dtype=np.uint32) << 23)
    near = np.concatenate([p2 - 1, p2, p2 + 1]).astype(np.uint32).view(np.float32)
    rng = np.random.default_rng(3)
    x = np.concatenate([bf, near, np.abs(rng.standard_normal(100000)).astype(np.float32) * np.float32(0.01)])
    got = F.ue8m0_encode_roundup(x)
    want = _call(ref.ref_cutlass_ue8m0, x, np.uint8)
    assert np.array_equal(got, want)
    codes = np.arange(0, 255, dtype=np.uint8)
    assert np.array_equal(F.ue8m0_decode(codes), _call(ref.ref_cutlass_ue8m0_value, codes, np.float32))
    inv = F.ue8m0_decode((254 - codes.astype(np.int64)) & 255)
    assert np.array_equal(inv, _call(ref.ref_cutlass_ue8m0_inverse, codes, np.float32))


def test_scale_factor_layout_matches_reference_offsets(ref):
    for rows, groups in ((1, 1), (50, 64), (129, 5), (400, 32), (816, 128)):
        offs = OB.sf_offsets(rows, groups)
        kt = (groups + 3) // 4
        for r in sorted({0, 1, 31, 32, 127, rows - 1} & set(range(rows))):
            for g in range(groups):
                assert offs[r, g] == ref.ref_scale_offset(r, g, kt)
        # the reference sizes the buffer from (rows, columns) with 32 columns per factor
        assert OB.sf_bytes(rows, groups) == ref.ref_scale_storage_size(rows, groups * 32)
