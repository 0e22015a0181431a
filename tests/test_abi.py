"""The C-ABI library loads and exports every symbol that include/rk_b200.h declares (no compute)."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "rk_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(rk_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def built_library():
    import __graft_entry__ as entry

    return ctypes.CDLL(str(entry.build()))


def test_header_declares_the_expected_families():
    names = declared_symbols()
    for required in ("rk_quant_rows", "rk_gemm_int", "rk_gemm_w4a16_g128", "rk_gemm_fp8", "rk_gemm_mxfp8",
                     "rk_gemm_nvfp4", "rk_pack_mxfp8", "rk_pack_nvfp4", "rk_workspace_bytes"):
        assert required in names


def test_library_exports_every_declared_symbol(built_library):
    missing = [name for name in declared_symbols() if not hasattr(built_library, name)]
    assert not missing, f"declared but not exported: {missing}"


def test_python_binding_covers_every_declared_symbol():
    from rk_b200 import _lib

    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_host_only_entry_points(built_library):
    from rk_b200 import _lib

    lib = _lib.load()
    assert lib.rk_version() >= 1000
    assert lib.rk_supports_device(10, 0) == 1
    assert lib.rk_supports_device(9, 0) == 0 and lib.rk_supports_device(8, 9) == 0
    # scale-factor buffer of the MXFP8 activations / weights of the 816 x 16384 x 2048 GEMM
    assert lib.rk_sf_bytes(816, 2048 // 32) == 7 * 16 * 512
    assert lib.rk_sf_bytes(16384, 2048 // 32) == 1 << 20
    assert lib.rk_workspace_bytes(_lib.OP_W8A8, 64, 2048, 2048) >= _lib.WORKSPACE_HEADER
    # W4A4 widens both operands to int8 in the scratch buffer
    assert lib.rk_workspace_bytes(_lib.OP_W4A4, 64, 2048, 2048) >= (64 + 2048) * 2048


def test_argument_errors_are_reported_without_a_gpu(built_library):
    from rk_b200 import _lib

    lib = _lib.load()
    assert lib.rk_quant_rows(None, 1, 128, 128, None, 0, None, 0, 8, None, None, None) == _lib.RK_EINVAL
    assert b"null" in lib.rk_last_error_string()
    with pytest.raises(ValueError):
        _lib.check(_lib.RK_EINVAL, "probe")
    with pytest.raises(RuntimeError):
        _lib.check(_lib.RK_EUNSUPPORTED, "probe")


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from rk_b200 import _lib

    monkeypatch.setenv("RK_B200_SO", str(tmp_path / "absent.so"))
    monkeypatch.setattr(_lib, "_lib", None)
    ok, error = _lib.backend_status()
    assert not ok and "does not exist" in error
    with pytest.raises(RuntimeError):
        _lib.load()
