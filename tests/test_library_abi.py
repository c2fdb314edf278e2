"""The C-ABI library loads and exports exactly what include/slinoss_b200.h
declares.  No kernel is launched (CPU only)."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "slinoss_b200.h"
SELFTEST_HEADER = ROOT / "include" / "slinoss_b200_selftest.h"


def _declared(header=HEADER):
    text = header.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(slx_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from slinoss_b200 import _lib, build

    build.build()
    return _lib.lib()


def test_every_declared_symbol_is_exported_and_bound(lib):
    from slinoss_b200 import _lib

    names = _declared()
    assert len(names) >= 16
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes table and header disagree"


def test_selftest_library_exports_its_header():
    from slinoss_b200 import _lib, build

    build.build_selftest()
    names = _declared(SELFTEST_HEADER)
    handle = _lib.selftest_lib()
    for n in names:
        assert hasattr(handle, n), f"{n} declared in the self-test header but not exported"
    assert sorted(_lib.SELFTEST_SIGNATURES) == names
    # the product library carries no diagnostics
    assert not hasattr(_lib.lib(), "slx_umma_selftest")
    assert not hasattr(_lib.lib(), "slx_read_phase_clock")


def test_abi_version(lib):
    assert lib.slx_abi_version() == 5


def test_argument_errors_are_reported_without_touching_the_gpu(lib):
    from slinoss_b200 import _lib

    # NULL shape -> SLX_E_NULL before any CUDA call
    assert lib.slx_chunk_increment_fwd(None, *([None] * 7), 0, None, None) == -1
    assert b"NULL" in lib.slx_last_error_string()
    s = _lib.ScanShape(4, 64, 32, 16, 48, 0)  # chunk 48 is not a kernel size
    assert lib.slx_chunk_scan_fwd(ctypes.byref(s), *([None] * 10)) == -3
    assert b"chunk" in lib.slx_last_error_string()
    s = _lib.ScanShape(4, 64, 128, 16, 64, 0)  # P too large
    assert lib.slx_chunk_scan_fwd(ctypes.byref(s), *([None] * 10)) == -3
    s = _lib.ScanShape(4, 64, 32, 16, 64, 0)
    assert lib.slx_chunk_scan_fwd(ctypes.byref(s), *([None] * 10)) == -1
    assert lib.slx_v2x2ssd_bwd_workspace_bytes(ctypes.byref(s)) > 0
    with pytest.raises(ValueError):
        _lib.check(-2, "probe")
    with pytest.raises(TypeError):
        _lib.check(-5, "probe")
    with pytest.raises(RuntimeError):
        _lib.check(700, "probe")


def test_missing_library_is_a_loud_error(monkeypatch, tmp_path):
    from slinoss_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.lib()
