"""The C-ABI library loads and exports every symbol include/q4b200.h declares (no compute calls)."""
import ctypes
import os
import re

from conftest import ROOT
from llama_cu_awq_b200 import _lib


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "q4b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(q4_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported():
    L = ctypes.CDLL(_lib.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 35
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_binding_covers_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_status_strings_and_arch():
    L = _lib.lib()
    assert L.q4_abi_version() == 1
    assert L.q4_build_arch() == b"sm_100a"
    assert _lib.status_string(_lib.Q4_ERR_UNSUPPORTED_SIZE) == "Unsupported matmul size"
    assert _lib.status_string(0) == "ok"


def test_struct_layouts():
    assert ctypes.sizeof(_lib.q4_config) == 32          # the 32-byte file header
    assert ctypes.sizeof(_lib.q4_qweight) == 24
    assert ctypes.sizeof(_lib.q4_shared_data) == 4 + 4 * 128 * 1024


def test_missing_library_fails_loudly(monkeypatch):
    import pytest
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libq4b200.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.lib()


def test_measurement_switches_live_in_the_test_build_only():
    """The product library exports no q4_test_* symbol and reads no environment variable on the decode path; the test
    build (same sources, -DQ4_TEST_BUILD) exports every switch the tests use."""
    prod = ctypes.CDLL(_lib.LIB_PATH)
    test = ctypes.CDLL(_lib.TEST_LIB_PATH)
    for name in _lib.TEST_SIGNATURES:
        assert hasattr(test, name), name
        assert not hasattr(prod, name), name
    csrc = os.path.join(ROOT, "llama_cu_awq_b200", "csrc")
    for f in os.listdir(csrc):
        if f.endswith((".cu", ".cuh", ".h")):
            assert "getenv" not in open(os.path.join(csrc, f)).read(), f
