"""The C-ABI library loads and exports every symbol ``include/ossm_b200.h``
declares, and the ctypes table binds exactly that set (no compute calls)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "ossm_b200.h")


def _declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ossm_b200_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from ossm_b200 import build as _build
    from ossm_b200 import _lib

    _build.build()
    return _lib.load()


def test_header_declares_something():
    syms = _declared_symbols()
    assert "ossm_b200_lti_scan_forward" in syms and len(syms) >= 10


def test_every_declared_symbol_is_exported(lib):
    for name in _declared_symbols():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_ctypes_table_matches_header(lib):
    from ossm_b200 import _lib

    assert sorted(_lib.SIGNATURES) == _declared_symbols()


def test_pure_host_entry_points(lib):
    assert lib.ossm_b200_version() >= 1
    chunk = lib.ossm_b200_lti_chunk()
    assert chunk == 32
    assert lib.ossm_b200_lti_carry_bytes(4096, 64, 256) == (4096 // chunk - 1) * 64 * 256 * 16
    assert lib.ossm_b200_lti_carry_bytes(chunk, 2, 3) == 0
    assert lib.ossm_b200_lti_carry_bytes(chunk + 1, 2, 3) == 2 * 3 * 16
    assert lib.ossm_b200_lti_backward_workspace_bytes(10, 2, 3) == 6 * 2 * 3 * 4
    assert lib.ossm_b200_lti_backward_workspace_bytes(0, 2, 3) == 0


def test_invalid_arguments_are_rejected_without_a_gpu(lib):
    # argument validation happens before any CUDA call
    rc = lib.ossm_b200_lti_scan_forward(99, None, None, None, None, None, None, None, 4, 1, 1, None)
    assert rc == -1 and b"variant" in lib.ossm_b200_last_error()
    rc = lib.ossm_b200_lti_scan_forward(0, None, None, None, None, None, None, None, 4, 1, 1, None)
    assert rc == -1 and b"null" in lib.ossm_b200_last_error()
    dummy = ctypes.c_void_p(256)
    rc = lib.ossm_b200_lti_scan_forward(0, dummy, dummy, dummy, dummy, None, None, None, 4, 1, 1, None)
    assert rc == -1
    rc = lib.ossm_b200_lti_scan_forward(0, dummy, dummy, dummy, dummy, dummy, None, None, -1, 1, 1, None)
    assert rc == -1
    # empty problems are a successful no-op
    assert lib.ossm_b200_lti_scan_forward(0, dummy, dummy, dummy, None, None, None, None, 0, 4, 4, None) == 0
    rc = lib.ossm_b200_lti_set_tuning(b"no_such_key", 1)
    assert rc == -1
