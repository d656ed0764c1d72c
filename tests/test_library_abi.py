"""CPU checks of the C-ABI boundary: the library loads without a GPU and exports
every symbol that include/w4a4_b200.h declares; argument validation that needs
no device works."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from zip_kernel_b200 import build
    path = build.build()
    return ctypes.CDLL(path)


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "w4a4_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(w4a4_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_exported(lib):
    names = _declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/w4a4_b200.h but not exported"


def test_binding_table_matches_header():
    from zip_kernel_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared_symbols()


def test_host_only_calls(lib):
    lib.w4a4_status_string.restype = ctypes.c_char_p
    lib.w4a4_last_error.restype = ctypes.c_char_p
    lib.w4a4_workspace_bytes.restype = ctypes.c_size_t
    assert lib.w4a4_abi_version() == 1
    assert lib.w4a4_status_string(0) == b"ok"
    assert lib.w4a4_status_string(3) == b"workspace missing or too small"
    small = lib.w4a4_workspace_bytes(1, 4096, 4096, 0)
    big = lib.w4a4_workspace_bytes(8192, 4096, 4096, 0)
    assert 0 < small < big
    assert lib.w4a4_workspace_bytes(0, 4096, 4096, 0) == 0
    # argument errors are reported before any CUDA call
    rc = lib.w4a4_activation_quant(None, ctypes.c_longlong(100), None, None, None, None, 1, 100, None)
    assert rc == 1 and b"multiple of 128" in lib.w4a4_last_error()
    rc = lib.w4a4_activation_quant(None, ctypes.c_longlong(128), None, None, None, None, 1, 128, None)
    assert rc == 1 and b"NULL" in lib.w4a4_last_error()
