"""CPU: the C-ABI library loads and exports exactly what include/newt_b200.h declares."""

import ctypes
import os
import re

from newt_b200.runtime import abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "newt_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nb200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = _declared()
    for must in ("nb200_add_f32", "nb200_softmax_f32", "nb200_layernorm", "nb200_gemm",
                 "nb200_attention_fwd"):
        assert must in names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(abi.LIB_PATH)
    for name in _declared():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_binding_table_covers_header():
    assert sorted(abi.SIGNATURES) == _declared()


def test_abi_version_and_error_text():
    lib = abi.load()
    assert lib.nb200_abi_version() == 1
    # argument validation happens before any CUDA call, so it runs without a GPU
    rc = lib.nb200_add_f32(None, None, None, -1, None)
    assert rc == abi.E_INVALID
    assert "negative" in abi.last_error()
    rc = lib.nb200_softmax_f32(None, None, 4, 4, 4, 4, None)
    assert rc == abi.E_INVALID and "null" in abi.last_error()
    assert lib.nb200_add_f32(None, None, None, 0, None) == 0  # empty input is a no-op


def test_status_codes_become_exceptions():
    """abi.check: 0 passes, NB200_E_UNSUPPORTED has its own type, anything else (a kernel that
    gave up on a bounded wait reports NB200_E_DEVICE) is a KernelLibraryError with the code."""
    import pytest

    abi.check(abi.OK)
    with pytest.raises(abi.UnsupportedError) as e:
        abi.check(abi.E_UNSUPPORTED)
    assert e.value.code == abi.E_UNSUPPORTED
    for code in (abi.E_INVALID, abi.E_CUDA, abi.E_DEVICE):
        with pytest.raises(abi.KernelLibraryError) as e:
            abi.check(code)
        assert e.value.code == code and not isinstance(e.value, abi.UnsupportedError)
