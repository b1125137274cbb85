"""The C-ABI library loads without a GPU and exports every symbol the header declares."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "tritonkv_b200.h")


def _declared():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tkv_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_path():
    names = _declared()
    for must in ("tkv_quantize_pack", "tkv_fused_decode", "tkv_fp16_decode", "tkv_combine",
                 "tkv_pack_codes", "tkv_unpack_codes", "tkv_dequantize", "tkv_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from tritonkv_b200 import _cabi

    lib = _cabi.load()  # raises loudly if the .so is missing: there is no fallback
    for name in _declared():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in _cabi.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_cabi.SIGNATURES) == set(_declared())
    assert lib.tkv_version() >= 100


def test_argument_errors_need_no_gpu():
    """Validation failures come back as a status plus a message, before any launch."""
    from tritonkv_b200 import _cabi

    lib = _cabi.load()
    rc = lib.tkv_pack_codes(None, None, 4, 128, 3, None)
    assert rc == _cabi.TKV_ERR_INVALID
    assert "nbits must be one of (2, 4)" in _cabi.last_error()
    rc = lib.tkv_quantize_pack(None, 0, None, None, None, 4, 128, 4, 48, None)
    assert rc == _cabi.TKV_ERR_INVALID
    rc = lib.tkv_combine(None, None, None, None, None, None, 1, 1, 1, 128, None)
    assert rc == _cabi.TKV_ERR_INVALID
    with pytest.raises(ValueError):
        _cabi.check(rc)
