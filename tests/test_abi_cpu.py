"""The C-ABI library loads without a GPU and exports every symbol the header declares;
argument validation that needs no device also runs here."""
import ctypes
import os
import re

from polarengine_vllm_b200 import _native as nv

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "polar_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pe_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    lib = nv.lib()
    names = declared_symbols()
    assert "pe_gemv" in names and "pe_fwht128" in names
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/polar_b200.h but not exported"
        assert name in nv.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(nv.SIGNATURES) == names


def test_version_and_error_strings():
    lib = nv.lib()
    assert lib.pe_version() >= 100
    assert lib.pe_error_string(0) == b"ok"
    for code in range(-7, 0):
        assert lib.pe_error_string(code) not in (b"ok", b"unknown error")


def test_argument_validation_without_device():
    lib = nv.lib()
    assert lib.pe_gemv_workspace_bytes(1, 4096, 12288) > 0
    assert lib.pe_gemv_workspace_bytes(17, 4096, 4096) == 0      # batch beyond the decode kernel
    assert lib.pe_gemv_workspace_bytes(1, 4096, 100) == 0        # K not a multiple of 128
    assert lib.pe_gemv(None, 1, 64, None, 1, None, 16, None, 0, 1, 128, 128, None, 1, 16, None, 1, 16, 128, None, 0, None) == -1
    assert lib.pe_fwht128(None, 1, 128, None, 0, 128, 1, 128, 128, None) == -1
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p += (-p) % 16
    assert lib.pe_fwht128(p, 1, 128, p, 0, 128, 1, 100, 300, None) == -2   # padded size not a multiple of 128
    assert lib.pe_pack_nibble(p, p, 1, 100, None) == -2
