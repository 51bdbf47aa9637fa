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


def declared_arities():
    """Parameter count of every prototype in the header (comments stripped, `void` = none)."""
    text = open(os.path.join(ROOT, "include", "polar_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    out = {}
    for name, params in re.findall(r"\b(pe_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", text, flags=re.S):
        params = params.strip()
        out[name] = 0 if params in ("", "void") else params.count(",") + 1
    return out


def test_ctypes_signatures_have_the_header_arity():
    ar = declared_arities()
    assert set(ar) == set(nv.SIGNATURES)
    for name, (_, args) in nv.SIGNATURES.items():
        assert len(args) == ar[name], f"{name}: header declares {ar[name]} parameters, ctypes binds {len(args)}"


def test_size_queries_of_the_grouped_and_exchange_entry_points():
    lib = nv.lib()
    # grouped decode-size launch: counter zone + partials; too many problems for the counter zone -> 0
    assert lib.pe_gemv_grouped_workspace_bytes(160, 3712, 2688) > (4 << 20)
    assert lib.pe_gemv_grouped_workspace_bytes(60000, 3712, 2688) == 0
    assert lib.pe_gemv_grouped_workspace_bytes(8, 3712, 100) == 0
    # grouped tensor-core launch: status + tile count + tile list + bf16 activations
    assert lib.pe_gemm_grouped_workspace_bytes(128, 16384, 3712, 2688) >= 512 + 16384 * 2688 * 2
    assert lib.pe_gemm_grouped_workspace_bytes(2000, 16, 3712, 2688) == 0   # more than 1024 experts
    # exchange buffer: flags + two parities of world x rows x hidden fp32
    assert lib.pe_allreduce_buffer_bytes(8, 32, 4096) == 4096 + 2 * 8 * 32 * 4096 * 4
    assert lib.pe_allreduce_buffer_bytes(17, 1, 4096) == 0 and lib.pe_allreduce_buffer_bytes(8, 256, 4096) == 0
    assert lib.pe_decode_attention_workspace_bytes(1, 32, 8, 128) == 4096 + 8 * 16 * 4 * 130 * 4
    assert lib.pe_decode_attention_workspace_bytes(1, 32, 8, 64) == 0
    assert lib.pe_gemv_noalloc_max_bytes() == 8 << 20
    # NULL pointers are refused before anything touches a device
    assert lib.pe_moe_plan(None, None, 0, 8, 2, 4, 8, 8, None, None, None, None, None) == -1
    assert lib.pe_add_rmsnorm(None, None, 1, None, None, 1, 4096, 1e-6, None) == -1
    assert lib.pe_allreduce_add_rmsnorm(None, None, None, None, 1, 4096, 1e-6, None, 0, 1, 1, None, None, None) == -1
