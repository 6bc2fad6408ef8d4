"""The C-ABI library loads and exports every symbol that include/*.h declares (no compute calls)."""
import ctypes
import os
import re

from conftest import ROOT


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            names |= set(re.findall(r"^LIGER_API[^;(]*?\b(liger_[a-z0-9_]+)\s*\(", text, flags=re.M | re.S))
    return sorted(names)


def test_header_declares_entry_points():
    syms = declared_symbols()
    assert "liger_gemm_fp16" in syms and "liger_attention_prefill" in syms and len(syms) >= 15


def test_library_exports_every_declared_symbol(liger):
    liger.build_all()
    handle = ctypes.CDLL(liger.LIB_PATH)
    missing = [s for s in declared_symbols() if not hasattr(handle, s)]
    assert not missing, f"not exported: {missing}"


def test_bindings_cover_every_declared_symbol(liger):
    assert sorted(liger.capi.SIGNATURES) == declared_symbols()


def test_version_and_error_string(liger):
    lib = liger.lib()
    assert b"sm_100a" in lib.liger_version()
    assert isinstance(lib.liger_last_error(), bytes)


def test_missing_library_fails_loudly(liger, monkeypatch):
    """No silent fallback: a missing .so is an error, not a CPU path."""
    import pytest
    monkeypatch.setattr(liger.capi, "_lib", None)
    monkeypatch.setattr(liger.capi, "LIB_PATH", "/nonexistent/libliger_b200.so")
    with pytest.raises(liger.LigerError):
        liger.capi.lib()


def test_argument_validation_without_gpu(liger):
    """Bad arguments are rejected on the host before any CUDA call."""
    lib = liger.lib()
    args = liger.GemmArgs()
    assert lib.liger_gemm_fp16(ctypes.byref(args), None) == -1
    assert b"positive" in lib.liger_last_error()
    assert lib.liger_layernorm(None, None, None, None, 4, 64, None) == -1


def test_misaligned_pointers_and_short_rows_are_rejected_without_gpu(liger):
    """Entry points whose kernels use 16-byte vector accesses refuse pointers that are not 16-byte aligned, and the
    decode entry points refuse an output row shorter than heads * head_dim, before anything is launched (the
    pointers below are never dereferenced)."""
    lib = liger.lib()
    ok, odd = 0x7f0000001000, 0x7f0000001008   # 16-byte aligned / only 8-byte aligned
    assert lib.liger_add_bias_gelu(odd, ok, 4, 64, None) == -1
    assert b"aligned" in lib.liger_last_error()
    assert lib.liger_add_bias_gelu(ok, odd, 4, 64, None) == -1
    for bad in range(9):
        ptrs = [odd if i == bad else ok for i in range(9)]
        assert lib.liger_add_qkv_bias_transpose(*ptrs, 2, 8, 2, 64, None) == -1, bad
        assert b"aligned" in lib.liger_last_error()
    assert lib.liger_transpose_heads(odd, ok, 2, 8, 2, 64, None) == -1
    assert lib.liger_transpose_heads(ok, odd, 2, 8, 2, 64, None) == -1
    # decode: out row shorter than heads * head_dim; scratch not 4-byte aligned
    assert lib.liger_attention_decode(ok, ok, ok, ok, ok, 2, 4, 100, 128, 64, 4 * 64 - 8, 0.125, None) == -1
    assert b"ldo" in lib.liger_last_error()
    assert lib.liger_attention_decode(ok, ok, ok, ok, ok + 2, 2, 4, 100, 128, 64, 4 * 64, 0.125, None) == -1
    assert b"scratch" in lib.liger_last_error()
    assert lib.liger_attention_decode_noalloc(ok, ok, ok, ok, 2, 4, 100, 128, 64, 4 * 64 - 8, 0.125, None) == -1
    assert b"ldo" in lib.liger_last_error()
