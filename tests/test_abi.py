"""The C-ABI library loads without a GPU and exports every symbol include/*.h declares;
host-only entry points behave like their reference counterparts."""
import ctypes as C
import os
import re

import pytest

import vulkanforge_b200 as vf
from vulkanforge_b200 import _lib

INCLUDE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include")


def declared_functions():
    names = set()
    for header in sorted(os.listdir(INCLUDE)):
        if not header.endswith(".h"):
            continue
        text = open(os.path.join(INCLUDE, header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(vfkv_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_functions()
    assert len(names) >= 50
    lib = C.CDLL(vf.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ but not exported"
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)
    assert vf.load().vfkv_abi_version() == 1


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libvfkv.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.load()


def test_element_sizes_and_labels():
    # src/backend/vulkan/kv_cache.rs:505-515
    assert [d.element_size() for d in (vf.KvDtype.F32, vf.KvDtype.F16, vf.KvDtype.F8)] == [4, 2, 1]
    assert [d.label() for d in (vf.KvDtype.F32, vf.KvDtype.F16, vf.KvDtype.F8)] == ["FP32", "FP16", "FP8"]


def test_kv_bytes_per_token_matches_reference_integers():
    # kv_cache.rs:517-558
    f16 = vf.kv_bytes_per_token(40, 8, 128, None, None, 2)
    assert f16 == 2 * 2 * 40 * 8 * 128
    assert vf.kv_bytes_per_token(40, 8, 128, None, None, 1) * 2 == f16
    assert vf.kv_bytes_per_token(4, 999, 999, [256, 256, 512, 512], [2, 2, 4, 4], 1) == 10_240


def test_kv_dtype_from_env(monkeypatch):
    # kv_cache.rs:85-101
    monkeypatch.delenv("VULKANFORGE_KV_FP8", raising=False)
    monkeypatch.delenv("VULKANFORGE_FP16_KV", raising=False)
    assert vf.kv_dtype_from_env() == vf.KvDtype.F16
    monkeypatch.setenv("VULKANFORGE_FP16_KV", "0")
    assert vf.kv_dtype_from_env() == vf.KvDtype.F32
    monkeypatch.setenv("VULKANFORGE_KV_FP8", "TRUE")
    assert vf.kv_dtype_from_env() == vf.KvDtype.F8
    monkeypatch.setenv("VULKANFORGE_KV_FP8", "0")
    assert vf.kv_dtype_from_env() == vf.KvDtype.F32


def test_guard_kv_precision():
    # kv_cache.rs:588-630
    for kv in (vf.KvDtype.F32, vf.KvDtype.F16):
        with pytest.raises(vf.VfkvError) as e:
            vf.guard_kv_precision(True, kv, False)
        assert "VULKANFORGE_KV_FP8=1" in str(e.value)
        vf.guard_kv_precision(True, kv, True)
        vf.guard_kv_precision(False, kv, False)
    vf.guard_kv_precision(True, vf.KvDtype.F8, False)


def test_sliding_kv_start():
    assert vf.sliding_kv_start(0, 1024) == 0
    assert vf.sliding_kv_start(1024, 1024) == 1
    assert vf.sliding_kv_start(32767, 1024) == 31744


def test_null_handles_are_rejected_not_dereferenced():
    L = vf.load()
    assert L.vfkv_ctx_destroy(None) == 0
    assert L.vfkv_cache_destroy(None) == 0
    assert L.vfkv_cache_zero_fill(None, None) != 0
    assert L.vfkv_cache_row_bytes(None, 0) == 0
    assert L.vfkv_append(None, 0, None, None, 1, 0, 0, None) != 0
    assert L.vfkv_last_error(None) == b"null context"
    assert L.vfkv_status_string(6).startswith(b"device-side")
