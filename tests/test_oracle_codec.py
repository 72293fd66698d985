"""The CPU oracle's codecs against the reference's known answers and against
independent converters (torch's float8_e4m3fn, numpy's float16)."""
import json
import math
import os

import numpy as np
import pytest

import oracle

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_kats.json")))


def _val(x):
    if isinstance(x, str):
        return {"inf": math.inf, "-inf": -math.inf, "nan": math.nan, "-nan": -math.nan}[x]
    return x


def test_e4m3_reference_kats():
    # src/backend/vulkan/fp8_ext.rs:225-263
    for x, code in GOLD["e4m3_encode"]:
        assert oracle.f32_to_e4m3(x) == code, (x, code)
    for code, x in GOLD["e4m3_decode"]:
        got = oracle.e4m3_to_f32(code)
        assert got == x and math.copysign(1, got) == math.copysign(1, x), (code, x)


def test_e4m3_edges():
    for x, code in GOLD["e4m3_edges"]:
        if x == "-nan":
            bits = np.array([0xFFC00000], np.uint32)
            got = int(oracle.e4m3_range(int(bits[0]), 1)[0])
        else:
            got = oracle.f32_to_e4m3(_val(x))
        assert got == code, (x, hex(got), hex(code))


def test_e4m3_decode_all_codes_roundtrip():
    # every finite code decodes to a value that encodes back to itself
    for b in range(256):
        if b & 0x7F == 0x7F:
            assert math.isnan(oracle.e4m3_to_f32(b))
            continue
        assert oracle.f32_to_e4m3(oracle.e4m3_to_f32(b)) == b


def test_e4m3_matches_torch_in_range():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(7)
    bits = rng.integers(0, 2**32, size=2_000_000, dtype=np.uint64).astype(np.uint32)
    x = bits.view(np.float32)
    ours = oracle.kv_store_fp8(x)[: x.size]
    theirs = torch.from_numpy(x.copy()).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    # torch turns out-of-range values into NaN instead of saturating; compare below the clamp
    sel = np.isfinite(x) & (np.abs(x) < 448.0)
    assert np.array_equal(ours[sel], theirs[sel])
    big = np.isfinite(x) & (np.abs(x) >= 448.0)
    assert np.all((ours[big] & 0x7F) == 0x7E)


def test_e4m3_dense_sweep_small_magnitudes():
    # all floats in [2^-12, 2^-5): subnormal / normal boundary of E4M3, checked against torch
    torch = pytest.importorskip("torch")
    lo, hi = np.float32(2.0**-12).view(np.uint32), np.float32(2.0**-5).view(np.uint32)
    ours = oracle.e4m3_range(int(lo), int(hi - lo))
    x = np.arange(lo, hi, dtype=np.uint32).view(np.float32)
    theirs = torch.from_numpy(x.copy()).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(ours, theirs)


def test_f16_matches_numpy_rne():
    rng = np.random.default_rng(8)
    bits = rng.integers(0, 2**32, size=2_000_000, dtype=np.uint64).astype(np.uint32)
    x = bits.view(np.float32)
    ours = oracle.kv_copy_fp16(x)[: x.size]
    with np.errstate(all="ignore"):
        theirs = x.astype(np.float16).view(np.uint16)
    fin = ~np.isnan(x)
    assert np.array_equal(ours[fin], theirs[fin])
    nan = np.isnan(x)
    assert np.all((ours[nan] & 0x7C00) == 0x7C00) and np.all((ours[nan] & 0x03FF) != 0)


def test_store_packing_and_tail_padding():
    # vk_shaders/kv_store_fp8.comp:42-66: 4 codes per word, low byte first, zero-padded tail
    x = np.array([1.0, 2.0, -1.0, 0.5, 1.5], np.float32)
    out = oracle.kv_store_fp8(x)
    assert out.tolist() == [0x38, 0x40, 0xB8, 0x30, 0x3C, 0, 0, 0]
    words = out.view("<u4")
    assert words[0] == 0x38 | (0x40 << 8) | (0xB8 << 16) | (0x30 << 24)
    # vk_shaders/kv_copy_fp16.comp:46-50
    h = oracle.kv_copy_fp16(np.array([1.0, -2.0, 0.5], np.float32))
    assert h.tolist() == [0x3C00, 0xC000, 0x3800, 0x0000]


def test_fp8_to_f16_exact_for_all_codes():
    # examples/fp8_smoke.rs:371-397 checks all 256 codes against fp8_e4m3_to_f32
    codes = np.arange(256, dtype=np.uint8)
    h = oracle.kv_fp8_to_f16(codes).view(np.float16).astype(np.float32)
    for b in range(256):
        ref = oracle.e4m3_to_f32(b)
        if math.isnan(ref):
            assert math.isnan(h[b])
        else:
            assert h[b] == ref and math.copysign(1, h[b]) == math.copysign(1, ref)


def test_scaled_store_recipe():
    # vk_shaders/mul_coopmat_fp8_native_bn32.comp:149-152,214
    rng = np.random.default_rng(3)
    x = rng.standard_normal((8, 128)).astype(np.float32) * 30
    codes, scales = oracle.kv_store_fp8_scaled(x, 8, 128)
    for h in range(8):
        sc = max(np.float32(np.abs(x[h]).max()) * np.float32(1.0 / 448.0), np.float32(1e-12))
        assert scales[h] == sc
        inv = np.float32(1.0) / sc
        want = oracle.kv_store_fp8(np.clip(x[h] * inv, -448, 448))
        assert np.array_equal(codes.reshape(8, 128)[h], want)
    z, zs = oracle.kv_store_fp8_scaled(np.zeros(128, np.float32), 1, 128)
    assert zs[0] == np.float32(1e-12) and not z.any()
