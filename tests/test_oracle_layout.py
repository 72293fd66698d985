"""Cache layout arithmetic of the oracle against the integers the reference asserts
(src/backend/vulkan/kv_cache.rs:502-586)."""
import json
import os

import oracle

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_kats.json")))["layout"]


def test_element_sizes():
    L = oracle.lib()
    assert [L.vfo_elem_size(d) for d in (oracle.F32, oracle.F16, oracle.F8)] == [4, 2, 1]


def test_bytes_per_token_uniform_and_fp8_half():
    g = GOLD["bytes_per_token_uniform_f16"]
    f16 = oracle.kv_bytes_per_token(g["n_layers"], g["n_kv_heads"], g["head_dim"], None, None, g["elem"])
    assert f16 == g["expect"]
    lay = oracle.make_layout(g["n_layers"], g["n_kv_heads"], g["head_dim"], 12288, oracle.F16)
    assert f16 * 12288 == 2 * oracle.bytes_per_buffer(lay)
    fp8 = oracle.kv_bytes_per_token(g["n_layers"], g["n_kv_heads"], g["head_dim"], None, None, 1)
    assert fp8 * 2 == f16


def test_bytes_per_token_heterogeneous():
    g = GOLD["bytes_per_token_hetero_fp8"]
    assert oracle.kv_bytes_per_token(4, 999, 999, g["plhd"], g["plkv"], g["elem"]) == g["expect"]


def test_layer_size_scales_with_dtype():
    for key, dt in (("qwen3_8b_f32_total", oracle.F32), ("qwen3_8b_f16_total", oracle.F16)):
        g = GOLD[key]
        lay = oracle.make_layout(g["n_layers"], g["n_kv_heads"], g["head_dim"], g["max_seq"], dt)
        assert 2 * oracle.bytes_per_buffer(lay) == g["expect_bytes"]
        assert oracle.lib().vfo_layer_size_bytes(lay, 0) * g["n_layers"] * 2 == g["expect_bytes"]


def test_offsets_uniform_and_heterogeneous():
    L = oracle.lib()
    lay = oracle.make_layout(36, 8, 128, 2048, oracle.F8)
    assert L.vfo_row_bytes(lay, 3) == 1024
    assert L.vfo_layer_offset_bytes(lay, 5) == 5 * 2048 * 1024
    assert L.vfo_pos_offset_bytes(lay, 5, 77) == 5 * 2048 * 1024 + 77 * 1024
    het = oracle.make_layout(4, 999, 999, 100, oracle.F16, [256, 256, 512, 512], [2, 2, 4, 4])
    sizes = [100 * 2 * 256 * 2, 100 * 2 * 256 * 2, 100 * 4 * 512 * 2, 100 * 4 * 512 * 2]
    for i in range(4):
        assert L.vfo_layer_size_bytes(het, i) == sizes[i]
        assert L.vfo_layer_offset_bytes(het, i) == sum(sizes[:i])
    assert oracle.bytes_per_buffer(het) == sum(sizes)
    assert L.vfo_pos_offset_bytes(het, 2, 9) == sum(sizes[:2]) + 9 * 4 * 512 * 2


def test_overflow_is_an_error():
    lay = oracle.make_layout(2**31, 2**31, 2**31, 2**31, oracle.F32)
    assert oracle.bytes_per_buffer(lay) is None


def test_sliding_kv_start():
    # src/backend/vulkan/forward/arch/gemma4.rs:59-73
    L = oracle.lib()
    assert L.vfo_sliding_kv_start(0, 1024) == 0
    assert L.vfo_sliding_kv_start(1023, 1024) == 0
    assert L.vfo_sliding_kv_start(1024, 1024) == 1
    assert L.vfo_sliding_kv_start(32767, 1024) == 32768 - 1024
