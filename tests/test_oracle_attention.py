"""The oracle's attention restatement against the reference's own analytic cases and
algorithm-level properties (tests/correctness.rs, tests/flash_attn_tiled_ref.rs)."""
import os

import numpy as np
import pytest

import oracle
from util import GOLDEN_CASES, correctness_rs_inputs, golden_inputs, xorshift_floats


def naive_f64(q, k, v, hq, hkv, d, L, start=0, scale=None, softcap=0.0):
    """Independent numpy restatement (softmax in f64) used only to pin the C oracle."""
    scale = 1.0 / np.sqrt(d) if scale is None else scale
    g = hq // hkv
    out = np.zeros((hq, d))
    for h in range(hq):
        kk = k[start:L, h // g, :].astype(np.float64)
        vv = v[start:L, h // g, :].astype(np.float64)
        s = (kk @ q[h].astype(np.float64)) * scale
        if softcap > 0:
            s = softcap * np.tanh(s / softcap)
        p = np.exp(s - s.max())
        out[h] = (p[:, None] * vv).sum(0) / p.sum()
    return out


def test_seq1_output_equals_v():
    # tests/correctness.rs:1003-1035,1083-1123: Q=0.1, K=0.1, V=1.0, seq_len=1 -> out == 1.0 (1e-5)
    for hq, hkv, d in ((32, 8, 128), (4, 2, 64)):
        q = np.full((hq, d), 0.1, np.float32)
        k = np.full((2048, hkv, d), 0.1, np.float32)
        v = np.full((2048, hkv, d), 1.0, np.float32)
        o = oracle.attention_ref(q, k, v, oracle.F32, hq, hkv, d, 1)
        assert np.max(np.abs(o - 1.0)) < 1e-5


def test_layer_offset_binding_with_poisoned_layer0():
    # tests/correctness.rs:899-998: layer 0 = 999.0 garbage, layer 1 K=0.1 V=1.0, bind at layer 1
    hq, hkv, d, max_seq = 32, 8, 128, 2048
    lay = oracle.make_layout(2, hkv, d, max_seq, oracle.F32)
    off = oracle.lib().vfo_layer_offset_bytes(lay, 1) // 4
    size = max_seq * hkv * d
    k = np.full(2 * size, 999.0, np.float32)
    v = np.full(2 * size, 999.0, np.float32)
    k[off:off + size] = 0.1
    v[off:off + size] = 1.0
    q = np.full((hq, d), 0.1, np.float32)
    o = oracle.attention_ref(q, k[off:], v[off:], oracle.F32, hq, hkv, d, 1)
    assert np.max(np.abs(o - 1.0)) < 1e-5


@pytest.mark.parametrize("seq_len", [64, 200, 2048])
def test_split_reduce_matches_cpu_reference(seq_len):
    # tests/correctness.rs:2875-2894: split+reduce vs cpu_attention_reference, max-abs < 1e-3
    hq, hkv, d = 32, 8, 128
    q, k, v = correctness_rs_inputs(hq, hkv, d, seq_len)
    ref = oracle.attention_ref(q, k, v, oracle.F32, hq, hkv, d, seq_len)
    got = oracle.flash_attn_split_reduce(q, k, v, oracle.F32, hq, hkv, d, seq_len, tile=64)
    assert np.isfinite(got).all()
    assert np.max(np.abs(got - ref)) < 1e-3
    assert np.max(np.abs(ref - naive_f64(q, k, v, hq, hkv, d, seq_len))) < 1e-5


@pytest.mark.parametrize("kv_len,tile,seed", [(16, 4, 42), (64, 32, 43), (50, 32, 47), (96, 16, 45), (1152, 32, 200)])
def test_tiled_equals_naive_xorshift(kv_len, tile, seed):
    # tests/flash_attn_tiled_ref.rs:238-303 (tiled online softmax == naive, < 1e-4), one query row
    d = 128
    q = xorshift_floats(d, seed).reshape(1, d)
    k = xorshift_floats(kv_len * d, seed + 1).reshape(kv_len, 1, d)
    v = xorshift_floats(kv_len * d, seed + 2).reshape(kv_len, 1, d)
    a = oracle.attention_ref(q, k, v, oracle.F32, 1, 1, d, kv_len)
    b = oracle.flash_attn_split_reduce(q, k, v, oracle.F32, 1, 1, d, kv_len, tile=tile)
    assert np.max(np.abs(a - b)) < 1e-4
    assert np.max(np.abs(a - naive_f64(q, k, v, 1, 1, d, kv_len))) < 1e-5


def test_kv_start_masks_prefix_in_both_forms():
    # vk_shaders/flash_attn_split.comp:98-113: positions below kv_start contribute nothing
    hq, hkv, d, L, start = 8, 2, 64, 300, 171
    rng = np.random.default_rng(5)
    q = rng.standard_normal((hq, d), dtype=np.float32)
    k = rng.standard_normal((L, hkv, d), dtype=np.float32)
    v = rng.standard_normal((L, hkv, d), dtype=np.float32)
    a = oracle.attention_ref(q, k, v, oracle.F32, hq, hkv, d, L, start)
    b = oracle.flash_attn_split_reduce(q, k, v, oracle.F32, hq, hkv, d, L, start, tile=64)
    c = oracle.attention_ref(q, k[start:], v[start:], oracle.F32, hq, hkv, d, L - start)
    assert np.max(np.abs(a - b)) < 1e-4
    assert np.array_equal(a, c)
    assert np.max(np.abs(a - naive_f64(q, k, v, hq, hkv, d, L, start))) < 1e-5


@pytest.mark.parametrize("dt", [oracle.F16, oracle.F8])
def test_quantised_cache_reads_dequantised_values(dt):
    hq, hkv, d, L = 8, 2, 128, 100
    rng = np.random.default_rng(6)
    q = rng.standard_normal((hq, d), dtype=np.float32)
    k = rng.standard_normal((L, hkv, d), dtype=np.float32)
    v = rng.standard_normal((L, hkv, d), dtype=np.float32)
    kc, vc = oracle.store(k, dt).reshape(k.shape), oracle.store(v, dt).reshape(v.shape)
    if dt == oracle.F16:
        kd, vd = kc.view(np.float16).astype(np.float32), vc.view(np.float16).astype(np.float32)
    else:
        lut = np.array([oracle.e4m3_to_f32(b) for b in range(256)], np.float32)
        kd, vd = lut[kc], lut[vc]
    a = oracle.attention_ref(q, kc, vc, dt, hq, hkv, d, L)
    b = oracle.attention_ref(q, kd, vd, oracle.F32, hq, hkv, d, L)
    assert np.array_equal(a, b)


def test_softcap_and_scales_extensions():
    hq, hkv, d, L = 4, 2, 64, 90
    rng = np.random.default_rng(9)
    q = rng.standard_normal((hq, d), dtype=np.float32) * 4
    k = rng.standard_normal((L, hkv, d), dtype=np.float32)
    v = rng.standard_normal((L, hkv, d), dtype=np.float32)
    a = oracle.attention_ref(q, k, v, oracle.F32, hq, hkv, d, L, softcap=5.0)
    assert np.max(np.abs(a - naive_f64(q, k, v, hq, hkv, d, L, softcap=5.0))) < 1e-5
    ks = rng.random((L, hkv), dtype=np.float32) + 0.5
    vs = rng.random((L, hkv), dtype=np.float32) + 0.5
    b = oracle.attention_ref(q, k, v, oracle.F32, hq, hkv, d, L, k_scales=ks, v_scales=vs)
    c = naive_f64(q, k * ks[:, :, None], v * vs[:, :, None], hq, hkv, d, L)
    assert np.max(np.abs(b - c)) < 1e-5


def test_rope_neox_matches_reference_cpu_form():
    # tests/correctness.rs:819-838: head_dim 128, theta 1e6, positions 0 / 100 / 4096
    d = 128
    x = (0.1 + 3.4 * np.arange(d, dtype=np.float32) / np.float32(d - 1)).astype(np.float32)
    assert np.array_equal(oracle.rope_neox(x, 1, d, d, 0, 1e6), x)
    for pos, tol in ((100, 1e-4), (4096, 5e-4)):
        y = oracle.rope_neox(x, 1, d, d, pos, 1e6)
        half = d // 2
        i = np.arange(half)
        theta = pos * (1e6 ** (-2.0 * i / d))
        want = np.concatenate([x[:half] * np.cos(theta) - x[half:] * np.sin(theta),
                               x[:half] * np.sin(theta) + x[half:] * np.cos(theta)])
        assert np.max(np.abs(y - want)) < tol


def test_golden_attention_outputs_are_reproduced():
    import zlib
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "attention_small.npz"))
    for i, (name, hq, hkv, d, L, start, dt, cap) in enumerate(GOLDEN_CASES):
        q, kc, vc = golden_inputs(i)
        crc = zlib.crc32(q.tobytes()) ^ zlib.crc32(kc.tobytes()) ^ zlib.crc32(vc.tobytes())
        assert np.uint32(crc) == gold[name + "/crc"], "seeded generator drifted; regenerate the fixtures"
        o = oracle.attention_ref(q, kc, vc, dt, hq, hkv, d, L, start, None, cap)
        assert np.array_equal(o, gold[name + "/out"])


def test_decode_step_appends_then_attends():
    hq, hkv, d, n_seqs, slab = 8, 2, 64, 3, 40
    rng = np.random.default_rng(11)
    lens = np.array([1, 17, 40], np.uint32)
    for dt in (oracle.F32, oracle.F16, oracle.F8):
        k = np.zeros((n_seqs, slab, hkv, d), oracle.NP_DTYPE[dt])
        v = np.zeros_like(k)
        kf = rng.standard_normal((n_seqs, slab, hkv, d), dtype=np.float32)
        vf = rng.standard_normal((n_seqs, slab, hkv, d), dtype=np.float32)
        for s in range(n_seqs):
            k[s, : lens[s] - 1] = oracle.store(kf[s, : lens[s] - 1], dt).reshape(-1, hkv, d)
            v[s, : lens[s] - 1] = oracle.store(vf[s, : lens[s] - 1], dt).reshape(-1, hkv, d)
        q = rng.standard_normal((n_seqs, hq, d), dtype=np.float32)
        kn = np.stack([kf[s, lens[s] - 1] for s in range(n_seqs)])
        vn = np.stack([vf[s, lens[s] - 1] for s in range(n_seqs)])
        out = oracle.decode_step(q, kn, vn, k, v, dt, n_seqs, slab, hq, hkv, d, lens)
        for s in range(n_seqs):
            assert np.array_equal(k[s, lens[s] - 1], oracle.store(kn[s], dt).reshape(hkv, d))
            ref = oracle.attention_ref(q[s], k[s], v[s], dt, hq, hkv, d, int(lens[s]))
            assert np.array_equal(out[s], ref)
