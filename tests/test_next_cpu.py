"""Host-side entry points around the hot path, against the reference's own known answers
(no GPU needed: these are pure functions of the C ABI)."""
import numpy as np

import oracle
import vulkanforge_b200 as vf
from vulkanforge_b200 import _lib

G = 1024 * 1024 * 1024
HUGE = 1 << 20
SANE_CAP = 32768


def test_longest_common_prefix():
    # src/server/state.rs:49-51
    assert vf.longest_common_prefix([1, 2, 3, 4], [1, 2, 9]) == 2
    assert vf.longest_common_prefix([1, 2, 3], [1, 2, 3, 4, 5]) == 3
    assert vf.longest_common_prefix([], [1]) == 0
    assert vf.longest_common_prefix([7], [8]) == 0


def test_compute_auto_ctx_known_answers():
    # the unit tests of src/server/auto_ctx.rs (mod tests)
    kv_bpt = 160 * 1024
    ctx, bound, avail = vf.compute_auto_ctx(16 * G, 9 * G, 3 * G // 2, kv_bpt, 131072, HUGE, HUGE)
    assert bound == "VRAM" and avail == 16 * G - 9 * G - 3 * G // 2
    assert ctx <= avail // kv_bpt and ctx % 256 == 0
    assert vf.compute_auto_ctx(64 * G, 4 * G, G, 80 * 1024, 4096, HUGE, SANE_CAP)[:2] == (4096, "model max context")
    assert vf.compute_auto_ctx(64 * G, 4 * G, G, 40 * 1024, 131072, 16384, SANE_CAP)[:2] == (16384, "hardware limit")
    assert vf.compute_auto_ctx(64 * G, 4 * G, G, 40 * 1024, 131072, HUGE, SANE_CAP)[:2] == (SANE_CAP, "sane cap")
    # 10003 tokens fit -> rounded down to a multiple of 256
    kv_bpt = 100_000
    assert vf.compute_auto_ctx(10003 * kv_bpt, 0, 0, kv_bpt, 131072, HUGE, HUGE)[:2] == (9984, "VRAM")
    # pathologically tight -> floor of 512
    assert vf.compute_auto_ctx(9 * G + 100 * kv_bpt, 9 * G, 0, kv_bpt, 131072, HUGE, SANE_CAP)[:2] == (512, "VRAM")
    # weights exceed free memory: saturates
    ctx, bound, avail = vf.compute_auto_ctx(8 * G, 12 * G, G, 100_000, 131072, HUGE, SANE_CAP)
    assert (ctx, avail) == (512, 0)
    # zero divisor is treated as 1
    assert vf.compute_auto_ctx(G, 0, 0, 0, 4096, HUGE, HUGE)[0] == 4096


def test_gemma4_kv_read_layer():
    # src/backend/vulkan/forward/arch/gemma4.rs:27-49
    own, pub_s, pub_f, sub_s, sub_f = range(5)
    src = [own, own, pub_s, pub_f, sub_s, sub_s, sub_f, own]
    assert [vf.gemma4_kv_read_layer(src, i) for i in range(len(src))] == [0, 1, 2, 3, 2, 2, 3, 7]
    # a subscriber without a publisher reads itself
    assert vf.gemma4_kv_read_layer([own, sub_f], 1) == 1


def test_scalar_attn_route_threshold():
    # runs.rs:766-775: seq_len > 64 takes split + reduce
    lib = _lib.load()
    assert [lib.vfkv_scalar_attn_uses_split(p) for p in (0, 1, 62, 63, 64, 65, 8191)] == [0, 0, 0, 0, 1, 1, 1]


def test_oracle_batch_attention_properties():
    """The oracle's prefill form: query 0 at q_start 0 returns V[0]; every query equals the
    single-query oracle at its own causal length; kv_start and the per-query window mask."""
    rng = np.random.default_rng(11)
    hq, hkv, d, m, q_start = 8, 2, 64, 6, 10
    n_kv = q_start + m
    k = rng.standard_normal((n_kv, hkv, d), dtype=np.float32)
    v = rng.standard_normal((n_kv, hkv, d), dtype=np.float32)
    q = rng.standard_normal((m, hq, d), dtype=np.float32)
    out = oracle.batch_attention_ref(q, k, v, oracle.F32, hq, hkv, d, m, q_start, n_kv)
    for i in range(m):
        want = oracle.attention_ref(q[i], k, v, oracle.F32, hq, hkv, d, q_start + i + 1)
        assert np.array_equal(out[i], want)
    o0 = oracle.batch_attention_ref(q[:1], k, v, oracle.F32, hq, hkv, d, 1, 0, 1)
    assert np.allclose(o0[0], np.repeat(v[0], hq // hkv, axis=0), atol=1e-6)
    # n_kv clamps the causal length (flash_attn_batch.comp:118-119)
    oc = oracle.batch_attention_ref(q, k, v, oracle.F32, hq, hkv, d, m, q_start, q_start + 2)
    assert np.array_equal(oc[5], oracle.attention_ref(q[5], k, v, oracle.F32, hq, hkv, d, q_start + 2))
    ow = oracle.batch_attention_ref(q, k, v, oracle.F32, hq, hkv, d, m, q_start, n_kv, window=4)
    assert np.array_equal(ow[3], oracle.attention_ref(q[3], k, v, oracle.F32, hq, hkv, d, q_start + 4, q_start))
    # kv_start beyond a query's causal length: empty range -> zeros
    oz = oracle.batch_attention_ref(q, k, v, oracle.F32, hq, hkv, d, m, q_start, n_kv, kv_start=q_start + 3)
    assert not oz[0].any() and not oz[2].any() and oz[3].any()
