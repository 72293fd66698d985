"""The named workloads at full size: append + decode attention checked against the CPU oracle
where it finishes in seconds, and through size-independent properties (append-then-read bytes,
partial/merge == whole, split-count invariance) everywhere."""
import numpy as np
import pytest

import oracle
import vulkanforge_b200 as vf
from util import dev_view_bytes, kv_values, rel_err, to_dev

pytestmark = pytest.mark.gpu


def fill_cache(fwd, rng, layer, slot, n, hkv, d, fp8, chunk=4096):
    """Pre-fills positions [0, n) of one slab through the product's own prefill append and
    returns the f32 values that were stored."""
    k = kv_values(rng, (n, hkv, d), outlier_frac=0.01 if fp8 else 0.0)
    v = kv_values(rng, (n, hkv, d), outlier_frac=0.01 if fp8 else 0.0)
    for p in range(0, n, chunk):
        m = min(chunk, n - p)
        fwd.b_step_kv_write(layer, to_dev(k[p:p + m]), to_dev(v[p:p + m]), m, p, slot)
    return k, v


def slab_bytes(cache, layer, slot, n_rows):
    off = cache.slot_offset_bytes(layer, slot)
    nb = n_rows * cache.row_bytes(layer)
    return dev_view_bytes(cache.k_buffer + off, nb), dev_view_bytes(cache.v_buffer + off, nb)


def test_config1_llama8b_f16_2048(ctx):
    """32 q / 8 kv / 128, F16, 2047 pre-filled + 1 appended, RoPE-NeoX theta 500000 on Q and K,
    scale 1/sqrt(128); max-abs error < 2e-3."""
    import torch
    hq, hkv, d, L = 32, 8, 128, 2048
    rng = np.random.default_rng(1)
    cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, L), vf.KvDtype.F16)
    fwd = vf.CudaForward(ctx, cache, n_heads=hq)
    try:
        k = rng.standard_normal((L, hkv, d), dtype=np.float32)
        v = rng.standard_normal((L, hkv, d), dtype=np.float32)
        for t in range(L):
            k[t] = oracle.rope_neox(k[t], hkv, d, d, t, 500000.0)
        q = oracle.rope_neox(rng.standard_normal((hq, d), dtype=np.float32), hq, d, d, L - 1, 500000.0)
        fwd.b_step_kv_write(0, to_dev(k[:L - 1]), to_dev(v[:L - 1]), L - 1, 0)
        out = torch.zeros(hq, d, device="cuda")
        pos = to_dev(np.array([L - 1], np.uint32))
        fwd.decode_step(0, to_dev(q), to_dev(k[L - 1:]), to_dev(v[L - 1:]), out, None, pos, 1)
        torch.cuda.synchronize()
        kb, vb = slab_bytes(cache, 0, 0, L)
        assert np.array_equal(kb.view(np.uint16), oracle.kv_copy_fp16(k))
        assert np.array_equal(vb.view(np.uint16), oracle.kv_copy_fp16(v))
        want = oracle.attention_ref(q, kb.view(np.uint16), vb.view(np.uint16), oracle.F16, hq, hkv, d, L)
        assert float(np.max(np.abs(out.cpu().numpy() - want))) < 2e-3
    finally:
        fwd.workspace.destroy()
        cache.destroy()


def test_config2_qwen3_fp8_8192_16_splits(ctx):
    """FP8, 32 q / 8 kv / 128, context 8192, 16 splits, several of the 36 layers."""
    import torch
    hq, hkv, d, L, n_layers = 32, 8, 128, 8192, 4
    rng = np.random.default_rng(2)
    cache = vf.KvCache(ctx, vf.KvCacheConfig(n_layers, hkv, d, L), vf.KvDtype.F8)
    fwd = vf.CudaForward(ctx, cache, n_heads=hq, n_splits=16)
    try:
        for layer in range(n_layers):
            k, v = fill_cache(fwd, rng, layer, 0, L - 1, hkv, d, True)
            kn, vn = kv_values(rng, (1, hkv, d)), kv_values(rng, (1, hkv, d))
            q = rng.standard_normal((hq, d), dtype=np.float32)
            out = torch.zeros(hq, d, device="cuda")
            fwd.decode_step(layer, to_dev(q), to_dev(kn), to_dev(vn), out, None, to_dev(np.array([L - 1], np.uint32)), 1)
            torch.cuda.synchronize()
            kb, vb = slab_bytes(cache, layer, 0, L)
            assert np.array_equal(kb, oracle.kv_store_fp8(np.concatenate([k, kn])))      # bit-exact cache
            assert np.array_equal(vb, oracle.kv_store_fp8(np.concatenate([v, vn])))
            want = oracle.attention_ref(q, kb, vb, oracle.F8, hq, hkv, d, L)
            assert rel_err(out.cpu().numpy(), want) < 3e-2
    finally:
        fwd.workspace.destroy()
        cache.destroy()


def test_config3_batch64_ragged_fp8(ctx):
    """64 sequences, lengths U[512, 16384], one appended token each, FP8."""
    import torch
    hq, hkv, d, n_seqs, max_seq = 32, 8, 128, 64, 16384
    rng = np.random.default_rng(3)
    lens = rng.integers(512, 16385, n_seqs).astype(np.uint32)
    cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, max_seq, n_slots=n_seqs), vf.KvDtype.F8)
    fwd = vf.CudaForward(ctx, cache, n_heads=hq, max_batch=n_seqs)
    try:
        for s in range(n_seqs):
            fill_cache(fwd, rng, 0, s, int(lens[s]) - 1, hkv, d, True, chunk=8192)
        q = rng.standard_normal((n_seqs, hq, d), dtype=np.float32)
        kn, vn = kv_values(rng, (n_seqs, hkv, d)), kv_values(rng, (n_seqs, hkv, d))
        out = torch.zeros(n_seqs, hq, d, device="cuda")
        fwd.decode_step(0, to_dev(q), to_dev(kn), to_dev(vn), out, None, to_dev(lens - 1), n_seqs, int(lens.max()))
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        for s in range(n_seqs):
            kb, vb = slab_bytes(cache, 0, s, int(lens[s]))
            assert np.array_equal(kb[-1024:], oracle.kv_store_fp8(kn[s]))
            want = oracle.attention_ref(q[s], kb, vb, oracle.F8, hq, hkv, d, int(lens[s]))
            assert rel_err(got[s], want) < 3e-2
    finally:
        fwd.workspace.destroy()
        cache.destroy()


def test_config4_gemma_f16_window_softcap(ctx):
    """16 q / 8 kv / 256, F16, context 32768, sliding (window 1024) and global layers, soft-cap 50."""
    import torch
    hq, hkv, d, L, B = 16, 8, 256, 32768, 2
    rng = np.random.default_rng(4)
    cache = vf.KvCache(ctx, vf.KvCacheConfig(2, hkv, d, L, n_slots=B), vf.KvDtype.F16)
    fwd = vf.CudaForward(ctx, cache, n_heads=hq, max_batch=B, sliding_window=1024, sliding_layers=[0], softcap=50.0)
    try:
        for layer in range(2):
            for s in range(B):
                fill_cache(fwd, rng, layer, s, L - 1, hkv, d, False, chunk=8192)
            q = rng.standard_normal((B, hq, d), dtype=np.float32)
            kn = rng.standard_normal((B, hkv, d), dtype=np.float32)
            vn = rng.standard_normal((B, hkv, d), dtype=np.float32)
            out = torch.zeros(B, hq, d, device="cuda")
            pos = np.full(B, L - 1, np.uint32)
            fwd.decode_step(layer, to_dev(q), to_dev(kn), to_dev(vn), out, None, to_dev(pos), B, L)
            torch.cuda.synchronize()
            got = out.cpu().numpy()
            start = L - 1024 if layer == 0 else 0
            for s in range(B):
                kb, vb = slab_bytes(cache, layer, s, L)
                want = oracle.attention_ref(q[s], kb.view(np.uint16), vb.view(np.uint16), oracle.F16, hq, hkv, d, L,
                                            start, None, 50.0)
                assert float(np.max(np.abs(got[s] - want))) < 2e-3
    finally:
        fwd.workspace.destroy()
        cache.destroy()


def test_config5_long_context_fp8_chunked_prefill_and_sharded_merge(ctx):
    """64 q / 8 kv / 128, FP8, context 131072: a 512-token prefill chunk lands bit-exactly, and the
    attention over 8 position shards merged from (m, l, o) partials equals the single-pass result."""
    import torch
    hq, hkv, d, L = 64, 8, 128, 131072
    rng = np.random.default_rng(5)
    cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, L), vf.KvDtype.F8)
    fwd = vf.CudaForward(ctx, cache, n_heads=hq)
    try:
        k, v = fill_cache(fwd, rng, 0, 0, L - 512, hkv, d, True, chunk=16384)
        kc, vc = kv_values(rng, (512, hkv, d)), kv_values(rng, (512, hkv, d))
        fwd.b_step_kv_write(0, to_dev(kc), to_dev(vc), 512, L - 512)       # the chunked-prefill append
        kb, vb = slab_bytes(cache, 0, 0, L)
        assert np.array_equal(kb[-512 * 1024:], oracle.kv_store_fp8(kc))
        assert np.array_equal(vb[-512 * 1024:], oracle.kv_store_fp8(vc))
        assert np.array_equal(kb[:(L - 512) * 1024], oracle.kv_store_fp8(k))
        q = rng.standard_normal((hq, d), dtype=np.float32)
        dq = to_dev(q)
        full = torch.zeros(hq, d, device="cuda")
        fwd.step_attention(0, dq, full, L - 1)
        G = 8
        m = torch.zeros(G, hq, device="cuda"); l = torch.zeros(G, hq, device="cuda")
        o = torch.zeros(G, hq, d, device="cuda")
        for g in range(G):
            fwd.attend_partial(0, dq, g * L // G, (g + 1) * L // G, m[g], l[g], o[g])
        merged = torch.zeros(hq, d, device="cuda")
        fwd.merge_partials(m, l, o, G, hq, d, merged)
        torch.cuda.synchronize()
        want = oracle.attention_ref(q, kb, vb, oracle.F8, hq, hkv, d, L)
        assert rel_err(full.cpu().numpy(), want) < 3e-2
        assert rel_err(merged.cpu().numpy(), want) < 3e-2
        assert rel_err(merged.cpu().numpy(), full.cpu().numpy()) < 1e-3
    finally:
        fwd.workspace.destroy()
        cache.destroy()


def device_fill(fwd, gen, layer, slot, n, hkv, d, fp8, chunk=8192):
    """Pre-fills positions [0, n) from a device-side generator (N(0,1), 1 % x20 outliers for FP8);
    the oracle later reads the cache bytes back, so the values themselves need not reach the host."""
    import torch
    for p in range(0, n, chunk):
        m = min(chunk, n - p)
        kv = torch.randn(2, m, hkv * d, device="cuda", generator=gen)
        if fp8:
            kv = torch.where(torch.rand(2, m, hkv * d, device="cuda", generator=gen) < 0.01, kv * 20.0, kv)
        fwd.b_step_kv_write(layer, kv[0], kv[1], m, p, slot)


def test_config2_all_36_layers_in_one_decode_token_call(ctx):
    """The whole workload as the benchmark runs it: 36 layers, FP8, context 8192, 16 splits, one
    vfkv_decode_token call (36 fused launches), dependent-launch mode 2.  A sample of layers is
    checked against the oracle reading that layer's cache bytes; the appended rows are bit-exact."""
    import torch
    hq, hkv, d, L, n_layers = 32, 8, 128, 8192, 36
    rng = np.random.default_rng(22)
    gen = torch.Generator(device="cuda").manual_seed(22)
    cache = vf.KvCache(ctx, vf.KvCacheConfig(n_layers, hkv, d, L), vf.KvDtype.F8)
    fwd = vf.CudaForward(ctx, cache, n_heads=hq, n_splits=16)
    stream = torch.cuda.Stream()
    try:
        for layer in range(n_layers):
            device_fill(fwd, gen, layer, 0, L - 1, hkv, d, True)
        q = rng.standard_normal((n_layers, 1, hq, d), dtype=np.float32)
        kn, vn = kv_values(rng, (n_layers, 1, hkv, d)), kv_values(rng, (n_layers, 1, hkv, d))
        out = torch.zeros(n_layers, 1, hq, d, device="cuda")
        dq, dk, dv, dpos = to_dev(q), to_dev(kn), to_dev(vn), to_dev(np.array([L - 1], np.uint32))
        torch.cuda.synchronize()
        fwd.stream = stream.cuda_stream
        ctx.set_dependent_launch(2)
        with torch.cuda.stream(stream):
            fwd.decode_token(dq, dk, dv, out, None, dpos, 1, L)
        stream.synchronize()
        ctx.poll()
        got = out.cpu().numpy()
        for layer in (0, 1, 17, 34, 35):
            kb, vb = slab_bytes(cache, layer, 0, L)
            assert np.array_equal(kb[-1024:], oracle.kv_store_fp8(kn[layer, 0]))
            assert np.array_equal(vb[-1024:], oracle.kv_store_fp8(vn[layer, 0]))
            want = oracle.attention_ref(q[layer, 0], kb, vb, oracle.F8, hq, hkv, d, L)
            err = rel_err(got[layer, 0], want)
            assert err < 3e-2, (layer, err)
            assert err < 1e-4, ("regression gate", layer, err)
    finally:
        ctx.set_dependent_launch(0)
        fwd.workspace.destroy()
        cache.destroy()


def test_config4_batch8_over_the_six_layer_period_in_one_decode_token_call(ctx):
    """The Gemma-style workload at its stated size: batch 8, context 32768, F16, head_dim 256, five
    sliding layers (window 1024) and one global layer, soft-cap 50, through vfkv_decode_token with
    its per-layer windows.  A sliding and the global layer are checked for the first and the last
    sequence against the oracle."""
    import torch
    hq, hkv, d, L, B, n_layers = 16, 8, 256, 32768, 8, 6
    rng = np.random.default_rng(44)
    gen = torch.Generator(device="cuda").manual_seed(44)
    cache = vf.KvCache(ctx, vf.KvCacheConfig(n_layers, hkv, d, L, n_slots=B), vf.KvDtype.F16)
    fwd = vf.CudaForward(ctx, cache, n_heads=hq, max_batch=B, sliding_window=1024, sliding_layers=[0, 1, 2, 3, 4],
                         softcap=50.0)
    stream = torch.cuda.Stream()
    try:
        for layer in range(n_layers):
            for s in range(B):
                device_fill(fwd, gen, layer, s, L - 1, hkv, d, False, chunk=16384)
        q = rng.standard_normal((n_layers, B, hq, d), dtype=np.float32)
        kn = rng.standard_normal((n_layers, B, hkv, d), dtype=np.float32)
        vn = rng.standard_normal((n_layers, B, hkv, d), dtype=np.float32)
        out = torch.zeros(n_layers, B, hq, d, device="cuda")
        dq, dk, dv = to_dev(q), to_dev(kn), to_dev(vn)
        dpos = to_dev(np.full(B, L - 1, np.uint32))
        torch.cuda.synchronize()
        fwd.stream = stream.cuda_stream
        ctx.set_dependent_launch(2)
        with torch.cuda.stream(stream):
            fwd.decode_token(dq, dk, dv, out, None, dpos, B, L)
        stream.synchronize()
        ctx.poll()
        got = out.cpu().numpy()
        for layer in (3, 5):
            start = L - 1024 if layer < 5 else 0
            for s in (0, B - 1):
                kb, vb = slab_bytes(cache, layer, s, L)
                assert np.array_equal(kb.view(np.uint16)[-hkv * d:], oracle.kv_copy_fp16(kn[layer, s]))
                want = oracle.attention_ref(q[layer, s], kb.view(np.uint16), vb.view(np.uint16), oracle.F16, hq, hkv, d,
                                            L, start, None, 50.0)
                err = float(np.max(np.abs(got[layer, s] - want)))
                assert err < 2e-3, (layer, s, err)
                assert err < 2e-5, ("regression gate", layer, s, err)
    finally:
        ctx.set_dependent_launch(0)
        fwd.workspace.destroy()
        cache.destroy()
