"""The callers either side of the hot path on the GPU: decode attention routing
(run_scalar_attn / flash_attn), chunked-prefill causal attention over the cache, RoPE fused with
the append, and the prefix-reuse bookkeeping.  Everything is compared with the CPU oracle."""
import numpy as np
import pytest

import oracle
import vulkanforge_b200 as vf
from util import dev_view_bytes, encode_cache, kv_values, rel_err, to_dev

pytestmark = pytest.mark.gpu

ODT = {"F32": oracle.F32, "F16": oracle.F16, "F8": oracle.F8}


def _fill(fwd, k, v, layer=0, slot=0):
    fwd.b_step_kv_write(layer, to_dev(k), to_dev(v), k.shape[0], 0, slot)


def _check(got, want, dtype, abs_tol=2e-3):
    if dtype == "F8":
        assert rel_err(got, want) < 3e-2
    else:
        assert float(np.max(np.abs(got - want))) < abs_tol


# ---- decode routing (runs.rs:722-821; tests/correctness.rs:2708-2784 for the short cases) -----------
@pytest.mark.parametrize("dtype", ["F32", "F16", "F8"])
@pytest.mark.parametrize("seq_len", [1, 2, 63, 64, 65, 200])
def test_scalar_attn_routes_short_and_long(ctx, dtype, seq_len):
    import torch
    hq, hkv, d = 32, 8, 128
    rng = np.random.default_rng(seq_len)
    k, v = kv_values(rng, (seq_len, hkv, d)), kv_values(rng, (seq_len, hkv, d))
    q = rng.standard_normal((hq, d), dtype=np.float32)
    cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, 256), vf.KvDtype[dtype])
    fwd = vf.CudaForward(ctx, cache, n_heads=hq)
    try:
        _fill(fwd, k, v)
        out = torch.zeros(hq, d, device="cuda")
        n0 = ctx.launch_count()
        fwd.run_scalar_attn(to_dev(q), out, 0, seq_len - 1)
        torch.cuda.synchronize()
        kc, vc = encode_cache(k, ODT[dtype]), encode_cache(v, ODT[dtype])
        want = oracle.attention_ref(q, kc, vc, ODT[dtype], hq, hkv, d, seq_len)
        _check(out.cpu().numpy(), want, dtype, 1e-3)
        if seq_len <= 64:
            assert ctx.launch_count() - n0 == 1          # the single-pass route: one launch, no reduce
        if seq_len == 1:                                 # seq 1 => out == V (tests/correctness.rs:1003-1035)
            vdec = oracle.attention_ref(np.ones((hq, d), np.float32), kc, vc, ODT[dtype], hq, hkv, d, 1)
            assert np.allclose(out.cpu().numpy(), vdec, atol=1e-6)
        # the distinct flash_attn entry gives the same answer at any length and needs no workspace
        out2 = torch.zeros(hq, d, device="cuda")
        fwd.run_flash_attn(to_dev(q), out2, 0, seq_len - 1, 0, 0)
        torch.cuda.synchronize()
        _check(out2.cpu().numpy(), want, dtype, 1e-3)
    finally:
        fwd.workspace.destroy()
        cache.destroy()


# ---- prefill attention ---------------------------------------------------------------------------
def _reference_batch_inputs(m, q_start, hq, hkv, d):
    """The deterministic inputs of run_batch_attn (tests/correctness.rs:3093-3112), evaluated in
    f32 as there: sines / cosines of index combinations, so that a wrong stride or group size shows."""
    n_kv = q_start + m
    f = np.float32
    qi, h, dd = (a.astype(f) for a in np.meshgrid(np.arange(m), np.arange(hq), np.arange(d), indexing="ij"))
    q = np.sin(qi * f(0.017) + h * f(0.011) + dd * f(0.003)).astype(f)
    t, kh, dd = (a.astype(f) for a in np.meshgrid(np.arange(n_kv), np.arange(hkv), np.arange(d), indexing="ij"))
    k = np.cos((t + f(1.0)) * f(0.01) + dd * f(0.001) + kh * f(0.7)).astype(f)
    v = np.sin(t * f(0.013) + kh * f(0.5) + dd * f(0.0007)).astype(f)
    return q, k, v


@pytest.mark.parametrize("dtype", ["F32", "F16", "F8"])
@pytest.mark.parametrize("m,q_start,tol", [(1, 0, 1e-4), (4, 0, 1e-3), (16, 0, 1e-3), (64, 0, 1e-3), (200, 0, 1e-3),
                                           (4, 60, 1e-3)])
def test_batch_attn_reference_cases(ctx, dtype, m, q_start, tol):
    """test_batch_attn_m1/m4/m16/m64/m200_vs_cpu and _q_start_offset (tests/correctness.rs:3159-3200)
    at the reference's shape 32 / 8 / 128 and thresholds."""
    import torch
    hq, hkv, d = 32, 8, 128
    q, k, v = _reference_batch_inputs(m, q_start, hq, hkv, d)
    n_kv = q_start + m
    cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, 512), vf.KvDtype[dtype])
    fwd = vf.CudaForward(ctx, cache, n_heads=hq)
    try:
        _fill(fwd, k, v)
        out = torch.zeros(m, hq, d, device="cuda")
        fwd.run_flash_attn_batch(0, to_dev(q), out, m, q_start, n_kv, 0, 0)
        torch.cuda.synchronize()
        kc, vc = encode_cache(k, ODT[dtype]), encode_cache(v, ODT[dtype])
        want = oracle.batch_attention_ref(q, kc, vc, ODT[dtype], hq, hkv, d, m, q_start, n_kv)
        got = out.cpu().numpy()
        assert np.isfinite(got).all()
        if dtype == "F8":
            assert rel_err(got, want) < 3e-2
        else:
            assert float(np.max(np.abs(got - want))) < (tol if dtype == "F32" else max(tol, 1e-3))
    finally:
        fwd.workspace.destroy()
        cache.destroy()


@pytest.mark.parametrize("dtype,hq,hkv,d,m,q_start,kv_start,window,softcap,n_kv_cut", [
    ("F8", 32, 8, 128, 512, 1536, 0, 0, 0.0, 0),        # a 512-token chunk late in a 2048 context
    ("F8", 64, 8, 128, 100, 300, 0, 0, 0.0, 0),         # g = 8, ragged last row block
    ("F8", 32, 8, 128, 96, 200, 130, 0, 0.0, 0),        # chunk-wide kv_start (the reference's window form)
    ("F8", 32, 8, 128, 96, 200, 0, 64, 0.0, 0),         # exact per-query window
    ("F16", 32, 8, 128, 130, 70, 0, 0, 0.0, 0),
    ("F16", 16, 8, 256, 48, 500, 0, 128, 50.0, 0),      # Gemma-like: D 256, soft-cap, window
    ("F16", 8, 8, 64, 70, 0, 0, 0, 0.0, 0),             # g = 1, D 64
    ("F8", 32, 8, 256, 40, 90, 0, 0, 0.0, 0),
    ("F8", 32, 8, 128, 64, 100, 0, 0, 0.0, 20),         # n_kv below q_start + m clamps the causal length
    ("F8", 24, 8, 128, 50, 10, 0, 0, 0.0, 0),           # g = 3 does not tile 64 rows: CUDA-core kernel
    ("F32", 32, 8, 128, 33, 40, 7, 0, 30.0, 0),
    ("F8", 32, 8, 128, 80, 0, 50, 0, 0.0, 0),           # early queries have an empty range -> zeros
])
def test_prefill_attention_shapes(ctx, dtype, hq, hkv, d, m, q_start, kv_start, window, softcap, n_kv_cut):
    import torch
    n_kv = q_start + m - n_kv_cut
    rng = np.random.default_rng(m * 7 + q_start)
    # N(0,1); the x20 outliers belong to the FP8 configurations only
    frac = 0.01 if dtype == "F8" else 0.0
    k, v = kv_values(rng, (q_start + m, hkv, d), frac), kv_values(rng, (q_start + m, hkv, d), frac)
    q = rng.standard_normal((m, hq, d), dtype=np.float32)
    cache = vf.KvCache(ctx, vf.KvCacheConfig(2, hkv, d, q_start + m + 3, n_slots=2), vf.KvDtype[dtype])
    fwd = vf.CudaForward(ctx, cache, n_heads=hq, softcap=softcap)
    try:
        _fill(fwd, k, v, layer=1, slot=1)                  # non-zero layer and slot offsets
        out = torch.zeros(m, hq, d, device="cuda")
        fwd.run_flash_attn_batch(1, to_dev(q), out, m, q_start, n_kv, 1, kv_start, slot=1, window=window)
        torch.cuda.synchronize()
        kc, vc = encode_cache(k, ODT[dtype]), encode_cache(v, ODT[dtype])
        want = oracle.batch_attention_ref(q, kc, vc, ODT[dtype], hq, hkv, d, m, q_start, n_kv, kv_start, window,
                                          softcap=softcap)
        got = out.cpu().numpy()
        assert np.isfinite(got).all()
        _check(got, want, dtype)
        # the other implementations agree as well: 1 = CUDA cores, 3 = mma.sync, 2 = tensor cores
        # only, which for FP8 or F16 / head_dim 128 / g dividing 128 is the tcgen05 kernel whatever
        # the chunk size (the automatic choice takes it only for chunks that fill the GPU)
        tc5 = dtype in ("F8", "F16") and d == 128 and 128 % (hq // hkv) == 0
        for impl in (1, 3) + ((2,) if tc5 else ()):
            ctx.set_attn_impl(impl)
            out2 = torch.zeros(m, hq, d, device="cuda")
            fwd.run_flash_attn_batch(1, to_dev(q), out2, m, q_start, n_kv, 1, kv_start, slot=1, window=window)
            torch.cuda.synchronize()
            _check(out2.cpu().numpy(), want, dtype)
        # the three forms of the tcgen05 kernel (1 simple, 2 pipelined, 3 roles on separate warps),
        # whichever of them the automatic choice takes for this cache type
        if tc5:
            ctx.set_attn_impl(2)
            for stages in (1, 2, 3):
                ctx.set_attn_tuning(4, stages)
                out3 = torch.zeros(m, hq, d, device="cuda")
                fwd.run_flash_attn_batch(1, to_dev(q), out3, m, q_start, n_kv, 1, kv_start, slot=1, window=window)
                torch.cuda.synchronize()
                ctx.poll()
                _check(out3.cpu().numpy(), want, dtype)
    finally:
        ctx.set_attn_tuning(0, 0)
        ctx.set_attn_impl(0)
        fwd.workspace.destroy()
        cache.destroy()


def test_prefill_large_chunk_takes_tcgen05_and_matches_mma(ctx):
    """A chunk big enough that the automatic choice is the tcgen05 kernel (128-row blocks x kv-heads
    >= SM count): compared with the mma.sync kernel everywhere and with the oracle on sampled queries."""
    import torch
    hq, hkv, d, m, q_start = 32, 8, 128, 640, 1500
    L = q_start + m
    rng = np.random.default_rng(21)
    k, v = kv_values(rng, (L, hkv, d)), kv_values(rng, (L, hkv, d))
    q = rng.standard_normal((m, hq, d), dtype=np.float32)
    cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, L), vf.KvDtype.F8)
    fwd = vf.CudaForward(ctx, cache, n_heads=hq)
    try:
        _fill(fwd, k, v)
        outs = {}
        for impl in (0, 3):
            ctx.set_attn_impl(impl)
            out = torch.zeros(m, hq, d, device="cuda")
            fwd.run_flash_attn_batch(0, to_dev(q), out, m, q_start, L, 0, 0)
            torch.cuda.synchronize()
            outs[impl] = out.cpu().numpy()
        assert rel_err(outs[0], outs[3]) < 5e-3
        kc, vc = encode_cache(k, oracle.F8), encode_cache(v, oracle.F8)
        for i in (0, 1, 127, 128, 333, m - 1):
            want = oracle.attention_ref(q[i], kc, vc, oracle.F8, hq, hkv, d, q_start + i + 1)
            assert rel_err(outs[0][i], want) < 3e-2
    finally:
        ctx.set_attn_impl(0)
        fwd.workspace.destroy()
        cache.destroy()


@pytest.mark.parametrize("dtype,m,q_start,kv_start,window,softcap,tune", [
    ("F8", 640, 3000, 0, 0, 0.0, (8, 3)),        # 80 items of ~27 tiles in 148 shares: heads merge in the kernel
    ("F8", 1000, 3000, 100, 0, 0.0, (8, 3)),     # kv_start, ragged last row block
    ("F8", 1024, 5000, 0, 2048, 0.0, (8, 3)),    # per-query window: items start late
    ("F8", 640, 3000, 0, 0, 30.0, (8, 3)),       # soft-cap
    ("F8", 64, 20000, 0, 0, 0.0, (0, 0)),        # 8 items of 157 tiles: taken automatically, ~20 pieces an item -> merge kernel
    ("F16", 64, 20000, 0, 0, 0.0, (0, 0)),       # so few items that F16 rows take the specialised form too
    ("F16", 640, 3000, 0, 0, 0.0, (8, 3)),
])
def test_prefill_even_shares_of_tiles(ctx, dtype, m, q_start, kv_start, window, softcap, tune):
    """The specialised tcgen05 form with one CTA per SM and an even share of all K/V tiles each:
    items cut between CTAs are put together by the CTA holding the head, or by the merge kernel.
    Compared everywhere with the one-CTA-per-item form and the mma.sync kernel, and with the
    oracle on sampled queries; launches counted to see which path ran."""
    import torch
    hq, hkv, d = 32, 8, 128
    L = q_start + m
    rng = np.random.default_rng(m + q_start + window)
    frac = 0.01 if dtype == "F8" else 0.0
    k, v = kv_values(rng, (L, hkv, d), frac), kv_values(rng, (L, hkv, d), frac)
    q = rng.standard_normal((m, hq, d), dtype=np.float32)
    cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, L), vf.KvDtype[dtype])
    fwd = vf.CudaForward(ctx, cache, n_heads=hq, softcap=softcap)
    try:
        _fill(fwd, k, v)
        outs, launches = {}, {}
        for name, impl, tn in (("shares", 2, tune), ("per_item", 2, (4, 3)), ("mma", 3, (0, 0))):
            ctx.set_attn_impl(impl)
            ctx.set_attn_tuning(*tn)
            out = torch.full((m, hq, d), float("nan"), device="cuda")
            before = ctx.launch_count()
            for _ in range(2):          # twice: the second launch finds the flags of the first
                fwd.run_flash_attn_batch(0, to_dev(q), out, m, q_start, L, 0, kv_start, window=window)
            torch.cuda.synchronize()
            ctx.poll()
            launches[name] = (ctx.launch_count() - before) // 2
            outs[name] = out.cpu().numpy()
            assert np.isfinite(outs[name]).all()
        assert launches["per_item"] == 1
        many_pieces = m == 64
        assert launches["shares"] == (2 if many_pieces else 1)      # the attention kernel (+ the merge kernel)
        # row by row against the one-CTA-per-item form: both round P to half precision, against
        # different reference maxima, so they differ by ~2^-11 of a row's largest value
        diff = np.max(np.abs(outs["shares"] - outs["per_item"]), axis=-1)
        assert float(np.max(diff / np.maximum(np.max(np.abs(outs["per_item"]), axis=-1), 1e-3))) < 4e-3
        assert rel_err(outs["shares"], outs["mma"]) < 5e-3
        kc, vc = encode_cache(k, ODT[dtype]), encode_cache(v, ODT[dtype])
        for i in (0, 1, 63, m // 2, m - 1):
            causal = q_start + i + 1
            lo = max(kv_start, causal - window) if window and causal > window else kv_start
            want = oracle.attention_ref(q[i], kc, vc, ODT[dtype], hq, hkv, d, causal, kv_start=lo, softcap=softcap)
            if dtype == "F8":
                assert rel_err(outs["shares"][i], want) < 3e-2
            else:
                assert float(np.max(np.abs(outs["shares"][i] - want))) < 2e-3
    finally:
        ctx.set_attn_tuning(0, 0)
        ctx.set_attn_impl(0)
        fwd.workspace.destroy()
        cache.destroy()


def test_prefill_piece_that_never_arrives_runs_into_the_time_limit(ctx):
    """Host-side failure injection: CTA 1 does not announce its piece of the item it shares with
    CTA 0, whose bounded wait runs out: status word set, the context stays usable, and the next
    call (injection off) is right again.  Nothing faults or hangs."""
    import torch
    hq, hkv, d, m, q_start = 32, 8, 128, 640, 3000
    L = q_start + m
    rng = np.random.default_rng(9)
    k, v = kv_values(rng, (L, hkv, d), 0.01), kv_values(rng, (L, hkv, d), 0.01)
    q = to_dev(rng.standard_normal((m, hq, d), dtype=np.float32))
    cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, L), vf.KvDtype.F8)
    fwd = vf.CudaForward(ctx, cache, n_heads=hq)
    try:
        _fill(fwd, k, v)
        ctx.set_attn_impl(2)
        ctx.set_attn_tuning(8, 3)
        good = torch.zeros(m, hq, d, device="cuda")
        fwd.run_flash_attn_batch(0, q, good, m, q_start, L, 0, 0)
        torch.cuda.synchronize()
        ctx.poll()
        ctx.set_merge_wait_ms(50)
        ctx.debug_fail_split(1)
        out = torch.zeros(m, hq, d, device="cuda")
        fwd.run_flash_attn_batch(0, q, out, m, q_start, L, 0, 0)
        torch.cuda.synchronize()
        with pytest.raises(vf.VfkvError):
            ctx.poll()
        ctx.debug_fail_split(None)
        out2 = torch.zeros(m, hq, d, device="cuda")
        fwd.run_flash_attn_batch(0, q, out2, m, q_start, L, 0, 0)
        torch.cuda.synchronize()
        ctx.poll()
        assert float(((out2 - good).abs().amax(-1) / good.abs().amax(-1).clamp_min(1e-3)).max()) < 4e-3
    finally:
        ctx.debug_fail_split(None)
        ctx.set_merge_wait_ms(1000)
        ctx.set_attn_tuning(0, 0)
        ctx.set_attn_impl(0)
        fwd.workspace.destroy()
        cache.destroy()


def test_prefill_even_shares_captured_in_a_graph(ctx):
    """Inside a stream capture the cut items go through the merge kernel (a replay would find the
    flag values of the replay before); the graph replays to the same result as a direct call."""
    import torch
    hq, hkv, d, m, q_start = 32, 8, 128, 640, 3000
    L = q_start + m
    rng = np.random.default_rng(5)
    k, v = kv_values(rng, (L, hkv, d), 0.01), kv_values(rng, (L, hkv, d), 0.01)
    q = to_dev(rng.standard_normal((m, hq, d), dtype=np.float32))
    cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, L), vf.KvDtype.F8)
    stream = torch.cuda.Stream()
    fwd = vf.CudaForward(ctx, cache, n_heads=hq, stream=stream.cuda_stream)
    try:
        ctx.set_attn_impl(2)
        ctx.set_attn_tuning(8, 3)
        with torch.cuda.stream(stream):
            _fill(fwd, k, v)
            direct = torch.zeros(m, hq, d, device="cuda")
            fwd.run_flash_attn_batch(0, q, direct, m, q_start, L, 0, 0)     # allocates the scratch
            stream.synchronize()
            out = torch.zeros(m, hq, d, device="cuda")
            graph = torch.cuda.CUDAGraph()
            before = ctx.launch_count()
            with torch.cuda.graph(graph, stream=stream):
                fwd.run_flash_attn_batch(0, q, out, m, q_start, L, 0, 0)
            assert ctx.launch_count() - before == 2
            for _ in range(3):
                out.fill_(float("nan"))
                graph.replay()
                stream.synchronize()
                assert float(((out - direct).abs().amax(-1) / direct.abs().amax(-1).clamp_min(1e-3)).max()) < 4e-3
        ctx.poll()
    finally:
        ctx.set_attn_tuning(0, 0)
        ctx.set_attn_impl(0)
        fwd.workspace.destroy()
        cache.destroy()


def test_prefill_then_decode_agree(ctx):
    """The last query of a prefill chunk and a decode step at the same position see the same
    cache: their outputs agree (the force_per_token_prefill bisect of executor/attention.rs:2207-2213)."""
    import torch
    hq, hkv, d, m, q_start = 32, 8, 128, 64, 448
    rng = np.random.default_rng(3)
    k, v = kv_values(rng, (q_start + m, hkv, d)), kv_values(rng, (q_start + m, hkv, d))
    q = rng.standard_normal((m, hq, d), dtype=np.float32)
    cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, 512), vf.KvDtype.F8)
    fwd = vf.CudaForward(ctx, cache, n_heads=hq)
    try:
        _fill(fwd, k, v)
        dq = to_dev(q)
        out = torch.zeros(m, hq, d, device="cuda")
        fwd.b_step_attention(0, dq, out, m, q_start)
        dec = torch.zeros(hq, d, device="cuda")
        for i in (0, 17, m - 1):
            fwd.step_attention(0, dq[i], dec, q_start + i)
            torch.cuda.synchronize()
            assert rel_err(out[i].cpu().numpy(), dec.cpu().numpy()) < 2e-2
    finally:
        fwd.workspace.destroy()
        cache.destroy()


# ---- RoPE + append ---------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,hkv,d,n_dims,n_tokens,base_pos", [
    ("F8", 8, 128, 128, 512, 1000), ("F16", 8, 128, 128, 33, 0), ("F32", 2, 64, 64, 5, 7),
    ("F8", 8, 128, 64, 20, 300),        # partial rotary: dims 64..127 pass through
    ("F16", 4, 256, 256, 9, 8000),
    ("F8", 2, 64, 24, 6, 11),           # half of 12 does not tile 16-byte pieces: rotate, then append
])
def test_rope_append_matches_oracle(ctx, dtype, hkv, d, n_dims, n_tokens, base_pos):
    import torch
    rng = np.random.default_rng(n_tokens)
    k, v = kv_values(rng, (n_tokens, hkv, d)), kv_values(rng, (n_tokens, hkv, d))
    cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, base_pos + n_tokens + 4), vf.KvDtype[dtype])
    fwd = vf.CudaForward(ctx, cache, n_heads=hkv)
    try:
        k_rot = torch.zeros(n_tokens, hkv, d, device="cuda")
        fwd.rope_kv_write(0, to_dev(k), to_dev(v), n_tokens, base_pos, k_rot=k_rot, n_dims=n_dims, freq_base=500000.0)
        torch.cuda.synchronize()
        got_rot = k_rot.cpu().numpy()
        want_rot = oracle.rope_neox_rows(k, hkv, d, n_dims, range(base_pos, base_pos + n_tokens), 500000.0)
        # same angles bit for bit; sin / cos differ from the host's by an ulp or two
        assert float(np.max(np.abs(got_rot - want_rot))) < 2e-5 * max(1.0, float(np.abs(k).max()))
        if n_dims < d:
            assert np.array_equal(got_rot[..., n_dims:], k[..., n_dims:])
        # the cache holds exactly the encoding of the rotated rows the kernel reports, and of V
        es = {"F32": 4, "F16": 2, "F8": 1}[dtype]
        row = hkv * d * es
        kb = dev_view_bytes(cache.k_buffer + base_pos * row, n_tokens * row)
        vb = dev_view_bytes(cache.v_buffer + base_pos * row, n_tokens * row)
        assert np.array_equal(kb, oracle.store(got_rot, ODT[dtype]).view(np.uint8).ravel())
        assert np.array_equal(vb, oracle.store(v, ODT[dtype]).view(np.uint8).ravel())
        # without the f32 copy the bytes are the same
        if (n_dims // 2) % 16 == 0:
            cache.zero_fill()
            fwd.rope_kv_write(0, to_dev(k), to_dev(v), n_tokens, base_pos, n_dims=n_dims, freq_base=500000.0)
            torch.cuda.synchronize()
            assert np.array_equal(dev_view_bytes(cache.k_buffer + base_pos * row, n_tokens * row), kb)
        else:
            with pytest.raises(vf.VfkvError):
                fwd.rope_kv_write(0, to_dev(k), to_dev(v), n_tokens, base_pos, n_dims=n_dims, freq_base=500000.0)
    finally:
        fwd.workspace.destroy()
        cache.destroy()


def test_rope_append_batch_and_q_rotation(ctx):
    import torch
    hq, hkv, d, n = 32, 8, 128, 5
    rng = np.random.default_rng(8)
    k, v = kv_values(rng, (n, hkv, d)), kv_values(rng, (n, hkv, d))
    q = rng.standard_normal((n, hq, d), dtype=np.float32)
    positions = np.array([0, 100, 7, 4095, 33], np.uint32)
    slots = np.array([4, 0, 2, 1, 3], np.uint32)
    cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, 4096, n_slots=5), vf.KvDtype.F8)
    fwd = vf.CudaForward(ctx, cache, n_heads=hq)
    try:
        k_rot = torch.zeros(n, hkv, d, device="cuda")
        fwd.rope_kv_write_batch(0, to_dev(k), to_dev(v), to_dev(slots), to_dev(positions), n, k_rot=k_rot,
                                freq_base=500000.0)
        dq = to_dev(q)
        fwd.run_rope_neox(dq, dq, n, hq, d, positions=to_dev(positions), freq_base=500000.0)   # in place
        torch.cuda.synchronize()
        want_k = oracle.rope_neox_rows(k, hkv, d, d, positions, 500000.0)
        want_q = oracle.rope_neox_rows(q, hq, d, d, positions, 500000.0)
        assert float(np.max(np.abs(k_rot.cpu().numpy() - want_k))) < 5e-4
        assert float(np.max(np.abs(dq.cpu().numpy() - want_q))) < 5e-5
        row = hkv * d
        for i in range(n):
            kb = dev_view_bytes(cache.k_buffer + cache.slot_offset_bytes(0, int(slots[i])) + int(positions[i]) * row, row)
            assert np.array_equal(kb, oracle.store(k_rot[i].cpu().numpy(), oracle.F8).view(np.uint8).ravel())
    finally:
        fwd.workspace.destroy()
        cache.destroy()


# ---- prefix reuse (src/server/state.rs:199-229,284-287; tests/kv_reuse_ident.rs) --------------------
def test_kv_reuse_prepare_and_invalidate(ctx):
    cache = vf.KvCache(ctx, vf.KvCacheConfig(1, 2, 64, 64, n_slots=2), vf.KvDtype.F8)
    try:
        cache.set_seq_len(0, 5)
        assert cache.reuse_prepare([1, 2, 3, 4, 5], [1, 2, 3, 9]) == 3 and cache.seq_len(0) == 3
        # identical prompt: one token is always left to prefill
        assert cache.reuse_prepare([1, 2, 3, 4, 5], [1, 2, 3, 4, 5]) == 4 and cache.seq_len(0) == 4
        # the new prompt is a prefix of the cached sequence
        assert cache.reuse_prepare([1, 2, 3, 4, 5], [1, 2]) == 1 and cache.seq_len(0) == 1
        # nothing in common, or reuse switched off: reset
        cache.set_seq_len(0, 5)
        assert cache.reuse_prepare([1, 2, 3], [7, 8]) == 0 and cache.seq_len(0) == 0
        cache.set_seq_len(0, 5)
        assert cache.reuse_prepare([1, 2, 3], [1, 2, 3, 4], reuse=False) == 0 and cache.seq_len(0) == 0
        # slots are independent
        cache.set_seq_len(1, 9)
        assert cache.reuse_prepare([5, 6, 7], [5, 6, 1], slot=1) == 2 and cache.seq_len(1) == 2 and cache.seq_len(0) == 0
        cache.invalidate(1)
        assert cache.seq_len(1) == 0
    finally:
        cache.destroy()


def test_kv_reuse_is_byte_identical_and_an_overshoot_is_caught(ctx, monkeypatch):
    """tests/kv_reuse_ident.rs:224-320 at cache level.  Reusing the longest common prefix and
    prefilling the rest leaves exactly the bytes of a fresh prefill; with the reference's teeth hook
    VF_KV_REUSE_OVERSHOOT the reuse keeps rows of the OLD prompt past the common prefix, and both
    the cache bytes and the attention output differ from the fresh ones."""
    import torch
    hq, hkv, d, max_seq, vocab = 8, 2, 64, 128, 50
    rng = np.random.default_rng(8)
    table_k = kv_values(rng, (vocab, hkv, d))                 # a token's K and V rows depend on the token only
    table_v = kv_values(rng, (vocab, hkv, d))
    old = [int(x) for x in rng.integers(0, vocab, 60)]
    new = old[:37] + [int(x) for x in (rng.integers(0, vocab, 30) + 1) % vocab]
    new[37] = (old[37] + 1) % vocab                           # the prompts part ways at position 37
    q = rng.standard_normal((hq, d), dtype=np.float32)

    def prefill(fwd, tokens, base):
        if len(tokens) > base:
            ids = np.array(tokens[base:])
            fwd.b_step_kv_write(0, to_dev(table_k[ids]), to_dev(table_v[ids]), len(ids), base, 0)

    def run(overshoot):
        if overshoot:
            monkeypatch.setenv("VF_KV_REUSE_OVERSHOOT", str(overshoot))
        else:
            monkeypatch.delenv("VF_KV_REUSE_OVERSHOOT", raising=False)
        cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, max_seq), vf.KvDtype.F8)
        fwd = vf.CudaForward(ctx, cache, n_heads=hq)
        try:
            prefill(fwd, old, 0)
            cache.set_seq_len(0, len(old))
            k = cache.reuse_prepare(old, new)
            prefill(fwd, new, k)
            out = torch.zeros(hq, d, device="cuda")
            fwd.step_attention(0, to_dev(q), out, len(new) - 1)
            torch.cuda.synchronize()
            nb = len(new) * cache.row_bytes(0)
            return k, dev_view_bytes(cache.k_buffer, nb), out.cpu().numpy()
        finally:
            fwd.workspace.destroy()
            cache.destroy()

    fresh = oracle.kv_store_fp8(table_k[np.array(new)])
    k, kb, out = run(0)
    assert k == 37 and np.array_equal(kb, fresh)
    want = oracle.attention_ref(q, fresh, oracle.kv_store_fp8(table_v[np.array(new)]), oracle.F8, hq, hkv, d, len(new))
    assert rel_err(out, want) < 1e-4
    k2, kb2, out2 = run(5)
    assert k2 == 42
    assert not np.array_equal(kb2, fresh)                     # rows 37..41 still hold the old prompt
    assert np.array_equal(kb2[:37 * hkv * d], fresh[:37 * hkv * d]) and np.array_equal(kb2[42 * hkv * d:], fresh[42 * hkv * d:])
    assert rel_err(out2, want) > 1e-3                         # and the output shows it
    k3, _, _ = run(10 ** 6)                                   # bounded by the resident rows and the new prompt
    assert k3 == min(len(old), len(new) - 1)
