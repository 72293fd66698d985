"""KV append and FP8->F16 read on the GPU, through the C ABI, against the CPU oracle.
Cache bytes must be bit-exact (FP8, F32) or equal to round-to-nearest-even (F16)."""
import numpy as np
import pytest

import oracle
import vulkanforge_b200 as vf
from util import dev_view_bytes, dev_write_bytes, kv_values, to_dev

pytestmark = pytest.mark.gpu


def _raw_store(ctx, kind, x, n, offset, dst_bytes):
    import torch
    L = ctx._lib
    src = to_dev(x)
    dst = torch.full((dst_bytes,), 0xAB, dtype=torch.uint8, device="cuda")
    fn = L.vfkv_kv_store_fp8 if kind == "fp8" else L.vfkv_kv_copy_fp16
    ctx.check(fn(ctx.handle, src.data_ptr(), dst.data_ptr(), n, offset, None))
    torch.cuda.synchronize()
    return dst.cpu().numpy()


@pytest.mark.parametrize("n,offset", [(1024, 0), (1024, 4096), (1, 4), (3, 8), (5, 0), (1021, 12), (4096, 16),
                                      (17, 20), (524288, 1024)])
def test_kv_store_fp8_bit_exact(ctx, n, offset):
    # vk_shaders/kv_store_fp8.comp + runs.rs:2437-2478
    rng = np.random.default_rng(n + offset)
    x = kv_values(rng, n)
    want = oracle.kv_store_fp8(x)
    got = _raw_store(ctx, "fp8", x, n, offset, offset + want.size + 64)
    assert np.array_equal(got[offset:offset + want.size], want)
    assert np.all(got[:offset] == 0xAB) and np.all(got[offset + want.size:] == 0xAB)


@pytest.mark.parametrize("n,offset", [(1024, 0), (2048, 4096), (1, 4), (3, 8), (1023, 12), (9, 20), (262144, 64)])
def test_kv_copy_fp16_rne(ctx, n, offset):
    # vk_shaders/kv_copy_fp16.comp + runs.rs:2389-2430
    rng = np.random.default_rng(n + offset)
    x = kv_values(rng, n)
    want = oracle.kv_copy_fp16(x).view(np.uint8)
    got = _raw_store(ctx, "f16", x, n, offset, offset + want.size + 64)
    assert np.array_equal(got[offset:offset + want.size], want)
    assert np.all(got[:offset] == 0xAB) and np.all(got[offset + want.size:] == 0xAB)


def test_misaligned_offset_is_rejected(ctx):
    import torch
    # runs.rs:2448-2452 (debug_assert on uint alignment) becomes an error status
    src = torch.zeros(16, device="cuda")
    dst = torch.zeros(64, dtype=torch.uint8, device="cuda")
    rc = ctx._lib.vfkv_kv_store_fp8(ctx.handle, src.data_ptr(), dst.data_ptr(), 4, 2, None)
    assert rc == vf.kv_cache.ERR_INVALID


def test_fp8_converter_exhaustive_all_f32(ctx):
    """Every one of the 2^32 float bit patterns converts to the oracle's code."""
    import torch
    L = ctx._lib
    chunk = 1 << 26
    dst = torch.empty(chunk, dtype=torch.uint8, device="cuda")
    base = torch.arange(chunk, dtype=torch.int64, device="cuda")
    bad = 0
    for c in range((1 << 32) // chunk):
        first = c * chunk
        bits = (base + first)
        bits = torch.where(bits >= (1 << 31), bits - (1 << 32), bits).to(torch.int32)
        src = bits.view(torch.float32)
        ctx.check(L.vfkv_kv_store_fp8(ctx.handle, src.data_ptr(), dst.data_ptr(), chunk, 0, None))
        got = dst.cpu().numpy()
        want = oracle.e4m3_range(first, chunk)
        if not np.array_equal(got, want):
            idx = np.nonzero(got != want)[0]
            bad += idx.size
            print(f"chunk {c}: {idx.size} mismatches, first bits={first + int(idx[0]):#x} "
                  f"gpu={got[idx[0]]:#x} oracle={want[idx[0]]:#x}")
    assert bad == 0


def test_f16_converter_sweep(ctx):
    """Sampled sweep (every 64th bit pattern); NaNs compare as NaN (payload is not pinned anywhere)."""
    import torch
    L = ctx._lib
    chunk = 1 << 26
    dst = torch.empty(chunk, dtype=torch.int16, device="cuda")
    bits = (torch.arange(chunk, dtype=torch.int64, device="cuda") * 64 + 17)
    bits = torch.where(bits >= (1 << 31), bits - (1 << 32), bits).to(torch.int32)
    ctx.check(L.vfkv_kv_copy_fp16(ctx.handle, bits.view(torch.float32).data_ptr(), dst.data_ptr(), chunk, 0, None))
    got = dst.cpu().numpy().view(np.uint16)
    x = bits.cpu().numpy().view(np.float32)
    want = oracle.kv_copy_fp16(x)
    nan = np.isnan(x)
    assert np.array_equal(got[~nan], want[~nan])
    assert np.all((got[nan] & 0x7C00) == 0x7C00) and np.all((got[nan] & 0x3FF) != 0)


def test_kv_fp8_to_f16_all_codes_and_bulk(ctx):
    # vk_shaders/kv_fp8_to_f16.comp; examples/fp8_smoke.rs:371-397 checks all 256 codes
    import torch
    L = ctx._lib
    rng = np.random.default_rng(1)
    for n in (256, 1, 15, 1000003):
        codes = np.arange(n, dtype=np.uint64).astype(np.uint8) if n == 256 else rng.integers(0, 256, n, dtype=np.uint8)
        src = to_dev(codes)
        dst = torch.full((n + 8,), 0x1234, dtype=torch.int16, device="cuda")
        ctx.check(L.vfkv_kv_fp8_to_f16(ctx.handle, src.data_ptr(), dst.data_ptr(), n, None))
        got = dst.cpu().numpy().view(np.uint16)
        want = oracle.kv_fp8_to_f16(codes)
        nan = (codes & 0x7F) == 0x7F
        assert np.array_equal(got[:n][~nan], want[~nan])
        assert np.all((got[:n][nan] & 0x7C00) == 0x7C00) and np.all((got[:n][nan] & 0x3FF) != 0)
        assert np.all(got[n:] == 0x1234)


def _expected_buffer(cache, fill):
    return np.full(cache.bytes_per_buffer(), fill, np.uint8)


@pytest.mark.parametrize("dtype", [vf.KvDtype.F8, vf.KvDtype.F16, vf.KvDtype.F32])
def test_cache_append_layout_and_bytes(ctx, dtype):
    """Rows land at [layer][slot][pos] offsets, nothing else is touched
    (kv_cache.rs:431-490; executor/attention.rs:546-596,2134-2190)."""
    cfg = vf.KvCacheConfig(n_layers=3, n_kv_heads=8, head_dim=128, max_seq_len=96, n_slots=4)
    cache = vf.KvCache(ctx, cfg, dtype)
    try:
        es = dtype.element_size()
        assert cache.row_bytes(1) == 8 * 128 * es
        assert cache.layer_size_bytes(1) == 96 * 8 * 128 * es
        assert cache.layer_offset_bytes(2) == 2 * 4 * 96 * 8 * 128 * es
        assert cache.bytes_per_buffer() == 3 * 4 * 96 * 8 * 128 * es
        nbytes = cache.bytes_per_buffer()
        ctx.check(ctx._lib.vfkv_memset(ctx.handle, cache.k_buffer, 0xAB, nbytes, None))
        ctx.check(ctx._lib.vfkv_memset(ctx.handle, cache.v_buffer, 0xCD, nbytes, None))
        rng = np.random.default_rng(int(dtype))
        fwd = vf.CudaForward(ctx, cache, n_heads=32)
        want_k, want_v = _expected_buffer(cache, 0xAB), _expected_buffer(cache, 0xCD)
        # a 37-token prefill chunk into layer 1 / slot 2 at base_pos 11, then single tokens elsewhere
        writes = [(1, 2, 11, 37), (0, 0, 0, 1), (2, 3, 95, 1), (1, 2, 48, 1), (1, 0, 5, 3)]
        for layer, slot, base, n in writes:
            k = kv_values(rng, (n, 8, 128))
            v = kv_values(rng, (n, 8, 128))
            fwd.b_step_kv_write(layer, to_dev(k), to_dev(v), n, base, slot)
            off = cache.slot_offset_bytes(layer, slot) + base * cache.row_bytes(layer)
            kb = oracle.store(k, int(dtype)).view(np.uint8)
            vb = oracle.store(v, int(dtype)).view(np.uint8)
            want_k[off:off + kb.size] = kb
            want_v[off:off + vb.size] = vb
        assert np.array_equal(dev_view_bytes(cache.k_buffer, nbytes), want_k)
        assert np.array_equal(dev_view_bytes(cache.v_buffer, nbytes), want_v)
        fwd.workspace.destroy()
    finally:
        cache.destroy()


def test_append_batch_and_stale_overwrite(ctx):
    """One token per sequence at device-side positions; appending over stale rows gives the same
    bytes as a fresh append (the cache-level form of tests/kv_reuse_ident.rs:224-320)."""
    import torch
    cfg = vf.KvCacheConfig(n_layers=2, n_kv_heads=8, head_dim=128, max_seq_len=64, n_slots=8)
    rng = np.random.default_rng(77)
    k = kv_values(rng, (5, 8, 128))
    v = kv_values(rng, (5, 8, 128))
    slots = np.array([7, 0, 3, 4, 1], np.uint32)
    pos = np.array([63, 0, 10, 10, 33], np.uint32)
    images = []
    for stale in (False, True):
        cache = vf.KvCache(ctx, cfg, vf.KvDtype.F8)
        fwd = vf.CudaForward(ctx, cache, n_heads=32)
        cache.zero_fill()
        if stale:   # an earlier request left other tokens in exactly those rows
            junk = kv_values(rng, (5, 8, 128)) * 3
            fwd.step_kv_write_batch(1, to_dev(junk), to_dev(junk), to_dev(slots), to_dev(pos), 5)
        fwd.step_kv_write_batch(1, to_dev(k), to_dev(v), to_dev(slots), to_dev(pos), 5)
        images.append((dev_view_bytes(cache.k_buffer, cache.bytes_per_buffer()),
                       dev_view_bytes(cache.v_buffer, cache.bytes_per_buffer())))
        if not stale:
            want = np.zeros(cache.bytes_per_buffer(), np.uint8)
            for i in range(5):
                off = cache.slot_offset_bytes(1, int(slots[i])) + int(pos[i]) * cache.row_bytes(1)
                want[off:off + 1024] = oracle.kv_store_fp8(k[i])
            assert np.array_equal(images[0][0], want)
        # reset() only zeroes the counter; bytes persist (kv_cache.rs:492-494)
        cache.set_seq_len(3, 11)
        cache.reset(3)
        assert cache.seq_len(3) == 0
        fwd.workspace.destroy()
        cache.destroy()
    assert np.array_equal(images[0][0], images[1][0]) and np.array_equal(images[0][1], images[1][1])


def test_append_rejects_context_overflow(ctx):
    # src/backend/vulkan/decode.rs:523-533: prefill + new tokens must fit max_seq
    import torch
    cfg = vf.KvCacheConfig(n_layers=1, n_kv_heads=8, head_dim=128, max_seq_len=16)
    cache = vf.KvCache(ctx, cfg, vf.KvDtype.F16)
    try:
        x = torch.zeros(4 * 1024, device="cuda")
        L = ctx._lib
        assert L.vfkv_append(cache.handle, 0, x.data_ptr(), x.data_ptr(), 4, 0, 13, None) == vf.kv_cache.ERR_INVALID
        assert b"max_seq_len" in L.vfkv_last_error(ctx.handle)
        assert L.vfkv_append(cache.handle, 1, x.data_ptr(), x.data_ptr(), 1, 0, 0, None) == vf.kv_cache.ERR_INVALID
        assert L.vfkv_append(cache.handle, 0, x.data_ptr(), x.data_ptr(), 1, 1, 0, None) == vf.kv_cache.ERR_INVALID
        assert L.vfkv_append(cache.handle, 0, x.data_ptr(), x.data_ptr(), 4, 0, 12, None) == 0
    finally:
        cache.destroy()


def test_append_batch_out_of_range_row_is_skipped_and_reported(ctx, request):
    request.node.expects_status = True
    cfg = vf.KvCacheConfig(n_layers=1, n_kv_heads=8, head_dim=128, max_seq_len=16, n_slots=2)
    cache = vf.KvCache(ctx, cfg, vf.KvDtype.F8)
    fwd = vf.CudaForward(ctx, cache, n_heads=32)
    try:
        cache.zero_fill()
        k = np.ones((2, 8, 128), np.float32)
        fwd.step_kv_write_batch(0, to_dev(k), to_dev(k), to_dev(np.array([0, 1], np.uint32)),
                                to_dev(np.array([3, 16], np.uint32)), 2)
        with pytest.raises(vf.VfkvError) as e:
            ctx.poll()
        assert e.value.status == vf.kv_cache.ERR_TIMEOUT
        img = dev_view_bytes(cache.k_buffer, cache.bytes_per_buffer())
        assert np.all(img[3 * 1024:4 * 1024] == 0x38) and img.sum() == 0x38 * 1024
        ctx.poll()   # cleared by the previous poll
    finally:
        fwd.workspace.destroy()
        cache.destroy()


def test_scaled_append_matches_oracle(ctx):
    cfg = vf.KvCacheConfig(n_layers=2, n_kv_heads=8, head_dim=128, max_seq_len=32, n_slots=2, scale_mode=1)
    cache = vf.KvCache(ctx, cfg, vf.KvDtype.F8)
    fwd = vf.CudaForward(ctx, cache, n_heads=32)
    try:
        cache.zero_fill()
        rng = np.random.default_rng(5)
        k = kv_values(rng, (6, 8, 128)) * 40
        v = kv_values(rng, (6, 8, 128)) * 0.01
        k[2, 3] = 0.0
        fwd.b_step_kv_write(1, to_dev(k), to_dev(v), 6, 9, 1)
        kb = dev_view_bytes(cache.k_buffer, cache.bytes_per_buffer())
        vb = dev_view_bytes(cache.v_buffer, cache.bytes_per_buffer())
        n_scales = 2 * 2 * 32 * 8
        ks = dev_view_bytes(cache.k_scales, n_scales * 4).view(np.float32)
        vs = dev_view_bytes(cache.v_scales, n_scales * 4).view(np.float32)
        for t in range(6):
            off = cache.slot_offset_bytes(1, 1) + (9 + t) * 1024
            soff = ((1 * 2 + 1) * 32 + 9 + t) * 8
            ck, sk = oracle.kv_store_fp8_scaled(k[t], 8, 128)
            cv, sv = oracle.kv_store_fp8_scaled(v[t], 8, 128)
            assert np.array_equal(kb[off:off + 1024], ck) and np.array_equal(vb[off:off + 1024], cv)
            assert np.array_equal(ks[soff:soff + 8], sk) and np.array_equal(vs[soff:soff + 8], sv)
    finally:
        fwd.workspace.destroy()
        cache.destroy()


def test_cache_create_errors_and_heterogeneous_layout(ctx):
    L = ctx._lib
    with pytest.raises(vf.VfkvError) as e:
        vf.KvCache(ctx, vf.KvCacheConfig(2**31, 2**31, 2**31, 2**31), vf.KvDtype.F32)
    assert e.value.status == vf.kv_cache.ERR_OVERFLOW          # kv_cache.rs:273-291 checked_mul
    with pytest.raises(vf.VfkvError):
        vf.KvCache(ctx, vf.KvCacheConfig(2, 8, 128, 16, per_layer_head_dim=[128]), vf.KvDtype.F16)
    with pytest.raises(vf.VfkvError):
        vf.KvCache(ctx, vf.KvCacheConfig(2, 8, 128, 16, scale_mode=1), vf.KvDtype.F16)
    cache = vf.KvCache(ctx, vf.KvCacheConfig(4, 999, 999, 100, per_layer_head_dim=[256, 256, 512, 512],
                                             per_layer_n_kv_heads=[2, 2, 4, 4]), vf.KvDtype.F16)
    try:
        lay = oracle.make_layout(4, 999, 999, 100, oracle.F16, [256, 256, 512, 512], [2, 2, 4, 4])
        O = oracle.lib()
        for i in range(4):
            assert cache.head_dim_for(i) == O.vfo_head_dim_for(lay, i)
            assert cache.kv_heads_for(i) == O.vfo_kv_heads_for(lay, i)
            assert cache.row_bytes(i) == O.vfo_row_bytes(lay, i)
            assert cache.layer_size_bytes(i) == O.vfo_layer_size_bytes(lay, i)
            assert cache.layer_offset_bytes(i) == O.vfo_layer_offset_bytes(lay, i)
            assert cache.layer_offset_elems(i) == O.vfo_layer_offset_bytes(lay, i) // 2
            assert cache.pos_offset_bytes(i, 7) == O.vfo_pos_offset_bytes(lay, i, 7)
        assert cache.bytes_per_buffer() == oracle.bytes_per_buffer(lay)
        assert cache.is_fp16() and not cache.is_fp8()
        # zero_layer touches exactly one layer (kv_cache.rs:384-407)
        n = cache.bytes_per_buffer()
        ctx.check(L.vfkv_memset(ctx.handle, cache.k_buffer, 0xEE, n, None))
        cache.zero_layer(2)
        img = dev_view_bytes(cache.k_buffer, n)
        a, b = cache.layer_offset_bytes(2), cache.layer_offset_bytes(3)
        assert not img[a:b].any() and np.all(img[:a] == 0xEE) and np.all(img[b:] == 0xEE)
    finally:
        cache.destroy()
