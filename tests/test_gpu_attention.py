"""Split-K GQA decode attention on the GPU, through the C ABI, against the CPU oracle
(the restatement of the reference's cpu_attention_reference, tests/correctness.rs:2567-2617).

Two gates per comparison.  Acceptance gate: F32 / F16 cache max-abs error below 1e-3 (the
reference's own threshold for split+reduce, tests/correctness.rs:2875-2894; the stated limit is
2e-3), FP8 cache error relative to the output's max below 3e-2 against the oracle reading the same
E4M3 bytes (the reference's class for half-precision operands is 2e-3 / 2e-2,
tests/coopmat_fa_gemma.rs:260,330).  Regression gate: what the kernels deliver by design -- f32
accumulation, and on the tensor cores Q and P carried as a high plus a low half-precision term --
is f32-grade, so F32 / F16 results must stay within 2e-5 and FP8 results within 1e-4 relative; a
change that dropped the low terms (operand rounding 2^-11) fails it.  The one path that feeds
single half-precision operands (F16 cache, more than 8 q-heads per kv-head on the tensor cores)
is held to the acceptance gate only."""
import os

import numpy as np
import pytest

import oracle
import vulkanforge_b200 as vf
from util import (GOLDEN_CASES, correctness_rs_inputs, dev_write_bytes, encode_cache, golden_inputs,
                  kv_values, rel_err, to_dev)

pytestmark = pytest.mark.gpu

ABS_TOL = 1e-3
FP8_REL_TOL = 3e-2
REGRESSION_ABS_TOL = 2e-5
REGRESSION_FP8_REL_TOL = 1e-4


def single_term_path(impl, dtype, hq, hkv, d):
    """True where the tensor-core kernel runs without the high + low operand split."""
    return impl != 1 and int(dtype) == oracle.F16 and hq // hkv > 8 and d in (64, 128, 256)


def check(got, want, dtype, single_term=False, relative=False):
    """relative: the absolute gates are meant for outputs of order one; where tens of thousands of
    positions with outliers give outputs of order 30, the error is taken relative to the largest
    output (f32 accumulation alone is 1e-6 of it there, on the CUDA cores as on the tensor cores)."""
    assert np.isfinite(got).all()
    if int(dtype) == oracle.F8:
        err = rel_err(got, want)
        assert err < FP8_REL_TOL, err
        assert single_term or err < REGRESSION_FP8_REL_TOL, ("regression gate", err)
    else:
        err = float(np.max(np.abs(got - want)))
        if relative:
            err /= max(1.0, float(np.max(np.abs(want))))
        assert err < ABS_TOL, err
        assert single_term or err < REGRESSION_ABS_TOL, ("regression gate", err)


class Rig:
    """A cache with caller-chosen contents (written as raw bytes so attention is tested
    independently of append) plus the forward-side wrapper."""

    def __init__(self, ctx, dtype, hq, hkv, d, max_seq, n_layers=1, n_slots=1, scale_mode=0, **fw):
        self.ctx, self.dtype, self.hq, self.hkv, self.d = ctx, vf.KvDtype(dtype), hq, hkv, d
        self.cache = vf.KvCache(ctx, vf.KvCacheConfig(n_layers, hkv, d, max_seq, n_slots=n_slots,
                                                      scale_mode=scale_mode), self.dtype)
        self.fwd = vf.CudaForward(ctx, self.cache, n_heads=hq, max_batch=max(n_slots, 1), **fw)

    def put(self, layer, slot, k_cache, v_cache, pos0=0):
        off = self.cache.slot_offset_bytes(layer, slot) + pos0 * self.cache.row_bytes(layer)
        dev_write_bytes(self.cache.k_buffer + off, k_cache.view(np.uint8).ravel())
        dev_write_bytes(self.cache.v_buffer + off, v_cache.view(np.uint8).ravel())

    def attend(self, q, layer, seq_len, kv_start=0, n_splits=0, slot=0, kv_layer=None):
        import torch
        out = torch.full((self.hq, self.d), float("nan"), device="cuda")
        self.fwd.run_flash_attn_split_reduce(to_dev(q), out, layer, seq_len - 1, n_splits,
                                             layer if kv_layer is None else kv_layer, kv_start, slot)
        torch.cuda.synchronize()
        return out.cpu().numpy()

    def close(self):
        self.fwd.workspace.destroy()
        self.cache.destroy()


@pytest.fixture(params=[1, 0], ids=["cuda-core", "auto"])
def impl(request, ctx):
    ctx.set_attn_impl(request.param)
    yield request.param
    ctx.set_attn_impl(0)


@pytest.mark.parametrize("seq_len", [64, 200, 2048])
@pytest.mark.parametrize("n_splits", [0, 1, 4, 32])
def test_reference_split_attn_cases(ctx, impl, seq_len, n_splits):
    """tests/correctness.rs:2791-2894: 32 q / 8 kv / 128, F32 cache, deterministic inputs, < 1e-3."""
    hq, hkv, d = 32, 8, 128
    q, k, v = correctness_rs_inputs(hq, hkv, d, seq_len)
    rig = Rig(ctx, vf.KvDtype.F32, hq, hkv, d, 2048)
    try:
        rig.put(0, 0, k, v)
        got = rig.attend(q, 0, seq_len, n_splits=n_splits)
        check(got, oracle.attention_ref(q, k, v, oracle.F32, hq, hkv, d, seq_len), oracle.F32)
    finally:
        rig.close()


def test_raw_pointer_entry_matches(ctx, impl):
    """vfkv_flash_attn_split_reduce on caller buffers (the Fixture::dispatch level of the reference)."""
    import torch
    hq, hkv, d, L = 32, 8, 128, 200
    q, k, v = correctness_rs_inputs(hq, hkv, d, L)
    ws = vf.Workspace(ctx, 1, hq, d, 16)
    try:
        out = torch.zeros(hq, d, device="cuda")
        dq, dk, dv = to_dev(q), to_dev(k), to_dev(v)     # keep the tensors alive across the call
        ctx.check(ctx._lib.vfkv_flash_attn_split_reduce(
            ctx.handle, ws.handle, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
            out.data_ptr(), oracle.F32, hq, hkv, d, L, L, 1.0 / np.sqrt(d), 0, 0.0, 4, None))
        torch.cuda.synchronize()
        check(out.cpu().numpy(), oracle.attention_ref(q, k, v, oracle.F32, hq, hkv, d, L), oracle.F32)
    finally:
        ws.destroy()


@pytest.mark.parametrize("dtype", [vf.KvDtype.F32, vf.KvDtype.F16, vf.KvDtype.F8])
def test_seq1_output_equals_v_and_layer_offset(ctx, impl, dtype):
    """tests/correctness.rs:899-1035: seq_len 1 => out == V; slab bound at a non-zero layer
    offset while layer 0 holds garbage."""
    hq, hkv, d, max_seq = 32, 8, 128, 2048
    rig = Rig(ctx, dtype, hq, hkv, d, max_seq, n_layers=2)
    try:
        garbage = np.full((max_seq, hkv, d), 999.0, np.float32)
        rig.put(0, 0, encode_cache(garbage, int(dtype)), encode_cache(garbage, int(dtype)))
        rig.put(1, 0, encode_cache(np.full((max_seq, hkv, d), 0.1, np.float32), int(dtype)),
                encode_cache(np.full((max_seq, hkv, d), 1.0, np.float32), int(dtype)))
        q = np.full((hq, d), 0.1, np.float32)
        for L in (1, 2, 65):
            got = rig.attend(q, 1, L)
            assert np.max(np.abs(got - 1.0)) < 1e-5
    finally:
        rig.close()


def test_golden_fixture_cases(ctx, impl):
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "attention_small.npz"))
    for i, (name, hq, hkv, d, L, start, dt, cap) in enumerate(GOLDEN_CASES):
        q, kc, vc = golden_inputs(i)
        rig = Rig(ctx, dt, hq, hkv, d, L + 3, softcap=cap)
        try:
            rig.put(0, 0, kc, vc)
            for n_splits in (0, 3):
                got = rig.attend(q, 0, L, kv_start=start, n_splits=n_splits)
                check(got, gold[name + "/out"], dt)
        finally:
            rig.close()


SHAPES = [  # hq, hkv, d
    (32, 8, 128), (64, 8, 128), (16, 8, 256), (8, 8, 64), (8, 1, 128), (40, 8, 128), (16, 2, 512), (4, 2, 64),
    (32, 2, 128), (24, 2, 256), (12, 1, 64)]


@pytest.mark.parametrize("dtype", [vf.KvDtype.F32, vf.KvDtype.F16, vf.KvDtype.F8])
@pytest.mark.parametrize("hq,hkv,d", SHAPES)
def test_shapes_lengths_and_starts(ctx, impl, dtype, hq, hkv, d):
    rng = np.random.default_rng(hq * 1000 + d + int(dtype))
    max_seq = 1200
    fp8 = dtype == vf.KvDtype.F8
    k = kv_values(rng, (max_seq, hkv, d), outlier_frac=0.01 if fp8 else 0.0)
    v = kv_values(rng, (max_seq, hkv, d), outlier_frac=0.01 if fp8 else 0.0)
    kc, vc = encode_cache(k, int(dtype)), encode_cache(v, int(dtype))
    q = rng.standard_normal((hq, d), dtype=np.float32)
    rig = Rig(ctx, dtype, hq, hkv, d, max_seq)
    try:
        rig.put(0, 0, kc, vc)
        for L, start, n_splits in [(1, 0, 0), (31, 0, 1), (64, 0, 2), (65, 0, 0), (129, 128, 0), (640, 0, 5),
                                   (1200, 0, 0), (1200, 1200 - 1024, 0), (1111, 17, 7), (1000, 999, 3),
                                   (257, 3, 64)]:
            got = rig.attend(q, 0, L, kv_start=start, n_splits=n_splits)
            want = oracle.attention_ref(q, kc, vc, int(dtype), hq, hkv, d, L, start)
            check(got, want, dtype, single_term_path(impl, dtype, hq, hkv, d))
    finally:
        rig.close()


def test_stale_nan_rows_beyond_seq_len_do_not_leak(ctx, impl):
    """Rows at and beyond seq_len (and below kv_start) may hold anything, including NaN codes."""
    for dtype in (vf.KvDtype.F8, vf.KvDtype.F16, vf.KvDtype.F32):
        hq, hkv, d, max_seq, L, start = 32, 8, 128, 512, 300, 40
        rng = np.random.default_rng(3)
        k = rng.standard_normal((max_seq, hkv, d), dtype=np.float32)
        v = rng.standard_normal((max_seq, hkv, d), dtype=np.float32)
        kc, vc = encode_cache(k, int(dtype)), encode_cache(v, int(dtype))
        nan_code = {vf.KvDtype.F8: 0x7F, vf.KvDtype.F16: 0x7E00, vf.KvDtype.F32: 0x7FC00000}[dtype]
        for arr in (kc, vc):
            a = arr.view({1: np.uint8, 2: np.uint16, 4: np.uint32}[arr.itemsize])
            a[L:] = nan_code
            a[:start] = nan_code
        q = rng.standard_normal((hq, d), dtype=np.float32)
        rig = Rig(ctx, dtype, hq, hkv, d, max_seq)
        try:
            rig.put(0, 0, kc, vc)
            for n_splits in (0, 1, 6):
                got = rig.attend(q, 0, L, kv_start=start, n_splits=n_splits)
                check(got, oracle.attention_ref(q, kc, vc, int(dtype), hq, hkv, d, L, start), dtype)
        finally:
            rig.close()


@pytest.mark.parametrize("dtype", [vf.KvDtype.F16, vf.KvDtype.F8])
def test_batch_variable_lengths_slots_and_windows(ctx, impl, dtype):
    """Independent sequences in their own slots, ragged lengths, permuted slot ids, per-sequence
    window starts; then the fused decode step (append + attend) for the same batch."""
    import torch
    hq, hkv, d, max_seq, n_slots = 32, 8, 128, 700, 6
    rng = np.random.default_rng(21)
    lens = np.array([1, 64, 65, 700, 333, 512], np.uint32)
    starts = np.array([0, 0, 1, 700 - 256, 0, 500], np.uint32)
    slots = np.array([4, 0, 5, 1, 3, 2], np.uint32)
    fp8 = dtype == vf.KvDtype.F8
    k = kv_values(rng, (n_slots, max_seq, hkv, d), outlier_frac=0.01 if fp8 else 0.0)
    v = kv_values(rng, (n_slots, max_seq, hkv, d), outlier_frac=0.01 if fp8 else 0.0)
    kc, vc = encode_cache(k, int(dtype)), encode_cache(v, int(dtype))
    q = rng.standard_normal((n_slots, hq, d), dtype=np.float32)
    rig = Rig(ctx, dtype, hq, hkv, d, max_seq, n_layers=2, n_slots=n_slots)
    try:
        for s in range(n_slots):
            rig.put(1, s, kc[s], vc[s])
        out = torch.zeros(n_slots, hq, d, device="cuda")
        for hint in (0, 700):
            rig.fwd.step_attention_batch(1, to_dev(q), out, to_dev(slots), to_dev(lens), to_dev(starts),
                                         n_slots, max_seq_len_hint=hint)
            torch.cuda.synchronize()
            got = out.cpu().numpy()
            for i in range(n_slots):
                s = int(slots[i])
                want = oracle.attention_ref(q[i], kc[s], vc[s], int(dtype), hq, hkv, d, int(lens[i]), int(starts[i]))
                check(got[i], want, dtype)
        # fused step: new token at position lens-1 (overwrites that row), global attention
        kn = kv_values(rng, (n_slots, hkv, d), outlier_frac=0.0)
        vn = kv_values(rng, (n_slots, hkv, d), outlier_frac=0.0)
        pos = (lens - 1).astype(np.uint32)
        rig.fwd.decode_step(1, to_dev(q), to_dev(kn), to_dev(vn), out, to_dev(slots), to_dev(pos), n_slots)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        for i in range(n_slots):
            s = int(slots[i])
            kk, vv = kc[s].copy(), vc[s].copy()
            kk[pos[i]] = encode_cache(kn[i], int(dtype))
            vv[pos[i]] = encode_cache(vn[i], int(dtype))
            check(got[i], oracle.attention_ref(q[i], kk, vv, int(dtype), hq, hkv, d, int(lens[i])), dtype)
    finally:
        rig.close()


def test_gemma_style_window_softcap_and_kv_share(ctx, impl):
    """16 q / 8 kv / 256, F16: sliding layers use kv_start = pos+1-window (gemma4.rs:59-73), a
    subscriber layer reads its publisher's slab (gemma4.rs:27-49), scores are soft-capped
    (extension) and scale is 1.0 (runs.rs:1483-1489)."""
    hq, hkv, d, max_seq, window = 16, 8, 256, 1500, 1024
    rng = np.random.default_rng(31)
    k = rng.standard_normal((max_seq, hkv, d), dtype=np.float32) * 0.3
    v = rng.standard_normal((max_seq, hkv, d), dtype=np.float32)
    kc, vc = encode_cache(k, oracle.F16), encode_cache(v, oracle.F16)
    q = rng.standard_normal((hq, d), dtype=np.float32)
    rig = Rig(ctx, vf.KvDtype.F16, hq, hkv, d, max_seq, n_layers=3, sliding_window=window,
              sliding_layers=[0, 2], kv_read_layer={2: 0}, attn_scale=1.0, softcap=50.0)
    try:
        import torch
        rig.put(0, 0, kc, vc)
        rig.put(1, 0, kc, vc)
        for layer, pos in [(0, 1499), (1, 1499), (2, 1499), (0, 500), (2, 1024)]:
            out = torch.zeros(hq, d, device="cuda")
            rig.fwd.step_attention(layer, to_dev(q), out, pos)
            torch.cuda.synchronize()
            start = vf.sliding_kv_start(pos, window) if layer in (0, 2) else 0
            want = oracle.attention_ref(q, kc, vc, oracle.F16, hq, hkv, d, pos + 1, start, 1.0, 50.0)
            check(out.cpu().numpy(), want, oracle.F16)
    finally:
        rig.close()


def test_fp8_per_token_head_scales(ctx, impl):
    """Extension: absmax-scaled E4M3 rows written by append, read back by attention."""
    import torch
    hq, hkv, d, max_seq, L = 32, 8, 128, 400, 389
    rng = np.random.default_rng(41)
    k = kv_values(rng, (L, hkv, d)) * 30
    v = kv_values(rng, (L, hkv, d)) * 0.02
    q = rng.standard_normal((hq, d), dtype=np.float32) * 0.05
    rig = Rig(ctx, vf.KvDtype.F8, hq, hkv, d, max_seq, scale_mode=1)
    try:
        rig.fwd.b_step_kv_write(0, to_dev(k), to_dev(v), L, 0)
        kc = np.zeros((L, hkv, d), np.uint8); vc = np.zeros_like(kc)
        ks = np.zeros((L, hkv), np.float32); vs = np.zeros_like(ks)
        for t in range(L):
            c, s = oracle.kv_store_fp8_scaled(k[t], hkv, d); kc[t] = c.reshape(hkv, d); ks[t] = s
            c, s = oracle.kv_store_fp8_scaled(v[t], hkv, d); vc[t] = c.reshape(hkv, d); vs[t] = s
        for n_splits in (0, 1, 5):
            got = rig.attend(q, 0, L, n_splits=n_splits)
            want = oracle.attention_ref(q, kc, vc, oracle.F8, hq, hkv, d, L, 0, None, 0.0, ks, vs)
            check(got, want, oracle.F8)
    finally:
        rig.close()


@pytest.mark.parametrize("dtype", [vf.KvDtype.F16, vf.KvDtype.F8])
def test_partials_over_position_ranges_merge_to_full(ctx, impl, dtype):
    """Sequence-dimension sharding: (m, l, o) over disjoint position ranges, merged with the
    reduce shader's update (flash_attn_reduce.comp:51-80), equals attention over the whole range."""
    import torch
    hq, hkv, d, L = 64, 8, 128, 3000
    rng = np.random.default_rng(51)
    k = rng.standard_normal((L, hkv, d), dtype=np.float32)
    v = rng.standard_normal((L, hkv, d), dtype=np.float32)
    kc, vc = encode_cache(k, int(dtype)), encode_cache(v, int(dtype))
    q = rng.standard_normal((hq, d), dtype=np.float32)
    rig = Rig(ctx, dtype, hq, hkv, d, L)
    try:
        rig.put(0, 0, kc, vc)
        bounds = [0, 700, 700, 1536, 2999, 3000]     # includes an empty range
        G = len(bounds) - 1
        m = torch.zeros(G, hq, device="cuda"); l = torch.zeros(G, hq, device="cuda")
        o = torch.zeros(G, hq, d, device="cuda")
        dq = to_dev(q)
        for g in range(G):
            rig.fwd.attend_partial(0, dq, bounds[g], bounds[g + 1], m[g], l[g], o[g])
        out = torch.zeros(hq, d, device="cuda")
        rig.fwd.merge_partials(m, l, o, G, hq, d, out)
        torch.cuda.synchronize()
        assert float(l[1].abs().max()) == 0.0 and float(m[1].max()) <= -1e29
        check(out.cpu().numpy(), oracle.attention_ref(q, kc, vc, int(dtype), hq, hkv, d, L), dtype)
    finally:
        rig.close()


def test_decode_token_host_all_layers(ctx, impl):
    """forward_token boundary with host buffers: every layer appends then attends."""
    hq, hkv, d, max_seq, n_layers, n_seqs = 32, 8, 128, 300, 3, 2
    rng = np.random.default_rng(61)
    pos = np.array([299, 130], np.uint32)
    rig = Rig(ctx, vf.KvDtype.F8, hq, hkv, d, max_seq, n_layers=n_layers, n_slots=n_seqs)
    try:
        kc = encode_cache(kv_values(rng, (n_layers, n_seqs, max_seq, hkv, d)), oracle.F8)
        vc = encode_cache(kv_values(rng, (n_layers, n_seqs, max_seq, hkv, d)), oracle.F8)
        for l in range(n_layers):
            for s in range(n_seqs):
                rig.put(l, s, kc[l, s], vc[l, s])
        q = rng.standard_normal((n_layers, n_seqs, hq, d), dtype=np.float32)
        kn = kv_values(rng, (n_layers, n_seqs, hkv, d))
        vn = kv_values(rng, (n_layers, n_seqs, hkv, d))
        out = np.zeros((n_layers, n_seqs, hq, d), np.float32)
        rig.fwd.decode_token_host(q, kn, vn, out, pos, n_seqs)
        for l in range(n_layers):
            want = oracle.decode_step(q[l], kn[l], vn[l], kc[l], vc[l], oracle.F8, n_seqs, max_seq, hq, hkv, d, pos + 1)
            check(out[l], want, oracle.F8)
    finally:
        rig.close()


@pytest.mark.parametrize("n_layers", [2, 9])
def test_decode_token_host_replays_a_graph_over_several_tokens(ctx, n_layers):
    """On a real stream the host-buffer entry point captures one token's launches once and replays
    them: successive tokens (positions advancing across a 1024 boundary, where the length hint and
    so the graphs change) must each append and attend correctly.  Nine layers form four uneven
    groups (2, 2, 2, 3) whose copies run on the workspace's second stream."""
    import torch
    hq, hkv, d, max_seq, n_seqs = 32, 8, 128, 1100, 2
    rng = np.random.default_rng(62)
    rig = Rig(ctx, vf.KvDtype.F8, hq, hkv, d, max_seq, n_layers=n_layers, n_slots=n_seqs)
    stream = torch.cuda.Stream()
    try:
        k_all = kv_values(rng, (n_layers, n_seqs, max_seq, hkv, d))
        v_all = kv_values(rng, (n_layers, n_seqs, max_seq, hkv, d))
        kc, vc = encode_cache(k_all, oracle.F8), encode_cache(v_all, oracle.F8)
        for l in range(n_layers):
            for s in range(n_seqs):
                rig.put(l, s, kc[l, s], vc[l, s])
        rig.fwd.stream = stream.cuda_stream
        n0 = ctx.launch_count()
        for step, p0 in enumerate((1020, 1021, 1022, 1023, 1024, 1025)):
            pos = np.array([p0, p0 - 500], np.uint32)
            q = rng.standard_normal((n_layers, n_seqs, hq, d), dtype=np.float32)
            kn = np.stack([np.stack([k_all[l, s, pos[s]] for s in range(n_seqs)]) for l in range(n_layers)])
            vn = np.stack([np.stack([v_all[l, s, pos[s]] for s in range(n_seqs)]) for l in range(n_layers)])
            out = np.zeros((n_layers, n_seqs, hq, d), np.float32)
            rig.fwd.decode_token_host(q, kn, vn, out, pos, n_seqs)
            for l in range(n_layers):
                want = oracle.decode_step(q[l], kn[l], vn[l], kc[l].copy(), vc[l].copy(), oracle.F8, n_seqs, max_seq,
                                          hq, hkv, d, pos + 1)
                check(out[l], want, oracle.F8)
        assert ctx.launch_count() - n0 == 6 * n_layers        # replays are counted like launches
    finally:
        rig.fwd.stream = None
        rig.close()


def test_decode_token_host_submit_and_wait_with_two_tokens_in_flight(ctx):
    """The asynchronous host-buffer step: two submits are interleaved before the first wait, a third
    one is refused while both staging sets are busy, and every token's output -- positions advance,
    so each token attends over the rows its predecessors appended -- matches the oracle."""
    import torch
    hq, hkv, d, max_seq, n_seqs, n_layers, base, steps = 32, 8, 128, 900, 2, 3, 700, 6
    rng = np.random.default_rng(63)
    rig = Rig(ctx, vf.KvDtype.F8, hq, hkv, d, max_seq, n_layers=n_layers, n_slots=n_seqs)
    stream = torch.cuda.Stream()
    try:
        kc = encode_cache(kv_values(rng, (n_layers, n_seqs, max_seq, hkv, d)), oracle.F8)
        vc = encode_cache(kv_values(rng, (n_layers, n_seqs, max_seq, hkv, d)), oracle.F8)
        for l in range(n_layers):
            for s in range(n_seqs):
                rig.put(l, s, kc[l, s], vc[l, s])
        rig.fwd.stream = stream.cuda_stream
        pin = lambda a: torch.from_numpy(a).pin_memory()
        q = [pin(rng.standard_normal((n_layers, n_seqs, hq, d), dtype=np.float32)) for _ in range(steps)]
        kn = [pin(kv_values(rng, (n_layers, n_seqs, hkv, d), outlier_frac=0.0)) for _ in range(steps)]
        vn = [pin(kv_values(rng, (n_layers, n_seqs, hkv, d), outlier_frac=0.0)) for _ in range(steps)]
        out = [torch.zeros(n_layers, n_seqs, hq, d).pin_memory() for _ in range(steps)]
        pos = [np.array([base + t, base - 300 + t], np.uint32) for t in range(steps)]
        want = []
        for t in range(steps):                     # the oracle appends token t's rows, then attends
            want.append([oracle.decode_step(q[t][l].numpy(), kn[t][l].numpy(), vn[t][l].numpy(), kc[l], vc[l], oracle.F8,
                                            n_seqs, max_seq, hq, hkv, d, pos[t] + 1) for l in range(n_layers)])
        tickets = {}
        submit = lambda t: tickets.__setitem__(t, rig.fwd.decode_token_host_submit(q[t], kn[t], vn[t], out[t], pos[t], n_seqs))
        submit(0)
        submit(1)
        with pytest.raises(vf.VfkvError):          # both staging sets are in flight
            rig.fwd.decode_token_host_submit(q[2], kn[2], vn[2], out[2], pos[2], n_seqs)
        for t in range(steps):
            rig.fwd.decode_token_host_wait(tickets[t])
            for l in range(n_layers):
                check(out[t][l].numpy(), want[t][l], oracle.F8)
            if t + 2 < steps:
                submit(t + 2)
        with pytest.raises(vf.VfkvError):
            rig.fwd.decode_token_host_wait(tickets[0])     # no longer in flight
        ctx.poll()
    finally:
        torch.cuda.synchronize()
        rig.fwd.stream = None
        rig.close()


def test_attend_argument_errors(ctx):
    import torch
    rig = Rig(ctx, vf.KvDtype.F16, 32, 8, 128, 64)
    try:
        L = ctx._lib
        x = torch.zeros(32 * 128, device="cuda")
        E = vf.kv_cache.ERR_INVALID
        h, w = rig.cache.handle, rig.fwd.workspace.handle
        assert L.vfkv_attend(h, w, 0, 0, x.data_ptr(), x.data_ptr(), 32, 0, 65, 0, 1.0, 0.0, 0, None) == E
        assert L.vfkv_attend(h, w, 0, 0, x.data_ptr(), x.data_ptr(), 32, 0, 10, 11, 1.0, 0.0, 0, None) == E
        assert L.vfkv_attend(h, w, 1, 0, x.data_ptr(), x.data_ptr(), 32, 0, 10, 0, 1.0, 0.0, 0, None) == E
        assert L.vfkv_attend(h, w, 0, 0, x.data_ptr(), x.data_ptr(), 30, 0, 10, 0, 1.0, 0.0, 0, None) == E
        assert L.vfkv_attend(h, w, 0, 0, x.data_ptr(), x.data_ptr(), 32, 1, 10, 0, 1.0, 0.0, 0, None) == E
        assert L.vfkv_attend(h, None, 0, 0, x.data_ptr(), x.data_ptr(), 32, 0, 10, 0, 1.0, 0.0, 4, None) == E
        assert L.vfkv_attend(h, w, 0, 0, None, x.data_ptr(), 32, 0, 10, 0, 1.0, 0.0, 0, None) == E
        # an empty visible range is defined as zeros
        out = torch.full((32, 128), 7.0, device="cuda")
        assert L.vfkv_attend(h, w, 0, 0, x.data_ptr(), out.data_ptr(), 32, 0, 10, 10, 1.0, 0.0, 0, None) == 0
        torch.cuda.synchronize()
        assert float(out.abs().max()) == 0.0
    finally:
        rig.close()


@pytest.mark.parametrize("dtype", [vf.KvDtype.F8, vf.KvDtype.F16])
def test_decode_token_kernel_shapes_dependent_launch_and_graph_replay(ctx, dtype):
    """vfkv_decode_token (every layer in one call) under each tensor-core kernel shape and each
    dependent-launch mode, launched directly and replayed from a CUDA graph: same results."""
    import torch
    hq, hkv, d, max_seq, n_layers, n_seqs = 32, 8, 128, 900, 3, 2
    rng = np.random.default_rng(71)
    pos = np.array([899, 400], np.uint32)
    fp8 = dtype == vf.KvDtype.F8
    kc = encode_cache(kv_values(rng, (n_layers, n_seqs, max_seq, hkv, d), outlier_frac=0.01 if fp8 else 0.0), int(dtype))
    vc = encode_cache(kv_values(rng, (n_layers, n_seqs, max_seq, hkv, d), outlier_frac=0.01 if fp8 else 0.0), int(dtype))
    q = rng.standard_normal((n_layers, n_seqs, hq, d), dtype=np.float32)
    kn = kv_values(rng, (n_layers, n_seqs, hkv, d), outlier_frac=0.0)
    vn = kv_values(rng, (n_layers, n_seqs, hkv, d), outlier_frac=0.0)
    want = []
    for l in range(n_layers):
        kk, vv = kc[l].copy(), vc[l].copy()
        want.append(oracle.decode_step(q[l], kn[l], vn[l], kk, vv, int(dtype), n_seqs, max_seq, hq, hkv, d, pos + 1))
    L = ctx._lib
    stream = torch.cuda.Stream()
    rig = Rig(ctx, dtype, hq, hkv, d, max_seq, n_layers=n_layers, n_slots=n_seqs, n_splits=5)
    try:
        dq, dk, dv, dpos = to_dev(q), to_dev(kn), to_dev(vn), to_dev(pos)
        out = torch.zeros(n_layers, n_seqs, hq, d, device="cuda")
        rig.fwd.stream = stream.cuda_stream
        for tune in ((4, 1), (4, 2), (4, 3), (8, 1), (8, 3), (0, 0)):
            for mode in (0, 1, 2):
                ctx.check(L.vfkv_ctx_set_attn_tuning(ctx.handle, *tune))
                ctx.check(L.vfkv_ctx_set_dependent_launch(ctx.handle, mode))
                for l in range(n_layers):
                    for s in range(n_seqs):
                        rig.put(l, s, kc[l, s], vc[l, s])        # restore the rows the step overwrites
                torch.cuda.synchronize()
                with torch.cuda.stream(stream):
                    out.zero_()
                    rig.fwd.decode_token(dq, dk, dv, out, None, dpos, n_seqs, 900)
                stream.synchronize()
                got = out.cpu().numpy()
                for l in range(n_layers):
                    check(got[l], want[l], dtype)
        # graph replay of the last configuration's successor: default shape, mode 2
        ctx.check(L.vfkv_ctx_set_attn_tuning(ctx.handle, 0, 0))
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            rig.fwd.decode_token(dq, dk, dv, out, None, dpos, n_seqs, 900)
        for _ in range(3):
            with torch.cuda.stream(stream):
                out.zero_()
                g.replay()
            stream.synchronize()
            got = out.cpu().numpy()
            for l in range(n_layers):
                check(got[l], want[l], dtype)
    finally:
        ctx.check(L.vfkv_ctx_set_attn_tuning(ctx.handle, 0, 0))
        ctx.check(L.vfkv_ctx_set_dependent_launch(ctx.handle, 0))
        rig.close()


def test_split_that_gives_up_is_reported_and_the_next_launch_is_clean(ctx):
    """A CTA whose bounded wait runs out (injected on the host: one split of kv-head 0 acts as if its
    tile never arrived) publishes no partial.  The merging CTA's wait for it is bounded too, the
    status word reports the failure, and -- because every CTA draws its split ticket before it can
    give up -- the workspace needs no repair: the very next launch on it is correct."""
    import torch
    hq, hkv, d, L = 32, 8, 128, 1500
    rng = np.random.default_rng(91)
    kc, vc = encode_cache(kv_values(rng, (L, hkv, d)), oracle.F8), encode_cache(kv_values(rng, (L, hkv, d)), oracle.F8)
    q = rng.standard_normal((hq, d), dtype=np.float32)
    want = oracle.attention_ref(q, kc, vc, oracle.F8, hq, hkv, d, L)
    rig = Rig(ctx, vf.KvDtype.F8, hq, hkv, d, L)
    try:
        rig.put(0, 0, kc, vc)
        ctx.set_merge_wait_ms(20)
        for failing in (0, 3):
            ctx.debug_fail_split(failing)
            rig.attend(q, 0, L, n_splits=4)
            with pytest.raises(vf.VfkvError) as err:
                ctx.poll()
            assert err.value.status == vf.kv_cache.ERR_TIMEOUT
            ctx.debug_fail_split(None)
            for n_splits in (4, 7):                      # no reset in between
                got = rig.attend(q, 0, L, n_splits=n_splits)
                ctx.poll()
                check(got, want, oracle.F8)
        rig.fwd.workspace.reset()                        # the explicit repair call is harmless too
        check(rig.attend(q, 0, L, n_splits=4), want, oracle.F8)
        ctx.poll()
    finally:
        ctx.debug_fail_split(None)
        ctx.set_merge_wait_ms(1000)
        rig.close()


@pytest.mark.parametrize("dtype,hq,hkv,d", [(vf.KvDtype.F8, 8, 1, 128), (vf.KvDtype.F8, 16, 2, 128),
                                            (vf.KvDtype.F16, 4, 1, 128), (vf.KvDtype.F8, 5, 1, 256)])
def test_few_kv_heads_cut_into_many_splits(ctx, dtype, hq, hkv, d):
    """A rank's share of a sequence sharded by kv-head group: one or two kv-heads, the whole length.
    The split count chosen for it runs to one CTA per SM and up to sixteen CTAs of a group share
    the merge; explicit counts cover slices that do not divide evenly, and a split that gives up is
    still reported when many CTAs wait for it."""
    L = 40000
    rng = np.random.default_rng(23)
    kc, vc = encode_cache(kv_values(rng, (L, hkv, d)), int(dtype)), encode_cache(kv_values(rng, (L, hkv, d)), int(dtype))
    q = rng.standard_normal((hq, d), dtype=np.float32)
    want = oracle.attention_ref(q, kc, vc, int(dtype), hq, hkv, d, L)
    rig = Rig(ctx, dtype, hq, hkv, d, L, max_splits=255)
    try:
        rig.put(0, 0, kc, vc)
        for n_splits in (0, 37, 128, 148, 255):
            got = rig.attend(q, 0, L, n_splits=n_splits)
            ctx.poll()
            check(got, want, int(dtype), relative=True)
        got = rig.attend(q, 0, 700, n_splits=0)          # shorter than one round of tiles per split
        ctx.poll()
        check(got, oracle.attention_ref(q, kc, vc, int(dtype), hq, hkv, d, 700), int(dtype), relative=True)
        ctx.set_merge_wait_ms(20)
        ctx.debug_fail_split(0)
        rig.attend(q, 0, L, n_splits=128)
        with pytest.raises(vf.VfkvError) as err:
            ctx.poll()
        assert err.value.status == vf.kv_cache.ERR_TIMEOUT
        ctx.debug_fail_split(None)
        check(rig.attend(q, 0, L, n_splits=128), want, int(dtype), relative=True)
        ctx.poll()
    finally:
        ctx.debug_fail_split(None)
        ctx.set_merge_wait_ms(1000)
        rig.close()


@pytest.mark.parametrize("dtype", [vf.KvDtype.F8, vf.KvDtype.F16])
def test_dependent_launch_mode2_on_one_layer_with_advancing_positions(ctx, dtype):
    """Mode 2 prefetches K/V before it waits for the kernel in front of it.  On a one-layer cache
    every decode step reads the slab the step before it appended to; the library must notice that
    and wait first.  Eight tokens are enqueued back to back without a host synchronisation; token
    t attends over the rows tokens 0..t-1 appended."""
    import torch
    hq, hkv, d, max_seq, base, steps = 32, 8, 128, 700, 600, 8
    rng = np.random.default_rng(17)
    fp8 = dtype == vf.KvDtype.F8
    kc = encode_cache(kv_values(rng, (1, max_seq, hkv, d), outlier_frac=0.01 if fp8 else 0.0), int(dtype))
    vc = encode_cache(kv_values(rng, (1, max_seq, hkv, d), outlier_frac=0.01 if fp8 else 0.0), int(dtype))
    q = rng.standard_normal((steps, 1, hq, d), dtype=np.float32)
    kn = kv_values(rng, (steps, 1, hkv, d), outlier_frac=0.0)
    vn = kv_values(rng, (steps, 1, hkv, d), outlier_frac=0.0)
    kk, vv = kc.copy(), vc.copy()
    want = [oracle.decode_step(q[t], kn[t], vn[t], kk, vv, int(dtype), 1, max_seq, hq, hkv, d,
                               np.array([base + t + 1], np.uint32)) for t in range(steps)]
    stream = torch.cuda.Stream()
    rig = Rig(ctx, dtype, hq, hkv, d, max_seq, n_splits=4)
    try:
        rig.put(0, 0, kc[0], vc[0])
        dq, dk, dv = to_dev(q), to_dev(kn), to_dev(vn)
        dpos = to_dev(np.arange(base, base + steps, dtype=np.uint32))
        out = torch.zeros(steps, 1, hq, d, device="cuda")
        rig.fwd.stream = stream.cuda_stream
        ctx.set_dependent_launch(2)
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            for t in range(steps):
                rig.fwd.decode_step(0, dq[t], dk[t], dv[t], out[t], None, dpos[t:t + 1], 1, max_seq)
        stream.synchronize()
        ctx.poll()
        got = out.cpu().numpy()
        for t in range(steps):
            check(got[t], want[t], dtype)
    finally:
        ctx.set_dependent_launch(0)
        rig.close()
