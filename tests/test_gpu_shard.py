"""Position-sharded decode attention: pages dealt round-robin to the ranks, local (m, l, o)
partials, packed merge.  On one GPU the ranks are emulated one after another (the exchange is
then just the packed buffer); with two or more GPUs a real NCCL all-gather runs between child
processes."""
import os
import socket

import numpy as np
import pytest

import oracle
import vulkanforge_b200 as vf
from util import encode_cache, kv_values, rel_err, to_dev
from vulkanforge_b200.shard import PositionShards, ShardedSequenceDecoder, packed_partial_floats

pytestmark = pytest.mark.gpu

HQ, HKV, D = 64, 8, 128


def _inputs(seq_len, seed):
    rng = np.random.default_rng(seed)
    k = kv_values(rng, (seq_len + 1, HKV, D))
    v = kv_values(rng, (seq_len + 1, HKV, D))
    q = rng.standard_normal((HQ, D), dtype=np.float32)
    return q, k, v


@pytest.mark.parametrize("dtype", ["F8", "F16"])
def test_sharded_chunk_append_stores_this_ranks_rows_in_one_launch(ctx, dtype):
    """vfkv_append_sharded against one vfkv_append per page piece: the same cache bytes on every
    rank, one launch per chunk; a chunk that would overrun the rank's rows is refused."""
    import torch
    from util import dev_view_bytes
    world, page, seq_len = 3, 64, 1000
    _, k, v = _inputs(seq_len, seed=77)
    sh = PositionShards(world, page)
    cap = sh.local_capacity(seq_len)
    dk, dv = to_dev(k), to_dev(v)
    for r in range(world):
        caches = [vf.KvCache(ctx, vf.KvCacheConfig(1, HKV, D, cap), vf.KvDtype[dtype]) for _ in range(2)]
        fwds = [vf.CudaForward(ctx, c, n_heads=HQ) for c in caches]
        try:
            for c in caches:
                c.zero_fill()
            for base, n in ((0, 37), (37, 500), (537, 463)):          # chunks that start and end inside pages
                n0 = ctx.launch_count()
                fwds[0].b_step_kv_write_sharded(0, dk[base:base + n], dv[base:base + n], n, base, world, page, r)
                assert ctx.launch_count() - n0 == 1
                p = base
                while p < base + n:
                    stop = min(base + n, (p // page + 1) * page)
                    if sh.owner(p) == r:
                        fwds[1].b_step_kv_write(0, dk[p:stop], dv[p:stop], stop - p, sh.local_pos(p))
                    p = stop
            torch.cuda.synchronize()
            ctx.poll()
            nbytes = caches[0].bytes_per_buffer()
            for buf in ("k_buffer", "v_buffer"):
                a = dev_view_bytes(getattr(caches[0], buf), nbytes)
                b = dev_view_bytes(getattr(caches[1], buf), nbytes)
                assert a.any() and np.array_equal(a, b)
            with pytest.raises(vf.VfkvError):
                fwds[0].b_step_kv_write_sharded(0, dk, dv, seq_len, world * cap, world, page, r)
        finally:
            for f, c in zip(fwds, caches):
                f.workspace.destroy()
                c.destroy()


@pytest.mark.parametrize("world,page,seq_len", [(4, 256, 5000), (8, 256, 9000), (2, 64, 700), (3, 256, 100)])
def test_emulated_ranks_chunked_prefill_append_and_merge(ctx, world, page, seq_len):
    import torch
    q, k, v = _inputs(seq_len, seed=world * 1000 + seq_len)
    sh = PositionShards(world, page)
    cap = sh.local_capacity(seq_len + 1)
    ranks = []
    try:
        for r in range(world):
            cache = vf.KvCache(ctx, vf.KvCacheConfig(1, HKV, D, cap), vf.KvDtype.F8)
            fwd = vf.CudaForward(ctx, cache, n_heads=HQ)
            ranks.append((cache, fwd, ShardedSequenceDecoder(fwd, sh, r)))
        # chunked prefill of 512-token chunks: every rank keeps the rows of its own pages
        dk, dv = to_dev(k), to_dev(v)
        for base in range(0, seq_len, 512):
            n = min(512, seq_len - base)
            stored = sum(dec.prefill(0, dk[base:base + n], dv[base:base + n], base, n) for _, _, dec in ranks)
            assert stored == n
        n_packed = packed_partial_floats(HQ, D)
        dq = to_dev(q)
        for L in (seq_len, seq_len + 1):
            if L == seq_len + 1:      # decode step: only the owner of the new position appends
                owners = [dec.append(0, dk[seq_len:], dv[seq_len:], seq_len) for _, _, dec in ranks]
                assert owners.count(True) == 1 and owners.index(True) == sh.owner(seq_len)
            packed = torch.zeros(world, n_packed, device="cuda")
            for r, (_, fwd, _) in enumerate(ranks):
                blk = packed[r]
                fwd.attend_partial(0, dq, 0, sh.local_len(L, r), blk[:HQ], blk[HQ:2 * HQ], blk[2 * HQ:])
            out = torch.zeros(HQ, D, device="cuda")
            ranks[0][1].merge_partials_packed(packed, world, HQ, D, out)
            torch.cuda.synchronize()
            kc, vc = encode_cache(k[:L], oracle.F8), encode_cache(v[:L], oracle.F8)
            want = oracle.attention_ref(q, kc, vc, oracle.F8, HQ, HKV, D, L)
            assert rel_err(out.cpu().numpy(), want) < 3e-2
    finally:
        for cache, fwd, _ in ranks:
            fwd.workspace.destroy()
            cache.destroy()


def _emulated_group(ctx, world, seq_len, dtype, hq=HQ, hkv=HKV, d=D, page=256):
    """world ranks of one process on one GPU: caches, forwards, decoders and connected exchanges."""
    sh = PositionShards(world, page)
    ranks = []
    for r in range(world):
        cache = vf.KvCache(ctx, vf.KvCacheConfig(1, hkv, d, sh.local_capacity(seq_len + 8)), dtype)
        fwd = vf.CudaForward(ctx, cache, n_heads=hq)
        ex = vf.PeerExchange(ctx, world, r, hq, d)
        ranks.append((cache, fwd, ShardedSequenceDecoder(fwd, sh, r), ex))
    for r, (_, _, _, ex) in enumerate(ranks):
        for o, (_, _, _, other) in enumerate(ranks):
            if o != r:
                ex.set_peer(o, other.local_ptr())
        assert ex.ready()
    return sh, ranks


def _destroy_group(ranks):
    for cache, fwd, _, ex in ranks:
        ex.destroy()
        fwd.workspace.destroy()
        cache.destroy()


@pytest.mark.parametrize("world,seq_len,dtype,hq,hkv,d", [
    (2, 3000, "F8", 64, 8, 128),      # tensor-core kernel, several splits: fan-out from the merging CTA
    (4, 900, "F8", 64, 8, 128),       # one split per rank: fan-out from the direct epilogue
    (8, 5000, "F16", 32, 8, 128),
    (3, 100, "F8", 64, 8, 128),       # ranks 1 and 2 hold nothing
    (2, 700, "F32", 8, 2, 64),        # CUDA-core kernel + push kernel
])
def test_peer_exchange_emulated_ranks(ctx, world, seq_len, dtype, hq, hkv, d):
    """The partial of every rank is stored by its attention kernel into all ranks' buffers; each
    rank's merge then finds every flag set.  Several decode steps in a row exercise the parity
    double-buffering and the device-side exchange counter.  On one GPU the producers all run
    before the consumers, so no kernel ever waits."""
    import torch
    kv_dtype = vf.KvDtype[dtype]
    odt = {"F8": oracle.F8, "F16": oracle.F16, "F32": oracle.F32}[dtype]
    rng = np.random.default_rng(world * 100 + seq_len)
    steps = 4
    k = kv_values(rng, (seq_len + steps, hkv, d))
    v = kv_values(rng, (seq_len + steps, hkv, d))
    sh, ranks = _emulated_group(ctx, world, seq_len, kv_dtype, hq, hkv, d)
    try:
        dk, dv = to_dev(k), to_dev(v)
        for _, _, dec, _ in ranks:
            dec.prefill(0, dk[:seq_len], dv[:seq_len], 0, seq_len)
        outs = [torch.zeros(hq, d, device="cuda") for _ in ranks]
        for t in range(steps):
            L = seq_len + t + 1
            q = rng.standard_normal((hq, d), dtype=np.float32)
            dq = to_dev(q)
            for r, (_, fwd, dec, ex) in enumerate(ranks):
                if t % 2 == 0:        # KvWrite as its own launch, then the attention
                    dec.append(0, dk[L - 1:L], dv[L - 1:L], L - 1)
                    fwd.attend_push(ex, 0, dq, 0, sh.local_len(L, r))
                else:                 # the owner's attention kernel stores the new row itself
                    mine = sh.owner(L - 1) == r
                    fwd.attend_push(ex, 0, dq, 0, sh.local_len(L, r), k_new=dk[L - 1] if mine else None,
                                    v_new=dv[L - 1] if mine else None)
            for r, (_, fwd, _, ex) in enumerate(ranks):
                fwd.exchange_merge(ex, outs[r])
            torch.cuda.synchronize()
            ctx.poll()
            kc, vc = encode_cache(k[:L], odt), encode_cache(v[:L], odt)
            want = oracle.attention_ref(q, kc, vc, odt, hq, hkv, d, L)
            for r in range(world):
                got = outs[r].cpu().numpy()
                if dtype == "F8":
                    assert rel_err(got, want) < 3e-2
                else:
                    assert np.max(np.abs(got - want)) < 2e-3
                assert np.array_equal(got, outs[0].cpu().numpy())      # every rank merges the same blocks
    finally:
        _destroy_group(ranks)


def test_peer_exchange_wait_runs_out_and_context_survives(ctx):
    """A flag that nothing sets: the merge gives up after its time limit, reports it through the
    status word, and the next exchanges work."""
    import torch
    world, seq_len = 2, 600
    rng = np.random.default_rng(5)
    k = kv_values(rng, (seq_len, HKV, D))
    v = kv_values(rng, (seq_len, HKV, D))
    q = rng.standard_normal((HQ, D), dtype=np.float32)
    sh, ranks = _emulated_group(ctx, world, seq_len, vf.KvDtype.F8)
    try:
        dk, dv, dq = to_dev(k), to_dev(v), to_dev(q)
        for _, _, dec, ex in ranks:
            dec.prefill(0, dk, dv, 0, seq_len)
            ex.set_timeout_ms(20)
        outs = [torch.ones(HQ, D, device="cuda") for _ in ranks]
        (_, f0, _, e0), (_, f1, _, e1) = ranks
        f0.attend_push(e0, 0, dq, 0, sh.local_len(seq_len, 0))
        f0.exchange_merge(e0, outs[0])                    # rank 1 has not pushed
        torch.cuda.synchronize()
        with pytest.raises(vf.VfkvError) as err:
            ctx.poll()
        assert err.value.status == vf.kv_cache.ERR_TIMEOUT
        assert float(outs[0].abs().max()) == 0.0          # the row is written as zeros, not garbage
        f1.attend_push(e1, 0, dq, 0, sh.local_len(seq_len, 1))
        f1.exchange_merge(e1, outs[1])                    # both blocks of exchange 1 are there now
        torch.cuda.synchronize()
        ctx.poll()
        kc, vc = encode_cache(k, oracle.F8), encode_cache(v, oracle.F8)
        want = oracle.attention_ref(q, kc, vc, oracle.F8, HQ, HKV, D, seq_len)
        assert rel_err(outs[1].cpu().numpy(), want) < 3e-2
        for r, (_, fwd, _, ex) in enumerate(ranks):       # exchange 2 on both ranks
            fwd.attend_push(ex, 0, dq, 0, sh.local_len(seq_len, r))
        for r, (_, fwd, _, ex) in enumerate(ranks):
            fwd.exchange_merge(ex, outs[r])
        torch.cuda.synchronize()
        ctx.poll()
        for r in range(world):
            assert rel_err(outs[r].cpu().numpy(), want) < 3e-2
    finally:
        _destroy_group(ranks)


@pytest.mark.parametrize("world,seq_len,n_splits", [(2, 3000, 0), (2, 900, 1), (1, 2500, 0), (4, 6000, 5)])
def test_one_launch_exchange_with_the_other_ranks_already_there(ctx, world, seq_len, n_splits):
    """vfkv_attend_exchange on the tensor-core path is ONE launch: attention, fan-out of the block
    to every rank, wait for the other ranks' blocks in this GPU's own buffer, final rows.  The
    waiting kernel needs the other ranks' kernels to run beside it, which one GPU cannot offer, so
    here ranks 1.. push first (two-call form) and rank 0 then runs the one-launch form: its waits
    are real polls that find the words there.  Several steps in a row cover the parity
    double-buffering and the exchange counter advanced by the kernel itself."""
    import torch
    hq, hkv, d = HQ, HKV, D
    rng = np.random.default_rng(world * 31 + seq_len)
    steps = 4
    k = kv_values(rng, (seq_len + steps, hkv, d))
    v = kv_values(rng, (seq_len + steps, hkv, d))
    sh, ranks = _emulated_group(ctx, world, seq_len, vf.KvDtype.F8)
    try:
        dk, dv = to_dev(k), to_dev(v)
        for _, fwd, dec, _ in ranks:
            fwd.n_splits = n_splits
            dec.prefill(0, dk[:seq_len], dv[:seq_len], 0, seq_len)
        outs = [torch.zeros(hq, d, device="cuda") for _ in ranks]
        for t in range(steps):
            L = seq_len + t + 1
            q = rng.standard_normal((hq, d), dtype=np.float32)
            dq = to_dev(q)
            new = lambda r: dict(k_new=dk[L - 1], v_new=dv[L - 1]) if sh.owner(L - 1) == r else {}
            for r in range(1, world):
                _, fwd, _, ex = ranks[r]
                fwd.attend_push(ex, 0, dq, 0, sh.local_len(L, r), **new(r))
            n0 = ctx.launch_count()
            _, fwd0, _, ex0 = ranks[0]
            fwd0.attend_exchange(ex0, 0, dq, 0, sh.local_len(L, 0), outs[0], **new(0))
            assert ctx.launch_count() - n0 == 1
            for r in range(1, world):
                _, fwd, _, ex = ranks[r]
                fwd.exchange_merge(ex, outs[r])
            torch.cuda.synchronize()
            ctx.poll()
            kc, vc = encode_cache(k[:L], oracle.F8), encode_cache(v[:L], oracle.F8)
            want = oracle.attention_ref(q, kc, vc, oracle.F8, hq, hkv, d, L)
            for r in range(world):
                assert rel_err(outs[r].cpu().numpy(), want) < 1e-4, (t, r)
    finally:
        _destroy_group(ranks)


def test_one_launch_exchange_wait_runs_out_and_context_survives(ctx):
    """The one-launch form with a peer that never stores: the kernel's wait is bounded, the status
    word says so, the rows are zeros, and the next exchanges work."""
    import torch
    world, seq_len = 2, 800
    rng = np.random.default_rng(6)
    k = kv_values(rng, (seq_len, HKV, D))
    v = kv_values(rng, (seq_len, HKV, D))
    q = rng.standard_normal((HQ, D), dtype=np.float32)
    sh, ranks = _emulated_group(ctx, world, seq_len, vf.KvDtype.F8)
    try:
        dk, dv, dq = to_dev(k), to_dev(v), to_dev(q)
        for _, _, dec, ex in ranks:
            dec.prefill(0, dk, dv, 0, seq_len)
            ex.set_timeout_ms(20)
        outs = [torch.ones(HQ, D, device="cuda") for _ in ranks]
        (_, f0, _, e0), (_, f1, _, e1) = ranks
        f0.attend_exchange(e0, 0, dq, 0, sh.local_len(seq_len, 0), outs[0])      # rank 1 has not pushed
        torch.cuda.synchronize()
        with pytest.raises(vf.VfkvError) as err:
            ctx.poll()
        assert err.value.status == vf.kv_cache.ERR_TIMEOUT
        assert float(outs[0].abs().max()) == 0.0
        f1.attend_push(e1, 0, dq, 0, sh.local_len(seq_len, 1))                   # exchange 1 of rank 1
        f1.exchange_merge(e1, outs[1])
        torch.cuda.synchronize()
        ctx.poll()
        kc, vc = encode_cache(k, oracle.F8), encode_cache(v, oracle.F8)
        want = oracle.attention_ref(q, kc, vc, oracle.F8, HQ, HKV, D, seq_len)
        assert rel_err(outs[1].cpu().numpy(), want) < 1e-4
        f1.attend_push(e1, 0, dq, 0, sh.local_len(seq_len, 1))                   # exchange 2 on both
        f0.attend_exchange(e0, 0, dq, 0, sh.local_len(seq_len, 0), outs[0])
        f1.exchange_merge(e1, outs[1])
        torch.cuda.synchronize()
        ctx.poll()
        for r in range(world):
            assert rel_err(outs[r].cpu().numpy(), want) < 1e-4
    finally:
        _destroy_group(ranks)


@pytest.mark.parametrize("world,dtype", [(2, "F8"), (4, "F16"), (3, "F8")])
def test_kv_head_group_sharding_needs_no_exchange(ctx, world, dtype):
    """Sharding by kv-head group: rank r holds the rows of its kv-heads only (a cache with fewer
    heads) and the q-heads that read them (kvh = h / g, flash_attn_split.comp:83-95).  Each rank's
    decode step writes a disjoint slice of the output heads; put side by side the slices are the
    full result.  Ranks are emulated one after the other: there is nothing to exchange."""
    import ctypes as C
    import torch
    hq, hkv, d, L = 32, 8, 128, 3000
    odt = {"F8": oracle.F8, "F16": oracle.F16}[dtype]
    rng = np.random.default_rng(world)
    k = kv_values(rng, (L, hkv, d), outlier_frac=0.01 if dtype == "F8" else 0.0)
    v = kv_values(rng, (L, hkv, d), outlier_frac=0.01 if dtype == "F8" else 0.0)
    q = rng.standard_normal((hq, d), dtype=np.float32)
    g = hq // hkv
    out = np.zeros((hq, d), np.float32)
    first, count = C.c_uint32(), C.c_uint32()
    for r in range(world):
        ctx.check(ctx._lib.vfkv_shard_kv_heads(world, r, hkv, C.byref(first), C.byref(count)))
        h0, n = first.value, count.value
        cache = vf.KvCache(ctx, vf.KvCacheConfig(1, n, d, L), vf.KvDtype[dtype])
        fwd = vf.CudaForward(ctx, cache, n_heads=n * g)
        try:
            fwd.b_step_kv_write(0, to_dev(k[:L - 1, h0:h0 + n]), to_dev(v[:L - 1, h0:h0 + n]), L - 1, 0)
            o = torch.zeros(n * g, d, device="cuda")
            pos = to_dev(np.array([L - 1], np.uint32))
            fwd.decode_step(0, to_dev(q[h0 * g:(h0 + n) * g]), to_dev(k[L - 1:, h0:h0 + n]), to_dev(v[L - 1:, h0:h0 + n]),
                            o, None, pos, 1)
            torch.cuda.synchronize()
            ctx.poll()
            out[h0 * g:(h0 + n) * g] = o.cpu().numpy()
        finally:
            fwd.workspace.destroy()
            cache.destroy()
    want = oracle.attention_ref(q, encode_cache(k, odt), encode_cache(v, odt), odt, hq, hkv, d, L)
    if dtype == "F8":
        assert rel_err(out, want) < 1e-4
    else:
        assert np.max(np.abs(out - want)) < 2e-5


def test_attend_allgather_on_a_communicator_of_one(ctx):
    """vfkv_attend_allgather (partial, ncclAllGather on the caller's communicator, merge) with a
    world of one: the collective is a copy, the result the plain attention."""
    import torch
    from util import NcclComm
    seq_len = 3000
    q, k, v = _inputs(seq_len, seed=12)
    cache = vf.KvCache(ctx, vf.KvCacheConfig(1, HKV, D, seq_len), vf.KvDtype.F8)
    fwd = vf.CudaForward(ctx, cache, n_heads=HQ)
    comm = NcclComm(1, 0, lambda raw: raw)
    try:
        fwd.b_step_kv_write(0, to_dev(k[:seq_len]), to_dev(v[:seq_len]), seq_len, 0)
        packed = torch.zeros(HQ * (D + 2), device="cuda")
        out = torch.zeros(HQ, D, device="cuda")
        fwd.attend_allgather(comm.handle, 1, 0, 0, to_dev(q), 0, seq_len, packed, out)
        torch.cuda.synchronize()
        ctx.poll()
        kc, vc = encode_cache(k[:seq_len], oracle.F8), encode_cache(v[:seq_len], oracle.F8)
        want = oracle.attention_ref(q, kc, vc, oracle.F8, HQ, HKV, D, seq_len)
        assert rel_err(out.cpu().numpy(), want) < 1e-4
        with pytest.raises(vf.VfkvError):
            fwd.attend_allgather(0, 1, 0, 0, to_dev(q), 0, seq_len, packed, out)
        with pytest.raises(vf.VfkvError):
            fwd.attend_allgather(comm.handle, 1, 1, 0, to_dev(q), 0, seq_len, packed, out)
    finally:
        comm.destroy()
        fwd.workspace.destroy()
        cache.destroy()


def _nccl_rank(rank, world, port, seq_len, result_dir):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        q, k, v = _inputs(seq_len, seed=7)
        sh = PositionShards(world, 256)
        ctx = vf.Context(rank)
        cache = vf.KvCache(ctx, vf.KvCacheConfig(1, HKV, D, sh.local_capacity(seq_len + 1)), vf.KvDtype.F8)
        fwd = vf.CudaForward(ctx, cache, n_heads=HQ)
        dec = ShardedSequenceDecoder(fwd, sh, rank)
        dk = torch.from_numpy(k).cuda()
        dv = torch.from_numpy(v).cuda()
        dec.prefill(0, dk[:seq_len], dv[:seq_len], 0, seq_len)
        dec.append(0, dk[seq_len:], dv[seq_len:], seq_len)
        out = torch.zeros(HQ, D, device="cuda")
        dec.attend(0, torch.from_numpy(q).cuda(), out, seq_len + 1)
        torch.cuda.synchronize()
        ctx.poll()
        kc, vc = encode_cache(k, oracle.F8), encode_cache(v, oracle.F8)
        want = oracle.attention_ref(q, kc, vc, oracle.F8, HQ, HKV, D, seq_len + 1)
        errs = [rel_err(out.cpu().numpy(), want)]
        # the same through the C entry that carries the collective: a raw communicator (its unique
        # id handed round over the process group), no PyTorch collective on the path
        from util import NcclComm

        def exchange_id(raw):
            box = [raw]
            dist.broadcast_object_list(box, src=0)
            return box[0]

        comm = NcclComm(world, rank, exchange_id)
        packed = torch.zeros(world * HQ * (D + 2), device="cuda")
        for _ in range(2):
            out.zero_()
            fwd.attend_allgather(comm.handle, world, rank, 0, torch.from_numpy(q).cuda(), 0,
                                 sh.local_len(seq_len + 1, rank), packed, out)
            torch.cuda.synchronize()
            ctx.poll()
            errs.append(rel_err(out.cpu().numpy(), want))
        comm.destroy()
        # the same attention with the partials exchanged by peer stores (IPC-mapped buffers),
        # first as plain launches, then replayed from a CUDA graph
        ex = vf.PeerExchange(ctx, world, rank, HQ, D)
        ex.connect()
        pdec = ShardedSequenceDecoder(fwd, sh, rank, exchange=ex)
        dq = torch.from_numpy(q).cuda()
        for _ in range(3):
            out.zero_()
            pdec.attend(0, dq, out, seq_len + 1)
            torch.cuda.synchronize()
            ctx.poll()
            errs.append(rel_err(out.cpu().numpy(), want))
        stream = torch.cuda.Stream()
        fwd.stream = stream.cuda_stream
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            pdec.attend(0, dq, out, seq_len + 1)
        for _ in range(4):
            out.zero_()
            torch.cuda.synchronize()
            graph.replay()
            torch.cuda.synchronize()
            ctx.poll()
            errs.append(rel_err(out.cpu().numpy(), want))
        fwd.stream = None
        dist.barrier()
        np.save(os.path.join(result_dir, f"err{rank}.npy"), np.array([max(errs)]))
        ex.destroy()
        fwd.workspace.destroy()
        cache.destroy()
        ctx.destroy()
    finally:
        dist.destroy_process_group()


def test_nccl_all_gather_between_gpus(tmp_path):
    import torch
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_nccl_rank, args=(world, port, 20000, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert float(np.load(tmp_path / f"err{r}.npy")[0]) < 3e-2
