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
        np.save(os.path.join(result_dir, f"err{rank}.npy"), np.array([rel_err(out.cpu().numpy(), want)]))
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
