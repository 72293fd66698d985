"""Host-side logic of the multi-GPU partitioning, on CPU: sequence assignment, the round-robin
position pages, and the all-gather of softmax partials over a 2-rank gloo group (the merge
itself runs on the GPU in the product; here a numpy restatement of flash_attn_reduce.comp:51-80
checks that what the collective delivers merges to the oracle's full attention)."""
import os
import socket

import numpy as np
import pytest

import oracle
from vulkanforge_b200.shard import PositionShards, assign_sequences, packed_partial_floats


def test_assign_sequences_balances_total_context():
    rng = np.random.default_rng(3)
    lens = rng.integers(512, 16385, 64)
    for world in (1, 2, 4, 8):
        owned = assign_sequences(lens, world)
        flat = sorted(i for o in owned for i in o)
        assert flat == list(range(64))                       # every sequence exactly once
        loads = [int(sum(lens[i] for i in o)) for o in owned]
        assert max(loads) - min(loads) <= int(lens.max())    # greedy bound
        assert max(loads) <= 1.05 * sum(loads) / world + int(lens.max()) / world
    assert assign_sequences([], 4) == [[], [], [], []]
    assert assign_sequences([5, 9], 4) == [[1], [0], [], []]


@pytest.mark.parametrize("world,page", [(1, 256), (2, 256), (8, 256), (3, 64), (4, 1)])
def test_position_shards_partition_exactly(world, page):
    sh = PositionShards(world, page)
    for seq_len in (0, 1, page - 1, page, page + 1, 5 * page + 7, 131072 if page >= 64 else 1000):
        seen = {}
        for r in range(world):
            pos = sh.global_positions(seq_len, r)
            assert len(pos) == sh.local_len(seq_len, r)
            for loc, p in enumerate(pos):
                assert sh.owner(p) == r and sh.local_pos(p) == loc
                seen[p] = r
        assert sorted(seen) == list(range(seq_len))
        lens = [sh.local_len(seq_len, r) for r in range(world)]
        assert sum(lens) == seq_len and max(lens) - min(lens) <= page
        assert max(lens) <= sh.local_capacity(max(seq_len, 1))
    # appends rotate: consecutive pages land on consecutive ranks
    assert [sh.owner(i * page) for i in range(2 * world)] == [i % world for i in range(2 * world)]


def _partial(q, k, v, scale):
    """(m, l, o) of one rank's rows: o = sum exp(s - m) v, per q-head (numpy, f64)."""
    hq, d = q.shape
    hkv = k.shape[1]
    g = hq // hkv
    m = np.full(hq, -1e30, np.float32)
    l = np.zeros(hq, np.float32)
    o = np.zeros((hq, d), np.float32)
    if k.shape[0] == 0:
        return m, l, o
    for h in range(hq):
        s = (k[:, h // g, :].astype(np.float64) @ q[h].astype(np.float64)) * scale
        mm = s.max()
        p = np.exp(s - mm)
        m[h], l[h] = mm, p.sum()
        o[h] = (p[:, None] * v[:, h // g, :].astype(np.float64)).sum(0)
    return m, l, o


def _merge(packed, hq, d):
    """flash_attn_reduce.comp:51-80 over [parts][m | l | o]."""
    m = packed[:, :hq].astype(np.float64)
    l = packed[:, hq:2 * hq].astype(np.float64)
    o = packed[:, 2 * hq:].reshape(-1, hq, d).astype(np.float64)
    M = m.max(0)
    w = np.exp(m - M)
    return ((o * w[:, :, None]).sum(0) / (l * w).sum(0)[:, None]).astype(np.float32)


def _rank_main(rank, world, port, seq_len, page, result_dir):
    import torch
    import torch.distributed as dist
    from vulkanforge_b200.shard import all_gather_partials
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        hq, hkv, d = 8, 2, 64
        rng = np.random.default_rng(99)                       # same stream on every rank
        q = rng.standard_normal((hq, d), dtype=np.float32)
        k = rng.standard_normal((seq_len, hkv, d), dtype=np.float32)
        v = rng.standard_normal((seq_len, hkv, d), dtype=np.float32)
        sh = PositionShards(world, page)
        mine = sh.global_positions(seq_len, rank)
        m, l, o = _partial(q, k[mine], v[mine], 1.0 / np.sqrt(d))
        packed = torch.from_numpy(np.concatenate([m, l, o.ravel()]).astype(np.float32))
        assert packed.numel() == packed_partial_floats(hq, d)
        gathered = all_gather_partials(packed).numpy()
        assert gathered.shape == (world, packed_partial_floats(hq, d))
        assert np.array_equal(gathered[rank], packed.numpy())
        out = _merge(gathered, hq, d)
        want = oracle.attention_ref(q, k, v, oracle.F32, hq, hkv, d, seq_len)
        err = float(np.max(np.abs(out - want)))
        np.save(os.path.join(result_dir, f"err{rank}.npy"), np.array([err]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("seq_len,page", [(1000, 64), (130, 256), (4097, 256)])
def test_all_gather_of_partials_over_gloo_world2(tmp_path, seq_len, page):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_rank_main, args=(2, port, seq_len, page, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        err = float(np.load(tmp_path / f"err{r}.npy")[0])
        assert err < 1e-4, err


class _FakeForward:
    """Records the calls ShardedSequenceDecoder makes (no GPU): enough to check which rank
    appends, which local range it attends over, and what it hands to the exchange."""

    class _Cfg:
        head_dim = 64

    class _Cache:
        pass

    def __init__(self, n_heads=8):
        self.n_heads = n_heads
        self.kv_cache = self._Cache()
        self.kv_cache.config = self._Cfg()
        self.calls = []

    def step_kv_write(self, layer, k, v, pos, slot):
        self.calls.append(("append", layer, pos, slot))

    def attend_exchange(self, exchange, layer, q, lo, hi, out, k_new=None, v_new=None):
        self.calls.append(("attend_exchange", layer, lo, hi, k_new is not None, v_new is not None))


def test_sharded_decoder_owner_logic_with_peer_exchange(monkeypatch):
    """decode(): every rank attends over its local rows [0, local_len(position + 1)); only the
    owner of the new position passes the new K/V rows to the (fused) call."""
    import sys
    import types
    from vulkanforge_b200.shard import ShardedSequenceDecoder
    fake_torch = types.SimpleNamespace(zeros=lambda *a, **k: None, float32=None)
    monkeypatch.setitem(sys.modules, "torch", fake_torch)      # the decoder only allocates its packed buffer
    world, page = 4, 256
    sh = PositionShards(world, page)
    for position in (0, 255, 256, 1023, 1024, 5000):
        owners = 0
        total = 0
        for rank in range(world):
            fwd = _FakeForward()
            dec = ShardedSequenceDecoder(fwd, sh, rank, exchange=object())
            dec.decode(3, "q", "k", "v", "out", position)
            (name, layer, lo, hi, has_k, has_v), = fwd.calls
            assert (name, layer, lo) == ("attend_exchange", 3, 0)
            assert hi == sh.local_len(position + 1, rank)
            assert has_k == has_v == (sh.owner(position) == rank)
            if has_k:
                owners += 1
                assert hi - 1 == sh.local_pos(position)        # the new row is the last local row of its owner
            total += hi
        assert owners == 1 and total == position + 1


def test_c_abi_sharding_plan_equals_the_python_forms():
    """A host without Python binds the plan through the C ABI (vfkv_shard_*, vfkv_assign_sequences):
    the same numbers as the forms above, on every position of several contexts."""
    import ctypes as C
    import vulkanforge_b200 as vf
    L = vf.load()
    rng = np.random.default_rng(12)
    for world, page in ((1, 256), (2, 256), (8, 256), (3, 64), (5, 7)):
        sh = PositionShards(world, page)
        for pos in list(range(0, 3 * world * page + 5)) + [131071, 2 ** 33 + 17]:
            assert L.vfkv_shard_owner(world, page, pos) == sh.owner(pos)
            assert L.vfkv_shard_local_pos(world, page, pos) == sh.local_pos(pos)
        for seq_len in (0, 1, page, page + 1, 5 * page + 3, 131072, 2 ** 33 + 9):
            for r in range(world):
                assert L.vfkv_shard_local_len(world, page, seq_len, r) == sh.local_len(seq_len, r)
            assert sum(L.vfkv_shard_local_len(world, page, seq_len, r) for r in range(world)) == seq_len
            assert L.vfkv_shard_local_capacity(world, page, seq_len) == sh.local_capacity(seq_len)
    assert L.vfkv_shard_owner(0, 256, 5) == 0 and L.vfkv_shard_local_len(4, 256, 1000, 4) == 0
    for n, world in ((64, 1), (64, 2), (64, 8), (7, 3), (0, 4), (5, 8)):
        lens = rng.integers(512, 16385, n).astype(np.uint32)
        if n > 2:
            lens[1] = lens[0]                                 # a tie
        owner = np.full(max(n, 1), 99, np.uint32)
        rc = L.vfkv_assign_sequences(lens.ctypes.data_as(C.POINTER(C.c_uint32)), n, world,
                                     owner.ctypes.data_as(C.POINTER(C.c_uint32)))
        assert rc == 0
        want = assign_sequences(lens, world)
        got = [[i for i in range(n) if owner[i] == r] for r in range(world)]
        assert got == want
    assert L.vfkv_assign_sequences(None, 3, 2, None) != 0 and L.vfkv_assign_sequences(None, 0, 0, None) != 0
    first, count = C.c_uint32(), C.c_uint32()
    for world, hkv in ((1, 8), (2, 8), (4, 8), (8, 8), (3, 8), (8, 2)):
        covered = []
        for r in range(world):
            assert L.vfkv_shard_kv_heads(world, r, hkv, C.byref(first), C.byref(count)) == 0
            covered += list(range(first.value, first.value + count.value))
            assert abs(count.value - hkv / world) < 1
        assert covered == list(range(hkv))
    assert L.vfkv_shard_kv_heads(2, 2, 8, C.byref(first), C.byref(count)) != 0
