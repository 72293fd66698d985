"""Shared helpers of the test-suite: seeded inputs and host<->device copies."""
from __future__ import annotations

import numpy as np

import oracle


def kv_values(rng: np.random.Generator, shape, outlier_frac=0.01, outlier_gain=20.0) -> np.ndarray:
    """N(0,1) with a fraction of elements multiplied by `outlier_gain` (the FP8 configs' distribution)."""
    x = rng.standard_normal(shape, dtype=np.float32)
    if outlier_frac > 0:
        mask = rng.random(shape) < outlier_frac
        x = np.where(mask, x * np.float32(outlier_gain), x).astype(np.float32)
    return x


def xorshift_floats(n: int, seed: int) -> np.ndarray:
    """The generator of the reference's tests/flash_attn_tiled_ref.rs:189-203: uniform in [-1, 1)."""
    mask = (1 << 64) - 1
    state = (seed * 0x9E3779B97F4A7C15 + 1) & mask
    out = np.empty(n, np.float32)
    for i in range(n):
        state ^= (state << 13) & mask
        state ^= state >> 7
        state ^= (state << 17) & mask
        bits = state & 0x00FFFFFF
        out[i] = np.float32(np.float32(bits) / np.float32(1 << 24)) * np.float32(2.0) - np.float32(1.0)
    return out


def correctness_rs_inputs(n_heads, n_kv_heads, head_dim, seq_len):
    """Deterministic Q/K/V of the reference's split-K test (tests/correctness.rs:2806-2817)."""
    i = np.arange(n_heads * head_dim, dtype=np.float32)
    q = np.sin(i * np.float32(0.001), dtype=np.float32)
    t = np.arange(seq_len, dtype=np.float32)[:, None, None]
    kvh = np.arange(n_kv_heads, dtype=np.float32)[None, :, None]
    d = np.arange(head_dim, dtype=np.float32)[None, None, :]
    k = np.cos((t + np.float32(1.0)) * np.float32(0.01) + d * np.float32(0.001) + kvh * 0, dtype=np.float32)
    v = np.sin(t * np.float32(0.013) + kvh * np.float32(0.7) + d * np.float32(0.0007), dtype=np.float32)
    return q.reshape(n_heads, head_dim), k.astype(np.float32), v.astype(np.float32)


def to_dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def dev_view_bytes(addr: int, nbytes: int):
    """Copies `nbytes` device bytes at raw address `addr` into a numpy uint8 array."""
    import ctypes as C
    import torch
    torch.cuda.synchronize()
    out = np.empty(nbytes, np.uint8)
    import vulkanforge_b200 as vf
    L = vf.load()
    # cudaMemcpy through the library's helper keeps the tests free of a second CUDA binding
    ctx = _helper_ctx()
    ctx.check(L.vfkv_memcpy_d2h(ctx.handle, out.ctypes.data, addr, nbytes, None))
    ctx.check(L.vfkv_stream_synchronize(ctx.handle, None))
    return out


def dev_write_bytes(addr: int, data: np.ndarray):
    import vulkanforge_b200 as vf
    L = vf.load()
    ctx = _helper_ctx()
    data = np.ascontiguousarray(data)
    ctx.check(L.vfkv_memcpy_h2d(ctx.handle, addr, data.ctypes.data, data.nbytes, None))
    ctx.check(L.vfkv_stream_synchronize(ctx.handle, None))


class NcclComm:
    """A raw NCCL communicator made with ctypes from the NCCL library the process has loaded (the
    one PyTorch brings): what a host without PyTorch would hand to vfkv_attend_allgather.
    ``exchange_id`` gets rank 0's 128-byte unique id and returns it on every rank."""

    def __init__(self, world: int, rank: int, exchange_id):
        import ctypes as C
        import torch  # noqa: F401  (loads libnccl.so.2)

        class UniqueId(C.Structure):
            _fields_ = [("internal", C.c_char * 128)]

        self._nccl = C.CDLL("libnccl.so.2")
        uid = UniqueId()
        if rank == 0:
            rc = self._nccl.ncclGetUniqueId(C.byref(uid))
            assert rc == 0, rc
        raw = exchange_id(bytes(C.string_at(C.addressof(uid), 128)))
        C.memmove(C.addressof(uid), raw, 128)
        self._nccl.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, UniqueId, C.c_int]
        comm = C.c_void_p()
        rc = self._nccl.ncclCommInitRank(C.byref(comm), world, uid, rank)
        assert rc == 0, rc
        self.handle = comm.value

    def destroy(self):
        import ctypes as C
        self._nccl.ncclCommDestroy.argtypes = [C.c_void_p]
        self._nccl.ncclCommDestroy(self.handle)


_CTX = None


def _helper_ctx():
    global _CTX
    if _CTX is None:
        import vulkanforge_b200 as vf
        _CTX = vf.Context(0)
    return _CTX


def rel_err(a: np.ndarray, b: np.ndarray) -> float:
    """max |a-b| relative to max |b| (the reference's 'rel-to-max' measure, tests/coopmat_fa_gemma.rs:260)."""
    return float(np.max(np.abs(a - b)) / max(float(np.max(np.abs(b))), 1e-30))


def encode_cache(x: np.ndarray, dtype: int) -> np.ndarray:
    """f32 [..] -> cache elements of `dtype`, same shape, via the oracle's store ops."""
    return oracle.store(x, dtype).reshape(x.shape)


# name, n_q_heads, n_kv_heads, head_dim, seq_len, kv_start, cache dtype, softcap
GOLDEN_CASES = [
    ("f16_32_8_128_L300", 32, 8, 128, 300, 0, oracle.F16, 0.0),
    ("fp8_32_8_128_L333", 32, 8, 128, 333, 0, oracle.F8, 0.0),
    ("f32_4_2_64_L70", 4, 2, 64, 70, 0, oracle.F32, 0.0),
    ("f16_16_8_256_L500_win", 16, 8, 256, 500, 500 - 128, oracle.F16, 50.0),
    ("fp8_64_8_128_L257", 64, 8, 128, 257, 0, oracle.F8, 0.0),
]


def golden_inputs(i: int):
    """Seeded (q, k_cache, v_cache) of golden case i; the cache arrays hold encoded elements."""
    _, hq, hkv, d, L, _, dt, _ = GOLDEN_CASES[i]
    rng = np.random.default_rng(1000 + i)
    q = rng.standard_normal((hq, d), dtype=np.float32)
    gen = (lambda: kv_values(rng, (L, hkv, d))) if dt == oracle.F8 else \
          (lambda: rng.standard_normal((L, hkv, d), dtype=np.float32))
    k, v = gen(), gen()
    return q, encode_cache(k, dt), encode_cache(v, dt)
