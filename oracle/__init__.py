"""ctypes/numpy front end of the CPU oracle (``libvfkv_oracle.so``).

TEST INFRASTRUCTURE ONLY: imported by the test-suite, by the smoke check and by
the benchmark's CPU-baseline leg.  The product package never imports it.

The parity status of each function is stated in ``vfkv_oracle.h``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libvfkv_oracle.so")

F32, F16, F8 = 0, 1, 2
ELEM_SIZE = {F32: 4, F16: 2, F8: 1}
NP_DTYPE = {F32: np.float32, F16: np.uint16, F8: np.uint8}


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it; returns the .so path."""
    src = [os.path.join(_HERE, f) for f in ("vfkv_oracle.c", "vfkv_oracle.h", "Makefile")]
    stale = (not os.path.exists(_SO)) or any(os.path.getmtime(s) > os.path.getmtime(_SO) for s in src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "libvfkv_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _declare(_lib)
    return _lib


class Layout(C.Structure):
    _fields_ = [("n_layers", C.c_uint32), ("n_kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
                ("max_seq_len", C.c_uint32), ("dtype", C.c_uint32),
                ("per_layer_head_dim", C.POINTER(C.c_uint32)),
                ("per_layer_n_kv_heads", C.POINTER(C.c_uint32))]


def _declare(L: C.CDLL) -> None:
    u8, u16, u32, u64, f32 = C.c_uint8, C.c_uint16, C.c_uint32, C.c_uint64, C.c_float
    vp = C.c_void_p
    L.vfo_f32_to_e4m3.restype, L.vfo_f32_to_e4m3.argtypes = u8, [f32]
    L.vfo_e4m3_to_f32.restype, L.vfo_e4m3_to_f32.argtypes = f32, [u8]
    L.vfo_f32_to_f16.restype, L.vfo_f32_to_f16.argtypes = u16, [f32]
    L.vfo_f16_to_f32.restype, L.vfo_f16_to_f32.argtypes = f32, [u16]
    L.vfo_f32_bits_to_e4m3_range.restype, L.vfo_f32_bits_to_e4m3_range.argtypes = None, [u32, u64, vp]
    L.vfo_f32_bits_to_f16_range.restype, L.vfo_f32_bits_to_f16_range.argtypes = None, [u32, u64, vp]
    L.vfo_kv_store_fp8.restype, L.vfo_kv_store_fp8.argtypes = None, [vp, u32, vp]
    L.vfo_kv_copy_fp16.restype, L.vfo_kv_copy_fp16.argtypes = None, [vp, u32, vp]
    L.vfo_kv_fp8_to_f16.restype, L.vfo_kv_fp8_to_f16.argtypes = None, [vp, u32, vp]
    L.vfo_kv_store_fp8_scaled.restype, L.vfo_kv_store_fp8_scaled.argtypes = None, [vp, u32, u32, vp, vp]
    lp = C.POINTER(Layout)
    L.vfo_elem_size.restype, L.vfo_elem_size.argtypes = u64, [u32]
    for name in ("vfo_head_dim_for", "vfo_kv_heads_for"):
        getattr(L, name).restype, getattr(L, name).argtypes = u32, [lp, u32]
    for name in ("vfo_row_bytes", "vfo_layer_size_bytes", "vfo_layer_offset_bytes"):
        getattr(L, name).restype, getattr(L, name).argtypes = u64, [lp, u32]
    L.vfo_pos_offset_bytes.restype, L.vfo_pos_offset_bytes.argtypes = u64, [lp, u32, u32]
    L.vfo_bytes_per_buffer.restype, L.vfo_bytes_per_buffer.argtypes = C.c_int, [lp, C.POINTER(u64)]
    L.vfo_kv_bytes_per_token.restype = u64
    L.vfo_kv_bytes_per_token.argtypes = [u32, u32, u32, C.POINTER(u32), C.POINTER(u32), u64]
    L.vfo_sliding_kv_start.restype, L.vfo_sliding_kv_start.argtypes = u32, [u32, u32]
    L.vfo_rope_neox.restype, L.vfo_rope_neox.argtypes = None, [vp, u32, u32, u32, u32, f32]
    L.vfo_attention_ref.restype = None
    L.vfo_attention_ref.argtypes = [vp, vp, vp, u32, u32, u32, u32, u32, u32, f32, f32, vp, vp, vp]
    L.vfo_flash_attn_split.restype = None
    L.vfo_flash_attn_split.argtypes = [vp, vp, vp, u32, u32, u32, u32, u32, u32, f32, u32, u32, vp, vp, vp]
    L.vfo_flash_attn_reduce.restype = None
    L.vfo_flash_attn_reduce.argtypes = [vp, vp, vp, u32, u32, u32, vp]
    L.vfo_decode_step.restype = None
    L.vfo_decode_step.argtypes = [vp, vp, vp, vp, vp, u32, u32, u64, u32, u32, u32, vp, vp, f32, f32, vp]
    L.vfo_num_threads.restype, L.vfo_num_threads.argtypes = C.c_int, []
    L.vfo_set_num_threads.restype, L.vfo_set_num_threads.argtypes = None, [C.c_int]


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


# ---- scalar codecs ---------------------------------------------------------
def f32_to_e4m3(x: float) -> int:
    return int(lib().vfo_f32_to_e4m3(C.c_float(x)))


def e4m3_to_f32(b: int) -> float:
    return float(lib().vfo_e4m3_to_f32(C.c_uint8(b)))


def f32_to_f16_bits(x: float) -> int:
    return int(lib().vfo_f32_to_f16(C.c_float(x)))


def e4m3_range(first_bits: int, count: int) -> np.ndarray:
    out = np.empty(count, np.uint8)
    lib().vfo_f32_bits_to_e4m3_range(first_bits, count, _p(out))
    return out


def f16_range(first_bits: int, count: int) -> np.ndarray:
    out = np.empty(count, np.uint16)
    lib().vfo_f32_bits_to_f16_range(first_bits, count, _p(out))
    return out


# ---- ops -------------------------------------------------------------------
def kv_store_fp8(src: np.ndarray) -> np.ndarray:
    src = _c(src, np.float32).ravel()
    out = np.empty((src.size + 3) // 4 * 4, np.uint8)
    lib().vfo_kv_store_fp8(_p(src), src.size, _p(out))
    return out


def kv_copy_fp16(src: np.ndarray) -> np.ndarray:
    src = _c(src, np.float32).ravel()
    out = np.empty((src.size + 1) // 2 * 2, np.uint16)
    lib().vfo_kv_copy_fp16(_p(src), src.size, _p(out))
    return out


def kv_fp8_to_f16(src: np.ndarray) -> np.ndarray:
    src = _c(src, np.uint8).ravel()
    out = np.empty(src.size, np.uint16)
    lib().vfo_kv_fp8_to_f16(_p(src), src.size, _p(out))
    return out


def kv_store_fp8_scaled(src: np.ndarray, n_heads: int, head_dim: int):
    src = _c(src, np.float32).ravel()
    assert src.size == n_heads * head_dim
    out = np.empty(src.size, np.uint8)
    scales = np.empty(n_heads, np.float32)
    lib().vfo_kv_store_fp8_scaled(_p(src), n_heads, head_dim, _p(out), _p(scales))
    return out, scales


def store(src: np.ndarray, dtype: int) -> np.ndarray:
    """Encode f32 values into cache elements of `dtype` (array of the storage type)."""
    if dtype == F8:
        return kv_store_fp8(src)[: np.asarray(src).size]
    if dtype == F16:
        return kv_copy_fp16(src)[: np.asarray(src).size]
    return _c(src, np.float32).ravel().copy()


def make_layout(n_layers, n_kv_heads, head_dim, max_seq_len, dtype, plhd=None, plkv=None):
    keep = []
    lay = Layout(n_layers, n_kv_heads, head_dim, max_seq_len, dtype, None, None)
    if plhd is not None:
        a = (C.c_uint32 * n_layers)(*plhd)
        keep.append(a)
        lay.per_layer_head_dim = C.cast(a, C.POINTER(C.c_uint32))
    if plkv is not None:
        a = (C.c_uint32 * n_layers)(*plkv)
        keep.append(a)
        lay.per_layer_n_kv_heads = C.cast(a, C.POINTER(C.c_uint32))
    lay._keep = keep
    return lay


def bytes_per_buffer(lay: Layout):
    out = C.c_uint64(0)
    rc = lib().vfo_bytes_per_buffer(C.byref(lay), C.byref(out))
    return None if rc != 0 else out.value


def kv_bytes_per_token(n_layers, n_kv_heads, head_dim, plhd, plkv, elem_size):
    a = (C.c_uint32 * n_layers)(*plhd) if plhd is not None else None
    b = (C.c_uint32 * n_layers)(*plkv) if plkv is not None else None
    return int(lib().vfo_kv_bytes_per_token(n_layers, n_kv_heads, head_dim, a, b, elem_size))


def rope_neox(x: np.ndarray, n_heads: int, head_dim: int, n_dims: int, pos: int, freq_base: float):
    y = _c(x, np.float32).copy()
    lib().vfo_rope_neox(_p(y), n_heads, head_dim, n_dims, pos, C.c_float(freq_base))
    return y


def attention_ref(q, k, v, dtype, n_heads, n_kv_heads, head_dim, seq_len, kv_start=0,
                  scale=None, softcap=0.0, k_scales=None, v_scales=None) -> np.ndarray:
    q = _c(q, np.float32)
    k = _c(k, NP_DTYPE[dtype])
    v = _c(v, NP_DTYPE[dtype])
    if scale is None:
        scale = 1.0 / np.sqrt(np.float32(head_dim))
    ks = None if k_scales is None else _c(k_scales, np.float32)
    vs = None if v_scales is None else _c(v_scales, np.float32)
    out = np.zeros(n_heads * head_dim, np.float32)
    lib().vfo_attention_ref(_p(q), _p(k), _p(v), dtype, n_heads, n_kv_heads, head_dim, seq_len,
                            kv_start, C.c_float(scale), C.c_float(softcap), _p(ks), _p(vs), _p(out))
    return out.reshape(n_heads, head_dim)


def flash_attn_split_reduce(q, k, v, dtype, n_heads, n_kv_heads, head_dim, seq_len, kv_start=0,
                            scale=None, tile=64) -> np.ndarray:
    q = _c(q, np.float32)
    k = _c(k, NP_DTYPE[dtype])
    v = _c(v, NP_DTYPE[dtype])
    if scale is None:
        scale = 1.0 / np.sqrt(np.float32(head_dim))
    n_tiles = (seq_len + tile - 1) // tile
    so = np.zeros(n_heads * n_tiles * head_dim, np.float32)
    sm = np.zeros(n_heads * n_tiles, np.float32)
    ss = np.zeros(n_heads * n_tiles, np.float32)
    out = np.zeros(n_heads * head_dim, np.float32)
    lib().vfo_flash_attn_split(_p(q), _p(k), _p(v), dtype, n_heads, n_kv_heads, head_dim, seq_len,
                               kv_start, C.c_float(scale), tile, n_tiles, _p(so), _p(sm), _p(ss))
    lib().vfo_flash_attn_reduce(_p(so), _p(sm), _p(ss), n_heads, head_dim, n_tiles, _p(out))
    return out.reshape(n_heads, head_dim)


def decode_step(q, k_new, v_new, k_slabs, v_slabs, dtype, n_seqs, slab_positions, n_heads,
                n_kv_heads, head_dim, seq_lens, kv_starts=None, scale=None, softcap=0.0):
    """In-place append into the slabs, then attention; returns out[n_seqs, n_heads, head_dim]."""
    assert k_slabs.flags.c_contiguous and v_slabs.flags.c_contiguous
    q = _c(q, np.float32)
    k_new = _c(k_new, np.float32)
    v_new = _c(v_new, np.float32)
    seq_lens = _c(seq_lens, np.uint32)
    kvs = None if kv_starts is None else _c(kv_starts, np.uint32)
    if scale is None:
        scale = 1.0 / np.sqrt(np.float32(head_dim))
    out = np.zeros((n_seqs, n_heads, head_dim), np.float32)
    lib().vfo_decode_step(_p(q), _p(k_new), _p(v_new), _p(k_slabs), _p(v_slabs), dtype, n_seqs,
                          slab_positions, n_heads, n_kv_heads, head_dim, _p(seq_lens), _p(kvs),
                          C.c_float(scale), C.c_float(softcap), _p(out))
    return out


def num_threads() -> int:
    return int(lib().vfo_num_threads())


def use_all_host_threads() -> int:
    """Sets the OpenMP thread count to the CPUs this process may run on (launchers export
    OMP_NUM_THREADS=1) and returns it."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().vfo_set_num_threads(n)
    return num_threads()


def batch_attention_ref(q, k, v, dtype, n_heads, n_kv_heads, head_dim, m, q_start, n_kv, kv_start=0,
                        window=0, scale=None, softcap=0.0) -> np.ndarray:
    """Causal attention of m queries over the cache rows: cpu_batch_attn_reference
    (tests/correctness.rs:3016-3071) with the kv_start mask of flash_attn_batch.comp:141-147.
    Query i attends over [lo_i, min(q_start + i + 1, n_kv)); lo_i = kv_start, or with
    window != 0 (the build's per-query extension) max(kv_start, causal_len_i - window).
    A query with an empty range yields zeros.  q: [m][n_heads][head_dim]."""
    q = _c(q, np.float32).reshape(m, n_heads, head_dim)
    out = np.zeros((m, n_heads, head_dim), np.float32)
    for i in range(m):
        causal = min(q_start + i + 1, n_kv)
        lo = kv_start
        if window and causal > window:
            lo = max(lo, causal - window)
        lo = min(lo, causal)
        if causal > lo:
            out[i] = attention_ref(q[i], k, v, dtype, n_heads, n_kv_heads, head_dim, causal, lo, scale, softcap)
    return out


def rope_neox_rows(x, n_heads: int, head_dim: int, n_dims: int, positions, freq_base: float) -> np.ndarray:
    """rope_neox applied row by row: x [rows][n_heads][head_dim], positions [rows]."""
    x = _c(x, np.float32).reshape(len(positions), n_heads, head_dim)
    return np.stack([rope_neox(x[r], n_heads, head_dim, n_dims, int(positions[r]), freq_base).reshape(n_heads, head_dim)
                     for r in range(len(positions))])
