"""Host-side mirror of VulkanForge's ``KvCache`` over the C ABI.

Names, argument meaning and error behaviour follow
``src/backend/vulkan/kv_cache.rs`` so that tests written against the reference
read the same here.  All arithmetic and all device work happen inside
``libvfkv.so``; this module only marshals arguments.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass
from typing import Optional, Sequence

from . import _lib


class VfkvError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"vfkv status {status} ({_status_text(status)}): {message}")
        self.status = status


def _status_text(status: int) -> str:
    return _lib.load().vfkv_status_string(status).decode()


# status codes of include/vfkv.h
OK, ERR_INVALID, ERR_OVERFLOW, ERR_OOM, ERR_CUDA, ERR_UNSUPPORTED, ERR_TIMEOUT, ERR_PRECISION = range(8)


class KvDtype(enum.IntEnum):
    """kv_cache.rs:42-74"""
    F32 = 0
    F16 = 1
    F8 = 2

    def element_size(self) -> int:
        return int(_lib.load().vfkv_dtype_element_size(int(self)))

    def label(self) -> str:
        return {0: "FP32", 1: "FP16", 2: "FP8"}[int(self)]


def kv_dtype_from_env() -> KvDtype:
    """kv_cache.rs:85-101"""
    return KvDtype(_lib.load().vfkv_dtype_from_env())


def guard_kv_precision(is_gemma4_moe: bool, kv_dtype: KvDtype, force: bool = False) -> None:
    """kv_cache.rs:118-151; raises VfkvError(ERR_PRECISION) where the reference returns Err."""
    rc = _lib.load().vfkv_guard_kv_precision(int(is_gemma4_moe), int(kv_dtype), int(force))
    if rc != OK:
        raise VfkvError(rc, "gemma-4-MoE requires VULKANFORGE_KV_FP8=1 (non-FP8 KV is known-broken)")


def _u32_array(values: Optional[Sequence[int]]):
    if values is None:
        return None
    return (C.c_uint32 * len(values))(*values)


def kv_bytes_per_token(n_layers, n_kv_heads, head_dim, per_layer_head_dim, per_layer_n_kv_heads,
                       elem_size) -> int:
    """kv_cache.rs:186-202"""
    return int(_lib.load().vfkv_kv_bytes_per_token(
        n_layers, n_kv_heads, head_dim, _u32_array(per_layer_head_dim),
        _u32_array(per_layer_n_kv_heads), elem_size))


def sliding_kv_start(position: int, window: int) -> int:
    """forward/arch/gemma4.rs:59-73 for a sliding layer"""
    return int(_lib.load().vfkv_sliding_kv_start(position, window))


@dataclass
class KvCacheConfig:
    """kv_cache.rs:153-176 plus n_slots / scale_mode."""
    n_layers: int
    n_kv_heads: int
    head_dim: int
    max_seq_len: int
    per_layer_head_dim: Optional[Sequence[int]] = None
    per_layer_n_kv_heads: Optional[Sequence[int]] = None
    n_slots: int = 1
    scale_mode: int = 0


def ptr(x) -> Optional[int]:
    """Device or host address of a tensor / array / int; None stays None."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if hasattr(x, "ctypes"):
        return x.ctypes.data
    raise TypeError(f"cannot take the address of {type(x)!r}")


class Context:
    """One per GPU; the stand-in for the device + pipeline-registry pair of the reference."""

    def __init__(self, device_ordinal: int = 0):
        self._lib = _lib.load()
        h = C.c_void_p()
        rc = self._lib.vfkv_ctx_create(device_ordinal, C.byref(h))
        if rc != OK:
            raise VfkvError(rc, f"vfkv_ctx_create(device {device_ordinal}) failed")
        self.handle = h
        self.device = device_ordinal

    def check(self, rc: int) -> None:
        if rc != OK:
            raise VfkvError(rc, self._lib.vfkv_last_error(self.handle).decode())

    def poll(self, stream=None) -> None:
        self.check(self._lib.vfkv_ctx_poll(self.handle, stream))

    def set_attn_impl(self, impl: int) -> None:
        self.check(self._lib.vfkv_ctx_set_attn_impl(self.handle, impl))

    def set_cluster_merge(self, on: bool) -> None:
        """Merge the splits of a (sequence, kv-head) inside a thread-block cluster where possible."""
        self.check(self._lib.vfkv_ctx_set_cluster_merge(self.handle, int(on)))

    def set_dependent_launch(self, mode: int) -> None:
        self.check(self._lib.vfkv_ctx_set_dependent_launch(self.handle, mode))

    def set_attn_tuning(self, warps: int, stages: int) -> None:
        self.check(self._lib.vfkv_ctx_set_attn_tuning(self.handle, warps, stages))

    def set_merge_wait_ms(self, ms: int) -> None:
        """Time limit of the merging CTA's wait for the other splits' partials."""
        self.check(self._lib.vfkv_ctx_set_merge_wait_ms(self.handle, ms))

    def debug_fail_split(self, split=None) -> None:
        """Test hook: one CTA of later attention launches acts as if its TMA wait had run out."""
        self.check(self._lib.vfkv_ctx_debug_fail_split(self.handle, 0xFFFFFFFF if split is None else split))

    def launch_count(self) -> int:
        return int(self._lib.vfkv_ctx_launch_count(self.handle))

    def destroy(self) -> None:
        if self.handle:
            self._lib.vfkv_ctx_destroy(self.handle)
            self.handle = None


class Workspace:
    """fa_scratch_out / _max / _sum of forward/setup.rs:203-230."""

    def __init__(self, ctx: Context, max_seqs: int, n_q_heads: int, head_dim: int, max_splits: int):
        self.ctx = ctx
        h = C.c_void_p()
        ctx.check(ctx._lib.vfkv_workspace_create(ctx.handle, max_seqs, n_q_heads, head_dim, max_splits,
                                                 C.byref(h)))
        self.handle = h

    def bytes(self) -> int:
        return int(self.ctx._lib.vfkv_workspace_bytes(self.handle))

    def reset(self, stream=None) -> None:
        """Zeroes the split tickets and partial tags (stream-ordered)."""
        self.ctx.check(self.ctx._lib.vfkv_workspace_reset(self.handle, stream))

    def destroy(self) -> None:
        if self.handle:
            self.ctx._lib.vfkv_workspace_destroy(self.handle)
            self.handle = None


def longest_common_prefix(a, b) -> int:
    """src/server/state.rs:49-51 over two token-id sequences."""
    import numpy as np
    a = np.ascontiguousarray(a, dtype=np.uint32)
    b = np.ascontiguousarray(b, dtype=np.uint32)
    pa = a.ctypes.data_as(C.POINTER(C.c_uint32))
    pb = b.ctypes.data_as(C.POINTER(C.c_uint32))
    return int(_lib.load().vfkv_longest_common_prefix(pa, a.size, pb, b.size))


AUTO_CTX_BOUNDS = ("VRAM", "model max context", "hardware limit", "sane cap")   # CtxBound::label, auto_ctx.rs:72-80


def compute_auto_ctx(free_bytes: int, weight_bytes: int, reserve_bytes: int, kv_bytes_per_token_: int,
                     model_max_ctx: int, hw_cap: int, sane_cap: int = 32768):
    """src/server/auto_ctx.rs:107-141 -> (ctx, bound label, bytes available for KV)."""
    ctx, bound, avail = C.c_uint32(), C.c_uint32(), C.c_uint64()
    rc = _lib.load().vfkv_compute_auto_ctx(free_bytes, weight_bytes, reserve_bytes, kv_bytes_per_token_, model_max_ctx,
                                      hw_cap, sane_cap, C.byref(ctx), C.byref(bound), C.byref(avail))
    if rc:
        raise VfkvError(rc, "vfkv_compute_auto_ctx")
    return ctx.value, AUTO_CTX_BOUNDS[bound.value], avail.value


KV_OWN, KV_PUBLISH_SLIDING, KV_PUBLISH_FULL, KV_SUBSCRIBE_SLIDING, KV_SUBSCRIBE_FULL = range(5)


def gemma4_kv_read_layer(kv_source, layer: int) -> int:
    """src/backend/vulkan/forward/arch/gemma4.rs:27-49 over a list of Gemma4KvSource codes."""
    import numpy as np
    src = np.ascontiguousarray(kv_source, dtype=np.uint32)
    return int(_lib.load().vfkv_gemma4_kv_read_layer(src.ctypes.data_as(C.POINTER(C.c_uint32)), src.size, layer))


class PeerExchange:
    """One GPU's end of the peer exchange of (m, l, o) partials used by position sharding
    (``vfkv_exchange_*``; no counterpart in the reference)."""

    def __init__(self, ctx: Context, world: int, rank: int, n_rows: int, head_dim: int):
        self.ctx, self.world, self.rank = ctx, world, rank
        h = C.c_void_p()
        ctx.check(ctx._lib.vfkv_exchange_create(ctx.handle, world, rank, n_rows, head_dim, C.byref(h)))
        self.handle = h

    def bytes(self) -> int:
        return int(self.ctx._lib.vfkv_exchange_bytes(self.handle))

    def local_ptr(self) -> int:
        return int(self.ctx._lib.vfkv_exchange_local_ptr(self.handle) or 0)

    def export_handle(self) -> bytes:
        buf = (C.c_uint8 * 64)()
        self.ctx.check(self.ctx._lib.vfkv_exchange_export(self.handle, buf))
        return bytes(buf)

    def import_handle(self, rank: int, handle: bytes) -> None:
        buf = (C.c_uint8 * 64).from_buffer_copy(handle)
        self.ctx.check(self.ctx._lib.vfkv_exchange_import(self.handle, rank, buf))

    def set_peer(self, rank: int, device_ptr: int) -> None:
        self.ctx.check(self.ctx._lib.vfkv_exchange_set_peer(self.handle, rank, C.c_void_p(device_ptr)))

    def set_timeout_ms(self, ms: int) -> None:
        self.ctx.check(self.ctx._lib.vfkv_exchange_set_timeout_ms(self.handle, ms))

    def ready(self) -> bool:
        return bool(self.ctx._lib.vfkv_exchange_ready(self.handle))

    def connect(self, group=None) -> None:
        """One process per GPU: swaps CUDA IPC handles over ``torch.distributed`` and ends with a
        barrier, after which pushes may start."""
        import torch.distributed as dist
        handles = [None] * self.world
        dist.all_gather_object(handles, self.export_handle(), group=group)
        for r, h in enumerate(handles):
            if r != self.rank:
                self.import_handle(r, h)
        dist.barrier(group=group)

    def destroy(self) -> None:
        if self.handle:
            self.ctx._lib.vfkv_exchange_destroy(self.handle)
            self.handle = None


class KvCache:
    """kv_cache.rs:204-499.  ``KvCache.new`` mirrors ``KvCache::new``; the dtype is explicit
    (pass ``kv_dtype_from_env()`` for the reference's environment selection)."""

    def __init__(self, ctx: Context, config: KvCacheConfig, kv_dtype: KvDtype):
        self.ctx = ctx
        self.config = config
        self.kv_dtype = KvDtype(kv_dtype)
        L = ctx._lib
        for name, v in (("per_layer_head_dim", config.per_layer_head_dim),
                        ("per_layer_n_kv_heads", config.per_layer_n_kv_heads)):
            if v is not None and len(v) != config.n_layers:
                raise VfkvError(ERR_INVALID, f"{name} length must equal n_layers")
        self._plhd = _u32_array(config.per_layer_head_dim)
        self._plkv = _u32_array(config.per_layer_n_kv_heads)
        cfg = _lib.CacheConfig(config.n_layers, config.n_kv_heads, config.head_dim, config.max_seq_len,
                               int(kv_dtype),
                               C.cast(self._plhd, _lib.pu32) if self._plhd is not None else None,
                               C.cast(self._plkv, _lib.pu32) if self._plkv is not None else None,
                               config.n_slots, config.scale_mode)
        h = C.c_void_p()
        ctx.check(L.vfkv_cache_create(ctx.handle, C.byref(cfg), C.byref(h)))
        self.handle = h

    @classmethod
    def new(cls, ctx: Context, config: KvCacheConfig, kv_dtype: Optional[KvDtype] = None) -> "KvCache":
        return cls(ctx, config, kv_dtype_from_env() if kv_dtype is None else kv_dtype)

    # ---- public fields of the reference ----
    @property
    def k_buffer(self) -> int:
        return int(self.ctx._lib.vfkv_cache_k_ptr(self.handle) or 0)

    @property
    def v_buffer(self) -> int:
        return int(self.ctx._lib.vfkv_cache_v_ptr(self.handle) or 0)

    @property
    def k_scales(self) -> int:
        return int(self.ctx._lib.vfkv_cache_k_scale_ptr(self.handle) or 0)

    @property
    def v_scales(self) -> int:
        return int(self.ctx._lib.vfkv_cache_v_scale_ptr(self.handle) or 0)

    @property
    def current_seq_len(self) -> int:
        return self.seq_len(0)

    @current_seq_len.setter
    def current_seq_len(self, n: int) -> None:
        self.set_seq_len(0, n)

    def seq_len(self, slot: int) -> int:
        out = C.c_uint32()
        self.ctx.check(self.ctx._lib.vfkv_cache_seq_len(self.handle, slot, C.byref(out)))
        return out.value

    def set_seq_len(self, slot: int, n: int) -> None:
        self.ctx.check(self.ctx._lib.vfkv_cache_set_seq_len(self.handle, slot, n))

    # ---- accessors (same names as the reference) ----
    def bytes_per_buffer(self) -> int:
        return int(self.ctx._lib.vfkv_cache_bytes_per_buffer(self.handle))

    def head_dim_for(self, layer: int) -> int:
        return int(self.ctx._lib.vfkv_cache_head_dim_for(self.handle, layer))

    def kv_heads_for(self, layer: int) -> int:
        return int(self.ctx._lib.vfkv_cache_kv_heads_for(self.handle, layer))

    def layer_offset_elems(self, layer: int) -> int:
        return int(self.ctx._lib.vfkv_cache_layer_offset_elems(self.handle, layer))

    def layer_offset_bytes(self, layer: int) -> int:
        return int(self.ctx._lib.vfkv_cache_layer_offset_bytes(self.handle, layer))

    def pos_offset_bytes(self, layer: int, pos: int) -> int:
        return int(self.ctx._lib.vfkv_cache_pos_offset_bytes(self.handle, layer, pos))

    def slot_offset_bytes(self, layer: int, slot: int) -> int:
        return int(self.ctx._lib.vfkv_cache_slot_offset_bytes(self.handle, layer, slot))

    def row_bytes(self, layer: int) -> int:
        return int(self.ctx._lib.vfkv_cache_row_bytes(self.handle, layer))

    def layer_size_bytes(self, layer: int) -> int:
        return int(self.ctx._lib.vfkv_cache_layer_size_bytes(self.handle, layer))

    def is_fp8(self) -> bool:
        return bool(self.ctx._lib.vfkv_cache_is_fp8(self.handle))

    def is_fp16(self) -> bool:
        return bool(self.ctx._lib.vfkv_cache_is_fp16(self.handle))

    def reset(self, slot: int = 0) -> None:
        self.ctx.check(self.ctx._lib.vfkv_cache_reset(self.handle, slot))

    def reuse_prepare(self, cached_tokens, full_tokens, reuse: bool = True, slot: int = 0) -> int:
        """The KV-prepare step of ServerSession::generate_reuse (src/server/state.rs:199-229):
        returns the start position k; rows [0, k) are kept and the counter is set to k."""
        import numpy as np
        a = np.ascontiguousarray(cached_tokens, dtype=np.uint32)
        b = np.ascontiguousarray(full_tokens, dtype=np.uint32)
        k = C.c_uint32()
        p32 = C.POINTER(C.c_uint32)
        self.ctx.check(self.ctx._lib.vfkv_kv_reuse_prepare(self.handle, slot, a.ctypes.data_as(p32), a.size,
                                                           b.ctypes.data_as(p32), b.size, int(reuse), C.byref(k)))
        return k.value

    def invalidate(self, slot: int = 0) -> None:
        """kv_invalidate (state.rs:284-287)."""
        self.ctx.check(self.ctx._lib.vfkv_kv_invalidate(self.handle, slot))

    def zero_fill(self, stream=None) -> None:
        self.ctx.check(self.ctx._lib.vfkv_cache_zero_fill(self.handle, stream))

    def zero_layer(self, layer: int, stream=None) -> None:
        self.ctx.check(self.ctx._lib.vfkv_cache_zero_layer(self.handle, layer, stream))

    def destroy(self) -> None:
        if self.handle:
            self.ctx._lib.vfkv_cache_destroy(self.handle)
            self.handle = None
