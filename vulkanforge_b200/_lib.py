"""ctypes declarations for ``libvfkv.so`` (the C ABI of ``include/vfkv.h``).

There is no CPU fallback: if the shared object is missing or a symbol cannot be
resolved, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libvfkv.so")

u32, u64, i32, f32, vp = C.c_uint32, C.c_uint64, C.c_int32, C.c_float, C.c_void_p
pu32 = C.POINTER(C.c_uint32)


class CacheConfig(C.Structure):
    _fields_ = [("n_layers", u32), ("n_kv_heads", u32), ("head_dim", u32), ("max_seq_len", u32),
                ("dtype", u32), ("per_layer_head_dim", pu32), ("per_layer_n_kv_heads", pu32),
                ("n_slots", u32), ("scale_mode", u32)]


class RopeParams(C.Structure):
    """vfkv_rope_params (include/vfkv_next.h)."""
    _fields_ = [("n_dims", u32), ("freq_base", f32), ("freq_scale", f32)]


# name -> (restype, argtypes); kept in the order of include/vfkv.h, then include/vfkv_next.h
SIGNATURES = {
    "vfkv_ctx_create": (i32, [i32, C.POINTER(vp)]),
    "vfkv_ctx_destroy": (i32, [vp]),
    "vfkv_last_error": (C.c_char_p, [vp]),
    "vfkv_status_string": (C.c_char_p, [i32]),
    "vfkv_abi_version": (u32, []),
    "vfkv_ctx_poll": (i32, [vp, vp]),
    "vfkv_cache_create": (i32, [vp, C.POINTER(CacheConfig), C.POINTER(vp)]),
    "vfkv_cache_destroy": (i32, [vp]),
    "vfkv_cache_zero_fill": (i32, [vp, vp]),
    "vfkv_cache_zero_layer": (i32, [vp, u32, vp]),
    "vfkv_cache_reset": (i32, [vp, u32]),
    "vfkv_cache_seq_len": (i32, [vp, u32, pu32]),
    "vfkv_cache_set_seq_len": (i32, [vp, u32, u32]),
    "vfkv_cache_head_dim_for": (u32, [vp, u32]),
    "vfkv_cache_kv_heads_for": (u32, [vp, u32]),
    "vfkv_cache_row_bytes": (u64, [vp, u32]),
    "vfkv_cache_layer_size_bytes": (u64, [vp, u32]),
    "vfkv_cache_layer_offset_bytes": (u64, [vp, u32]),
    "vfkv_cache_layer_offset_elems": (u64, [vp, u32]),
    "vfkv_cache_pos_offset_bytes": (u64, [vp, u32, u32]),
    "vfkv_cache_slot_offset_bytes": (u64, [vp, u32, u32]),
    "vfkv_cache_bytes_per_buffer": (u64, [vp]),
    "vfkv_cache_dtype": (u32, [vp]),
    "vfkv_cache_is_fp8": (i32, [vp]),
    "vfkv_cache_is_fp16": (i32, [vp]),
    "vfkv_cache_k_ptr": (vp, [vp]),
    "vfkv_cache_v_ptr": (vp, [vp]),
    "vfkv_cache_k_scale_ptr": (vp, [vp]),
    "vfkv_cache_v_scale_ptr": (vp, [vp]),
    "vfkv_kv_bytes_per_token": (u64, [u32, u32, u32, pu32, pu32, u64]),
    "vfkv_dtype_element_size": (u64, [u32]),
    "vfkv_dtype_from_env": (u32, []),
    "vfkv_guard_kv_precision": (i32, [i32, u32, i32]),
    "vfkv_sliding_kv_start": (u32, [u32, u32]),
    "vfkv_kv_store_fp8": (i32, [vp, vp, vp, u32, u64, vp]),
    "vfkv_kv_copy_fp16": (i32, [vp, vp, vp, u32, u64, vp]),
    "vfkv_kv_fp8_to_f16": (i32, [vp, vp, vp, u64, vp]),
    "vfkv_flash_attn_split_reduce": (i32, [vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, f32,
                                           u32, f32, u32, vp]),
    "vfkv_flash_attn_split_reduce_noalloc": (i32, [vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, f32, u32, f32,
                                                   u32, vp]),
    "vfkv_noalloc_last_error": (C.c_char_p, []),
    "vfkv_noalloc_scratch_bytes": (u64, []),
    "vfkv_workspace_create": (i32, [vp, u32, u32, u32, u32, C.POINTER(vp)]),
    "vfkv_workspace_destroy": (i32, [vp]),
    "vfkv_workspace_bytes": (u64, [vp]),
    "vfkv_workspace_reset": (i32, [vp, vp]),
    "vfkv_append": (i32, [vp, u32, vp, vp, u32, u32, u32, vp]),
    "vfkv_append_batch": (i32, [vp, u32, vp, vp, vp, vp, u32, vp]),
    "vfkv_fp8_to_f16": (i32, [vp, u32, u32, u32, vp, vp, vp]),
    "vfkv_attend": (i32, [vp, vp, u32, u32, vp, vp, u32, u32, u32, u32, f32, f32, u32, vp]),
    "vfkv_attend_batch": (i32, [vp, vp, u32, u32, vp, vp, u32, vp, vp, vp, u32, u32, f32, f32, u32, vp]),
    "vfkv_decode_step": (i32, [vp, vp, u32, vp, vp, vp, vp, u32, vp, vp, u32, u32, u32, f32, f32, u32, vp]),
    "vfkv_decode_token": (i32, [vp, vp, vp, vp, vp, vp, u32, vp, vp, u32, u32, vp, f32, f32, u32, vp]),
    "vfkv_decode_token_host": (i32, [vp, vp, vp, vp, vp, vp, u32, vp, vp, u32, vp, f32, f32, u32, vp]),
    "vfkv_decode_token_host_submit": (i32, [vp, vp, vp, vp, vp, vp, u32, vp, vp, u32, vp, f32, f32, u32, vp,
                                            C.POINTER(u64)]),
    "vfkv_decode_token_host_wait": (i32, [vp, u64]),
    "vfkv_attend_partial": (i32, [vp, vp, u32, u32, vp, u32, u32, u32, u32, f32, f32, u32, vp, vp, vp, vp]),
    "vfkv_merge_partials": (i32, [vp, vp, vp, vp, u32, u32, u32, vp, vp]),
    "vfkv_merge_partials_packed": (i32, [vp, vp, u32, u32, u32, vp, vp]),
    "vfkv_shard_owner": (u32, [u32, u32, u64]),
    "vfkv_shard_local_pos": (u64, [u32, u32, u64]),
    "vfkv_shard_local_len": (u64, [u32, u32, u64, u32]),
    "vfkv_shard_local_capacity": (u64, [u32, u32, u64]),
    "vfkv_assign_sequences": (i32, [pu32, u32, u32, pu32]),
    "vfkv_shard_kv_heads": (i32, [u32, u32, u32, pu32, pu32]),
    "vfkv_append_sharded": (i32, [vp, u32, vp, vp, u32, u32, u32, u32, u32, u32, vp]),
    "vfkv_attend_allgather": (i32, [vp, vp, vp, u32, u32, u32, u32, vp, u32, u32, u32, u32, f32, f32, u32, vp, vp, vp]),
    "vfkv_exchange_create": (i32, [vp, u32, u32, u32, u32, C.POINTER(vp)]),
    "vfkv_exchange_destroy": (None, [vp]),
    "vfkv_exchange_bytes": (u64, [vp]),
    "vfkv_exchange_local_ptr": (vp, [vp]),
    "vfkv_exchange_export": (i32, [vp, vp]),
    "vfkv_exchange_import": (i32, [vp, u32, vp]),
    "vfkv_exchange_set_peer": (i32, [vp, u32, vp]),
    "vfkv_exchange_set_timeout_ms": (i32, [vp, u32]),
    "vfkv_exchange_ready": (u32, [vp]),
    "vfkv_attend_push": (i32, [vp, vp, vp, u32, u32, vp, vp, vp, u32, u32, u32, u32, f32, f32, u32, vp]),
    "vfkv_exchange_merge": (i32, [vp, vp, vp]),
    "vfkv_attend_exchange": (i32, [vp, vp, vp, u32, u32, vp, vp, vp, u32, u32, u32, u32, f32, f32, u32, vp, vp]),
    "vfkv_malloc": (i32, [vp, u64, C.POINTER(vp)]),
    # ---- include/vfkv_next.h ----
    "vfkv_flash_attn": (i32, [vp, u32, u32, vp, vp, u32, u32, u32, u32, f32, f32, vp]),
    "vfkv_scalar_attn": (i32, [vp, vp, u32, u32, vp, vp, u32, u32, u32, u32, f32, f32, vp]),
    "vfkv_scalar_attn_uses_split": (u32, [u32]),
    "vfkv_attend_prefill": (i32, [vp, u32, u32, vp, vp, u32, u32, u32, u32, u32, u32, u32, f32, f32, vp]),
    "vfkv_rope_append": (i32, [vp, u32, vp, vp, u32, u32, u32, C.POINTER(RopeParams), vp, vp]),
    "vfkv_rope_append_batch": (i32, [vp, u32, vp, vp, vp, vp, u32, C.POINTER(RopeParams), vp, vp]),
    "vfkv_rope_neox": (i32, [vp, vp, vp, u32, u32, u32, vp, u32, C.POINTER(RopeParams), vp]),
    "vfkv_longest_common_prefix": (u64, [pu32, u64, pu32, u64]),
    "vfkv_kv_reuse_prepare": (i32, [vp, u32, pu32, u64, pu32, u64, i32, pu32]),
    "vfkv_kv_invalidate": (i32, [vp, u32]),
    "vfkv_compute_auto_ctx": (i32, [u64, u64, u64, u64, u32, u32, u32, pu32, pu32, C.POINTER(u64)]),
    "vfkv_gemma4_kv_read_layer": (u32, [pu32, u32, u32]),
    "vfkv_free": (i32, [vp, vp]),
    "vfkv_malloc_host": (i32, [vp, u64, C.POINTER(vp)]),
    "vfkv_free_host": (i32, [vp, vp]),
    "vfkv_memcpy_h2d": (i32, [vp, vp, vp, u64, vp]),
    "vfkv_memcpy_d2h": (i32, [vp, vp, vp, u64, vp]),
    "vfkv_memset": (i32, [vp, vp, i32, u64, vp]),
    "vfkv_stream_synchronize": (i32, [vp, vp]),
    "vfkv_ctx_set_attn_impl": (i32, [vp, u32]),
    "vfkv_ctx_set_attn_tuning": (i32, [vp, u32, u32]),
    "vfkv_ctx_set_dependent_launch": (i32, [vp, u32]),
    "vfkv_ctx_set_cluster_merge": (i32, [vp, u32]),
    "vfkv_ctx_set_merge_wait_ms": (i32, [vp, u32]),
    "vfkv_ctx_debug_fail_split": (i32, [vp, u32]),
    "vfkv_ctx_set_trace_buffer": (i32, [vp, vp]),
    "vfkv_ctx_set_trace_ring": (i32, [vp, u32]),
    "vfkv_ctx_launch_count": (u64, [vp]),
    "vfkv_profile_enable": (i32, [vp, i32]),
    "vfkv_profile_collect": (i32, [vp, u32, C.POINTER(u64), C.POINTER(C.c_double), C.POINTER(C.c_double), i32]),
}

_lib = None


def load() -> C.CDLL:
    """Loads libvfkv.so and binds every declared symbol; raises if anything is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m vulkanforge_b200.build` "
            "(nvcc, sm_100a). There is no CPU fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is not exported
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib
