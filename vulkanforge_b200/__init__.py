"""vulkanforge_b200 -- VulkanForge's KV-cache hot path on NVIDIA B200.

KV append (FP8 E4M3 / F16 / F32), the FP8->F16 cache read and split-K GQA decode
attention, as hand-written sm_100a CUDA behind the C ABI of ``include/vfkv.h``.
This package is the host-side mirror of the reference's interface for that path
(``KvCache``, the ``run_*`` helpers and the ``step_*`` executor steps).  It has
no CPU fallback: without ``libvfkv.so`` every entry point raises.
"""
from ._lib import LIB_PATH, load
from .forward import CudaForward
from .shard import PositionShards, ShardedSequenceDecoder, all_gather_partials, assign_sequences
from .kv_cache import (Context, KvCache, KvCacheConfig, KvDtype, VfkvError, Workspace, PeerExchange,
                       guard_kv_precision, kv_bytes_per_token, kv_dtype_from_env, ptr,
                       sliding_kv_start, longest_common_prefix, compute_auto_ctx, gemma4_kv_read_layer)

__all__ = ["LIB_PATH", "load", "CudaForward", "PositionShards", "ShardedSequenceDecoder", "all_gather_partials",
           "assign_sequences", "Context", "KvCache", "KvCacheConfig", "KvDtype",
           "VfkvError", "Workspace", "PeerExchange", "guard_kv_precision", "kv_bytes_per_token",
           "kv_dtype_from_env", "ptr", "sliding_kv_start", "longest_common_prefix", "compute_auto_ctx",
           "gemma4_kv_read_layer"]
