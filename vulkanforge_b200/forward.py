"""The forward pass's view of the hot path: ``run_*`` dispatch helpers and the
``step_*`` executor steps of VulkanForge, bound to the CUDA library.

Mirrors, name for name:
  src/backend/vulkan/forward/runs.rs      run_kv_store_fp8, run_kv_copy_fp16,
                                          run_scalar_attn, run_flash_attn_split_reduce
  src/backend/vulkan/forward/executor/attention.rs   step_kv_write, step_attention,
                                          b_step_kv_write

Arguments that are Vulkan plumbing in the reference (device, registry, command
buffer, descriptor sets) collapse into the context and a CUDA stream.  Buffers
are device addresses: ints, or anything with ``data_ptr()``.
"""
from __future__ import annotations

from typing import Optional

from .kv_cache import Context, KvCache, Workspace, ptr, sliding_kv_start


class CudaForward:
    def __init__(self, ctx: Context, kv_cache: KvCache, n_heads: int, workspace: Optional[Workspace] = None,
                 *, sliding_window: int = 0, sliding_layers=None, kv_read_layer=None,
                 attn_scale: Optional[float] = None, softcap: float = 0.0, n_splits: int = 0,
                 max_batch: int = 1, max_splits: int = 64, stream=None):
        self.ctx = ctx
        self.kv_cache = kv_cache
        self.n_heads = n_heads
        self.stream = stream
        self.sliding_window = sliding_window
        self.sliding_layers = set(sliding_layers or ())
        self.kv_read_layer = dict(kv_read_layer or {})
        # forward/setup.rs:786 -- 1/sqrt(head_dim) unless the model overrides it (runs.rs:1483-1489)
        self.attn_scale = attn_scale if attn_scale is not None else 1.0 / float(kv_cache.config.head_dim) ** 0.5
        self.softcap = softcap
        self.n_splits = n_splits
        hd = max([kv_cache.config.head_dim] + list(kv_cache.config.per_layer_head_dim or []))
        self.workspace = workspace or Workspace(ctx, max_batch, n_heads, hd, max_splits)
        self._L = ctx._lib

    # ---- raw dispatch helpers ------------------------------------------------
    def run_kv_store_fp8(self, src, dst, n_elements: int, dst_byte_offset: int, label: str = "kv_store_fp8"):
        """runs.rs:2437-2478"""
        self.ctx.check(self._L.vfkv_kv_store_fp8(self.ctx.handle, ptr(src), ptr(dst), n_elements,
                                                 dst_byte_offset, self.stream))

    def run_kv_copy_fp16(self, src, dst, n_elements: int, dst_byte_offset: int, label: str = "kv_copy_fp16"):
        """runs.rs:2389-2430"""
        self.ctx.check(self._L.vfkv_kv_copy_fp16(self.ctx.handle, ptr(src), ptr(dst), n_elements,
                                                 dst_byte_offset, self.stream))

    def run_kv_fp8_to_f16(self, src, dst, n_elements: int):
        """the convert pre-pass inside run_flash_attn_cm_gemma_rs, runs.rs:1103-1137"""
        self.ctx.check(self._L.vfkv_kv_fp8_to_f16(self.ctx.handle, ptr(src), ptr(dst), n_elements, self.stream))

    # ---- routing helpers (forward/arch/gemma4.rs) ------------------------------
    def gemma4_kv_read_layer(self, layer: int) -> int:
        """gemma4.rs:27-49: publisher layer for a KV subscriber, else the layer itself."""
        return self.kv_read_layer.get(layer, layer)

    def gemma4_kv_start(self, layer: int, position: int) -> int:
        """gemma4.rs:59-73"""
        if layer in self.sliding_layers and self.sliding_window:
            return sliding_kv_start(position, self.sliding_window)
        return 0

    # ---- attention -------------------------------------------------------------
    def run_flash_attn_split_reduce(self, q, out, layer: int, position: int, n_tiles: int, kv_layer: int,
                                    kv_start: int, slot: int = 0):
        """runs.rs:1463-1571.  ``n_tiles`` is the split count (0 = choose)."""
        self.ctx.check(self._L.vfkv_attend(self.kv_cache.handle, self.workspace.handle, layer, kv_layer,
                                           ptr(q), ptr(out), self.n_heads, slot, position + 1, kv_start,
                                           self.attn_scale, self.softcap, n_tiles, self.stream))

    def run_flash_attn(self, q, out, layer: int, position: int, kv_layer: int, kv_start: int, slot: int = 0):
        """The single-workgroup shader of runs.rs:776-821 (flash_attn.comp): one pass, no scratch."""
        self.ctx.check(self._L.vfkv_flash_attn(self.kv_cache.handle, layer, kv_layer, ptr(q), ptr(out), self.n_heads,
                                               slot, position + 1, kv_start, self.attn_scale, self.softcap,
                                               self.stream))

    def run_scalar_attn(self, q, out, layer: int, position: int, slot: int = 0):
        """runs.rs:722-821: kv_layer / kv_start routing; two or more 64-position tiles go to the
        split + reduce path, shorter sequences to ``run_flash_attn``.  A split count given to the
        constructor overrides the library's choice on the split path."""
        kv_layer = self.gemma4_kv_read_layer(layer)
        kv_start = self.gemma4_kv_start(layer, position)
        if self.n_splits and self._L.vfkv_scalar_attn_uses_split(position):
            self.run_flash_attn_split_reduce(q, out, layer, position, self.n_splits, kv_layer, kv_start, slot)
            return
        self.ctx.check(self._L.vfkv_scalar_attn(self.kv_cache.handle, self.workspace.handle, layer, kv_layer, ptr(q),
                                                ptr(out), self.n_heads, slot, position, kv_start, self.attn_scale,
                                                self.softcap, self.stream))

    # ---- prefill chunk ------------------------------------------------------------
    def run_flash_attn_batch(self, layer: int, q, out, m: int, q_start: int, n_kv: int, kv_layer: int,
                             kv_start: int, slot: int = 0, window: int = 0):
        """runs.rs:933-1010 (flash_attn_batch.comp): m queries, query i at position q_start + i over
        [kv_start, min(q_start + i + 1, n_kv)).  ``window`` (extension): exact per-query window."""
        self.ctx.check(self._L.vfkv_attend_prefill(self.kv_cache.handle, layer, kv_layer, ptr(q), ptr(out),
                                                   self.n_heads, slot, m, q_start, n_kv, kv_start, window,
                                                   self.attn_scale, self.softcap, self.stream))

    def b_step_attention(self, layer: int, q, out, seq_len: int, base_pos: int, slot: int = 0,
                         exact_window: bool = False):
        """executor/attention.rs:2192-2393: kv_start is the LAST query's window bound for the whole
        chunk (:2215-2219), as the reference documents; ``exact_window`` masks per query instead."""
        kv_layer = self.gemma4_kv_read_layer(layer)
        window = self.sliding_window if layer in self.sliding_layers else 0
        kv_start = max(0, base_pos + seq_len - window) if window and not exact_window else 0
        self.run_flash_attn_batch(layer, q, out, seq_len, base_pos, base_pos + seq_len, kv_layer, kv_start, slot,
                                  window if exact_window else 0)

    # ---- RoPE (input preparation; fused with the append) -------------------------------
    def _rope(self, n_dims: Optional[int], freq_base: float, freq_scale: float):
        from ._lib import RopeParams
        return RopeParams(n_dims or self.kv_cache.config.head_dim, freq_base, freq_scale)

    def run_rope_neox(self, x, out, n_rows: int, n_heads: int, head_dim: int, base_pos: int = 0, positions=None,
                      n_dims: Optional[int] = None, freq_base: float = 10000.0, freq_scale: float = 1.0):
        """runs.rs:647-720 (rope_funcs.glsl:73-107) for [rows][heads][head_dim] f32, e.g. Q."""
        import ctypes as C
        rp = self._rope(n_dims or head_dim, freq_base, freq_scale)
        self.ctx.check(self._L.vfkv_rope_neox(self.ctx.handle, ptr(x), ptr(out), n_rows, n_heads, head_dim,
                                              ptr(positions), base_pos, C.byref(rp), self.stream))

    def rope_kv_write(self, layer: int, k_src, v_src, n_tokens: int, base_pos: int, slot: int = 0, k_rot=None,
                      n_dims: Optional[int] = None, freq_base: float = 10000.0, freq_scale: float = 1.0):
        """K rotated at base_pos.. and stored, V stored, in one launch (rope dispatch + KvWrite of
        executor/attention.rs:435-530,546-596)."""
        import ctypes as C
        rp = self._rope(n_dims, freq_base, freq_scale)
        self.ctx.check(self._L.vfkv_rope_append(self.kv_cache.handle, layer, ptr(k_src), ptr(v_src), n_tokens, slot,
                                                base_pos, C.byref(rp), ptr(k_rot), self.stream))

    def rope_kv_write_batch(self, layer: int, k_src, v_src, slot_ids, positions, n_seqs: int, k_rot=None,
                            n_dims: Optional[int] = None, freq_base: float = 10000.0, freq_scale: float = 1.0):
        import ctypes as C
        rp = self._rope(n_dims, freq_base, freq_scale)
        self.ctx.check(self._L.vfkv_rope_append_batch(self.kv_cache.handle, layer, ptr(k_src), ptr(v_src),
                                                      ptr(slot_ids), ptr(positions), n_seqs, C.byref(rp), ptr(k_rot),
                                                      self.stream))

    # ---- executor steps ----------------------------------------------------------
    def step_kv_write(self, layer: int, k_src, v_src, position: int, slot: int = 0):
        """executor/attention.rs:546-596 (one token)."""
        self.ctx.check(self._L.vfkv_append(self.kv_cache.handle, layer, ptr(k_src), ptr(v_src), 1, slot,
                                           position, self.stream))

    def b_step_kv_write(self, layer: int, k_src, v_src, seq_len: int, base_pos: int, slot: int = 0):
        """executor/attention.rs:2134-2190 (a prefill chunk of seq_len tokens)."""
        self.ctx.check(self._L.vfkv_append(self.kv_cache.handle, layer, ptr(k_src), ptr(v_src), seq_len, slot,
                                           base_pos, self.stream))

    def b_step_kv_write_sharded(self, layer: int, k_src, v_src, seq_len: int, base_pos: int, world: int, page: int,
                                rank: int, slot: int = 0):
        """b_step_kv_write on a cache sharded by position: base_pos is global, this rank's rows of the
        chunk are stored at their local positions, in one launch."""
        self.ctx.check(self._L.vfkv_append_sharded(self.kv_cache.handle, layer, ptr(k_src), ptr(v_src), seq_len, slot,
                                                   base_pos, world, page, rank, self.stream))

    def step_attention(self, layer: int, q, attn_out, position: int, slot: int = 0):
        """executor/attention.rs:599-626"""
        self.run_scalar_attn(q, attn_out, layer, position, slot)

    # ---- batched forms (independent sequences; no counterpart in the single-stream reference) ----
    def step_kv_write_batch(self, layer: int, k_src, v_src, slot_ids, positions, n_seqs: int):
        self.ctx.check(self._L.vfkv_append_batch(self.kv_cache.handle, layer, ptr(k_src), ptr(v_src),
                                                 ptr(slot_ids), ptr(positions), n_seqs, self.stream))

    def step_attention_batch(self, layer: int, q, attn_out, slot_ids, seq_lens, kv_starts, n_seqs: int,
                             max_seq_len_hint: int = 0, kv_layer: Optional[int] = None):
        kv_layer = self.gemma4_kv_read_layer(layer) if kv_layer is None else kv_layer
        self.ctx.check(self._L.vfkv_attend_batch(self.kv_cache.handle, self.workspace.handle, layer, kv_layer,
                                                 ptr(q), ptr(attn_out), self.n_heads, ptr(slot_ids),
                                                 ptr(seq_lens), ptr(kv_starts), n_seqs, max_seq_len_hint,
                                                 self.attn_scale, self.softcap, self.n_splits, self.stream))

    def decode_step(self, layer: int, q, k_src, v_src, attn_out, slot_ids, positions, n_seqs: int,
                    max_seq_len_hint: int = 0):
        """KvWrite then Attention for one token per sequence (layer_plan.rs:472-483)."""
        window = self.sliding_window if layer in self.sliding_layers else 0
        self.ctx.check(self._L.vfkv_decode_step(self.kv_cache.handle, self.workspace.handle, layer, ptr(q),
                                                ptr(k_src), ptr(v_src), ptr(attn_out), self.n_heads,
                                                ptr(slot_ids), ptr(positions), n_seqs, max_seq_len_hint,
                                                window, self.attn_scale, self.softcap, self.n_splits,
                                                self.stream))

    def _windows_array(self):
        import ctypes as C
        n_layers = self.kv_cache.config.n_layers
        if self.sliding_layers and self.sliding_window:
            return (C.c_uint32 * n_layers)(*[self.sliding_window if l in self.sliding_layers else 0
                                             for l in range(n_layers)])
        return None

    def decode_token(self, q, k_src, v_src, attn_out, slot_ids, positions, n_seqs: int,
                     max_seq_len_hint: int = 0):
        """Every layer's KvWrite + Attention for one token in one call (device buffers
        [n_layers][n_seqs][...]); what record_decode_dispatches records for this path
        (forward/decode.rs:43-82)."""
        import ctypes as C
        win = self._windows_array()
        self.ctx.check(self._L.vfkv_decode_token(
            self.kv_cache.handle, self.workspace.handle, ptr(q), ptr(k_src), ptr(v_src), ptr(attn_out),
            self.n_heads, ptr(slot_ids), ptr(positions), n_seqs, max_seq_len_hint,
            C.cast(win, C.c_void_p) if win is not None else None, self.attn_scale, self.softcap,
            self.n_splits, self.stream))

    def decode_token_host(self, h_q, h_k, h_v, h_out, h_positions, n_seqs: int, h_slot_ids=None):
        """forward_token's boundary (forward/decode.rs:567-626) for this path: host buffers in and out."""
        import ctypes as C
        n_layers = self.kv_cache.config.n_layers
        win = None
        if self.sliding_layers and self.sliding_window:
            win = (C.c_uint32 * n_layers)(*[self.sliding_window if l in self.sliding_layers else 0
                                            for l in range(n_layers)])
        self.ctx.check(self._L.vfkv_decode_token_host(
            self.kv_cache.handle, self.workspace.handle, ptr(h_q), ptr(h_k), ptr(h_v), ptr(h_out), self.n_heads,
            ptr(h_slot_ids), ptr(h_positions), n_seqs, C.cast(win, C.c_void_p) if win is not None else None,
            self.attn_scale, self.softcap, self.n_splits, self.stream))

    def decode_token_host_submit(self, h_q, h_k, h_v, h_out, h_positions, n_seqs: int, h_slot_ids=None) -> int:
        """decode_token_host without the wait (pre_record / fill_embed_and_submit,
        forward/decode.rs:169-259): returns a ticket; at most two may be in flight."""
        import ctypes as C
        n_layers = self.kv_cache.config.n_layers
        win = None
        if self.sliding_layers and self.sliding_window:
            win = (C.c_uint32 * n_layers)(*[self.sliding_window if l in self.sliding_layers else 0
                                            for l in range(n_layers)])
        ticket = C.c_uint64()
        self.ctx.check(self._L.vfkv_decode_token_host_submit(
            self.kv_cache.handle, self.workspace.handle, ptr(h_q), ptr(h_k), ptr(h_v), ptr(h_out), self.n_heads,
            ptr(h_slot_ids), ptr(h_positions), n_seqs, C.cast(win, C.c_void_p) if win is not None else None,
            self.attn_scale, self.softcap, self.n_splits, self.stream, C.byref(ticket)))
        return int(ticket.value)

    def decode_token_host_wait(self, ticket: int) -> None:
        """wait_and_read_logits for this path: h_out of that ticket is complete on return."""
        self.ctx.check(self._L.vfkv_decode_token_host_wait(self.workspace.handle, ticket))

    # ---- sequence-dimension sharding ---------------------------------------------
    def attend_partial(self, layer: int, q, pos_begin: int, pos_end: int, m, l, o, slot: int = 0,
                       kv_layer: Optional[int] = None):
        kv_layer = self.gemma4_kv_read_layer(layer) if kv_layer is None else kv_layer
        self.ctx.check(self._L.vfkv_attend_partial(self.kv_cache.handle, self.workspace.handle, layer, kv_layer,
                                                   ptr(q), self.n_heads, slot, pos_begin, pos_end,
                                                   self.attn_scale, self.softcap, self.n_splits, ptr(m), ptr(l),
                                                   ptr(o), self.stream))

    def attend_allgather(self, nccl_comm: int, world: int, rank: int, layer: int, q, pos_begin: int, pos_end: int,
                         packed, out, slot: int = 0, kv_layer: Optional[int] = None):
        """Partial over [pos_begin, pos_end), an NCCL all-gather of every rank's partial on the
        caller's communicator (``nccl_comm`` = the ncclComm_t as an integer) and the merge, in one
        library call.  ``packed`` is scratch of world * n_heads * (head_dim + 2) floats."""
        kv_layer = self.gemma4_kv_read_layer(layer) if kv_layer is None else kv_layer
        self.ctx.check(self._L.vfkv_attend_allgather(self.kv_cache.handle, self.workspace.handle, nccl_comm, world,
                                                     rank, layer, kv_layer, ptr(q), self.n_heads, slot, pos_begin,
                                                     pos_end, self.attn_scale, self.softcap, self.n_splits,
                                                     ptr(packed), ptr(out), self.stream))

    def attend_push(self, exchange, layer: int, q, pos_begin: int, pos_end: int, slot: int = 0,
                    kv_layer: Optional[int] = None, k_new=None, v_new=None):
        """Local partial over [pos_begin, pos_end), stored by the kernel into every rank's exchange
        buffer.  k_new / v_new: the new token's rows when this rank owns local position pos_end - 1."""
        kv_layer = self.gemma4_kv_read_layer(layer) if kv_layer is None else kv_layer
        self.ctx.check(self._L.vfkv_attend_push(self.kv_cache.handle, self.workspace.handle, exchange.handle, layer,
                                                kv_layer, ptr(q), ptr(k_new), ptr(v_new), self.n_heads, slot,
                                                pos_begin, pos_end, self.attn_scale, self.softcap, self.n_splits,
                                                self.stream))

    def exchange_merge(self, exchange, out):
        """Waits (bounded) for every rank's partial of the current exchange and merges them into out."""
        self.ctx.check(self._L.vfkv_exchange_merge(exchange.handle, ptr(out), self.stream))

    def attend_exchange(self, exchange, layer: int, q, pos_begin: int, pos_end: int, out, slot: int = 0,
                        kv_layer: Optional[int] = None, k_new=None, v_new=None):
        kv_layer = self.gemma4_kv_read_layer(layer) if kv_layer is None else kv_layer
        self.ctx.check(self._L.vfkv_attend_exchange(self.kv_cache.handle, self.workspace.handle, exchange.handle,
                                                    layer, kv_layer, ptr(q), ptr(k_new), ptr(v_new), self.n_heads,
                                                    slot, pos_begin, pos_end, self.attn_scale, self.softcap,
                                                    self.n_splits, ptr(out), self.stream))

    def merge_partials(self, m, l, o, n_parts: int, n_rows: int, head_dim: int, out):
        self.ctx.check(self._L.vfkv_merge_partials(self.ctx.handle, ptr(m), ptr(l), ptr(o), n_parts, n_rows,
                                                   head_dim, ptr(out), self.stream))

    def merge_partials_packed(self, packed, n_parts: int, n_rows: int, head_dim: int, out):
        """Merge of all-gathered partials: n_parts blocks of m[n_rows], l[n_rows], o[n_rows][head_dim]."""
        self.ctx.check(self._L.vfkv_merge_partials_packed(self.ctx.handle, ptr(packed), n_parts, n_rows,
                                                          head_dim, ptr(out), self.stream))
