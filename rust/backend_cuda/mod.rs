//! `src/backend/cuda/mod.rs` -- the dispatch helpers of the KV-cache hot path on the CUDA backend.
//!
//! `Forward` keeps the method names it has in `src/backend/vulkan/forward/runs.rs` and
//! `forward/executor/attention.rs`: `run_kv_store_fp8`, `run_kv_copy_fp16`, `run_scalar_attn`,
//! `run_flash_attn_split_reduce`, `run_flash_attn_batch`, `step_kv_write`, `step_attention`,
//! `b_step_kv_write`, and at token level `record_decode_dispatches`, `forward_token`,
//! `submit_token` / `wait_token`.  What was
//! (device, registry, command buffer) becomes (device, stream): work is enqueued on the stream in
//! call order, which replaces the pipeline barriers the Vulkan code records between these
//! dispatches.  Buffers are device pointers.  A decode step may also be issued as ONE call,
//! `decode_step`, which appends the token and attends in a single kernel launch per layer.
//!
//! NOT COMPILED in the repository this file lives in (no Rust toolchain in its build image).
pub mod kv_cache;

use std::os::raw::c_void;
use std::ptr;

use kv_cache::{CudaDevice, KvCache};
use vfkv_sys as sys;

/// Per-layer routing the model configuration decides (forward/arch/gemma4.rs:27-73).
pub struct AttnRouting {
    pub sliding_window: u32,
    pub sliding_layers: Vec<bool>,
    /// publisher layer of each layer (itself unless it subscribes to another layer's K/V)
    pub kv_read_layer: Vec<u32>,
    pub attn_scale: f32,
    pub softcap: f32,
}

pub struct Forward {
    pub kv_cache: KvCache,
    pub n_heads: u32,
    pub routing: AttnRouting,
    /// fa_scratch_out / _max / _sum of forward/setup.rs:203-230
    workspace: *mut sys::vfkv_workspace,
    /// q_buf / attn_out of the current slot (device pointers, f32)
    pub q_buf: *const f32,
    pub attn_out: *mut f32,
}

impl Forward {
    pub fn new(
        dev: &CudaDevice,
        kv_cache: KvCache,
        n_heads: u32,
        routing: AttnRouting,
    ) -> Result<Forward, String> {
        let max_hd = (0..kv_cache.config.n_layers).map(|l| kv_cache.head_dim_for(l)).max().unwrap_or(0);
        let mut workspace = ptr::null_mut();
        dev.check(unsafe { sys::vfkv_workspace_create(dev.ctx, 1, n_heads, max_hd, 64, &mut workspace) })?;
        Ok(Forward { kv_cache, n_heads, routing, workspace, q_buf: ptr::null(), attn_out: ptr::null_mut() })
    }

    // ---- runs.rs -----------------------------------------------------------------------------

    /// runs.rs:2437-2478
    pub fn run_kv_store_fp8(
        &mut self,
        dev: &CudaDevice,
        stream: *mut c_void,
        src: *const f32,
        dst: *mut c_void,
        n_elements: u32,
        dst_byte_offset: u64,
        _label: &'static str,
    ) -> Result<(), String> {
        dev.check(unsafe { sys::vfkv_kv_store_fp8(dev.ctx, src, dst, n_elements, dst_byte_offset, stream) })
    }

    /// runs.rs:2389-2430
    pub fn run_kv_copy_fp16(
        &mut self,
        dev: &CudaDevice,
        stream: *mut c_void,
        src: *const f32,
        dst: *mut c_void,
        n_elements: u32,
        dst_byte_offset: u64,
        _label: &'static str,
    ) -> Result<(), String> {
        dev.check(unsafe { sys::vfkv_kv_copy_fp16(dev.ctx, src, dst, n_elements, dst_byte_offset, stream) })
    }

    fn kv_start(&self, layer: u32, position: u32) -> u32 {
        if self.routing.sliding_layers.get(layer as usize).copied().unwrap_or(false) {
            unsafe { sys::vfkv_sliding_kv_start(position, self.routing.sliding_window) }
        } else {
            0
        }
    }

    /// runs.rs:722-821: kv_layer / kv_start routing, split path from two 64-position tiles on.
    pub fn run_scalar_attn(
        &mut self,
        dev: &CudaDevice,
        stream: *mut c_void,
        layer: u32,
        position: u32,
    ) -> Result<(), String> {
        let kv_layer = self.routing.kv_read_layer.get(layer as usize).copied().unwrap_or(layer);
        let kv_start = self.kv_start(layer, position);
        dev.check(unsafe {
            sys::vfkv_scalar_attn(
                self.kv_cache.handle,
                self.workspace,
                layer,
                kv_layer,
                self.q_buf,
                self.attn_out,
                self.n_heads,
                0,
                position,
                kv_start,
                self.routing.attn_scale,
                self.routing.softcap,
                stream,
            )
        })
    }

    /// runs.rs:1463-1571; `n_tiles` is the split count here (0 = let the library choose).
    #[allow(clippy::too_many_arguments)]
    pub fn run_flash_attn_split_reduce(
        &mut self,
        dev: &CudaDevice,
        stream: *mut c_void,
        layer: u32,
        position: u32,
        n_tiles: u32,
        kv_layer: u32,
        kv_start: u32,
    ) -> Result<(), String> {
        dev.check(unsafe {
            sys::vfkv_attend(
                self.kv_cache.handle,
                self.workspace,
                layer,
                kv_layer,
                self.q_buf,
                self.attn_out,
                self.n_heads,
                0,
                position + 1,
                kv_start,
                self.routing.attn_scale,
                self.routing.softcap,
                n_tiles,
                stream,
            )
        })
    }

    // ---- executor/attention.rs ---------------------------------------------------------------

    /// step_kv_write (attention.rs:546-596): one token's rotated K and its V into the cache.
    pub fn step_kv_write(
        &mut self,
        dev: &CudaDevice,
        stream: *mut c_void,
        layer: u32,
        k_src: *const f32,
        v_src: *const f32,
        position: u32,
    ) -> Result<(), String> {
        dev.check(unsafe { sys::vfkv_append(self.kv_cache.handle, layer, k_src, v_src, 1, 0, position, stream) })
    }

    /// b_step_kv_write (attention.rs:2134-2190): `seq_len` consecutive tokens from `base_pos`.
    #[allow(clippy::too_many_arguments)]
    pub fn b_step_kv_write(
        &mut self,
        dev: &CudaDevice,
        stream: *mut c_void,
        layer: u32,
        k_src: *const f32,
        v_src: *const f32,
        seq_len: u32,
        base_pos: u32,
    ) -> Result<(), String> {
        dev.check(unsafe { sys::vfkv_append(self.kv_cache.handle, layer, k_src, v_src, seq_len, 0, base_pos, stream) })
    }

    /// b_step_kv_write on a cache sharded by position over `world` GPUs (pages of `page` positions
    /// dealt round-robin): `base_pos` is global; this rank's rows of the chunk are stored at their
    /// local positions by one launch.
    #[allow(clippy::too_many_arguments)]
    pub fn b_step_kv_write_sharded(
        &mut self,
        dev: &CudaDevice,
        stream: *mut c_void,
        layer: u32,
        k_src: *const f32,
        v_src: *const f32,
        seq_len: u32,
        base_pos: u32,
        world: u32,
        page: u32,
        rank: u32,
    ) -> Result<(), String> {
        dev.check(unsafe {
            sys::vfkv_append_sharded(self.kv_cache.handle, layer, k_src, v_src, seq_len, 0, base_pos, world, page, rank, stream)
        })
    }

    /// Attention of one query token over this rank's share [0, local_len) of a position-sharded
    /// sequence, merged over the ranks through the host's NCCL communicator (`nccl_comm` is the
    /// ncclComm_t): partial, all-gather and merge in one call.  `packed` is scratch of
    /// world * n_heads * (head_dim + 2) floats.
    #[allow(clippy::too_many_arguments)]
    pub fn attend_allgather(
        &mut self,
        dev: &CudaDevice,
        stream: *mut c_void,
        nccl_comm: *mut c_void,
        world: u32,
        rank: u32,
        layer: u32,
        local_len: u32,
        packed: *mut f32,
    ) -> Result<(), String> {
        let kv_layer = self.routing.kv_read_layer.get(layer as usize).copied().unwrap_or(layer);
        dev.check(unsafe {
            sys::vfkv_attend_allgather(
                self.kv_cache.handle, self.workspace, nccl_comm, world, rank, layer, kv_layer, self.q_buf,
                self.n_heads, 0, 0, local_len, self.routing.attn_scale, self.routing.softcap, 0, packed,
                self.attn_out, stream,
            )
        })
    }

    /// step_attention (attention.rs:599-626)
    pub fn step_attention(
        &mut self,
        dev: &CudaDevice,
        stream: *mut c_void,
        layer: u32,
        position: u32,
    ) -> Result<(), String> {
        self.run_scalar_attn(dev, stream, layer, position)
    }

    /// KvWrite + Attention of one layer as one launch (layer_plan.rs:472-483 in one step).
    /// `d_positions` is a device word holding `position`, so that a captured CUDA graph can be
    /// replayed token after token.
    #[allow(clippy::too_many_arguments)]
    pub fn decode_step(
        &mut self,
        dev: &CudaDevice,
        stream: *mut c_void,
        layer: u32,
        k_src: *const f32,
        v_src: *const f32,
        d_positions: *const u32,
        max_seq_len_hint: u32,
    ) -> Result<(), String> {
        let window = if self.routing.sliding_layers.get(layer as usize).copied().unwrap_or(false) {
            self.routing.sliding_window
        } else {
            0
        };
        dev.check(unsafe {
            sys::vfkv_decode_step(
                self.kv_cache.handle,
                self.workspace,
                layer,
                self.q_buf,
                k_src,
                v_src,
                self.attn_out,
                self.n_heads,
                ptr::null(),
                d_positions,
                1,
                max_seq_len_hint,
                window,
                self.routing.attn_scale,
                self.routing.softcap,
                0,
                stream,
            )
        })
    }

    /// run_flash_attn_batch (runs.rs:933-1010) behind b_step_attention (attention.rs:2192-2393):
    /// `m` queries at positions `q_start ..` attend causally over the cache rows `[kv_start, n_kv)`.
    #[allow(clippy::too_many_arguments)]
    pub fn run_flash_attn_batch(
        &mut self,
        dev: &CudaDevice,
        stream: *mut c_void,
        layer: u32,
        q_batch: *const f32,
        out_batch: *mut f32,
        m: u32,
        q_start: u32,
        n_kv: u32,
    ) -> Result<(), String> {
        let kv_layer = self.routing.kv_read_layer.get(layer as usize).copied().unwrap_or(layer);
        let window = if self.routing.sliding_layers.get(layer as usize).copied().unwrap_or(false) {
            self.routing.sliding_window
        } else {
            0
        };
        dev.check(unsafe {
            sys::vfkv_attend_prefill(
                self.kv_cache.handle,
                layer,
                kv_layer,
                q_batch,
                out_batch,
                self.n_heads,
                0,
                m,
                q_start,
                n_kv,
                0,
                window,
                self.routing.attn_scale,
                self.routing.softcap,
                stream,
            )
        })
    }

    /// Per-layer windows in the form the token-level calls take (0 = global layer).
    fn windows(&self) -> Vec<u32> {
        (0..self.kv_cache.config.n_layers as usize)
            .map(|l| if self.routing.sliding_layers.get(l).copied().unwrap_or(false) { self.routing.sliding_window } else { 0 })
            .collect()
    }

    /// record_decode_dispatches (forward/decode.rs:43-82) for this path: every layer's KvWrite +
    /// Attention of one token, device inputs `[n_layers][..]`, nothing synchronises or allocates,
    /// so the call can be captured in a CUDA graph once and replayed per token.
    #[allow(clippy::too_many_arguments)]
    pub fn record_decode_dispatches(
        &mut self,
        dev: &CudaDevice,
        stream: *mut c_void,
        d_q: *const f32,
        d_k: *const f32,
        d_v: *const f32,
        d_out: *mut f32,
        d_positions: *const u32,
        max_seq_len_hint: u32,
    ) -> Result<(), String> {
        let windows = self.windows();
        dev.check(unsafe {
            sys::vfkv_decode_token(
                self.kv_cache.handle,
                self.workspace,
                d_q,
                d_k,
                d_v,
                d_out,
                self.n_heads,
                ptr::null(),
                d_positions,
                1,
                max_seq_len_hint,
                windows.as_ptr(),
                self.routing.attn_scale,
                self.routing.softcap,
                0,
                stream,
            )
        })
    }

    /// forward_token (forward/decode.rs:567-626) reduced to this path, with pinned HOST buffers:
    /// copies in, all layers, copy out, wait.
    #[allow(clippy::too_many_arguments)]
    pub fn forward_token(
        &mut self,
        dev: &CudaDevice,
        stream: *mut c_void,
        h_q: *const f32,
        h_k: *const f32,
        h_v: *const f32,
        h_out: *mut f32,
        position: u32,
    ) -> Result<(), String> {
        let windows = self.windows();
        dev.check(unsafe {
            sys::vfkv_decode_token_host(
                self.kv_cache.handle,
                self.workspace,
                h_q,
                h_k,
                h_v,
                h_out,
                self.n_heads,
                ptr::null(),
                &position,
                1,
                windows.as_ptr(),
                self.routing.attn_scale,
                self.routing.softcap,
                0,
                stream,
            )
        })?;
        self.commit_position(position);
        Ok(())
    }

    /// fill_embed_and_submit (forward/decode.rs:169-259): the same step without waiting; returns
    /// the ticket that `wait_token` takes.  At most two tokens in flight; `stream` must not be
    /// the default stream; the host buffers stay untouched until the ticket was waited for.
    #[allow(clippy::too_many_arguments)]
    pub fn submit_token(
        &mut self,
        dev: &CudaDevice,
        stream: *mut c_void,
        h_q: *const f32,
        h_k: *const f32,
        h_v: *const f32,
        h_out: *mut f32,
        position: u32,
    ) -> Result<u64, String> {
        let windows = self.windows();
        let mut ticket: u64 = 0;
        dev.check(unsafe {
            sys::vfkv_decode_token_host_submit(
                self.kv_cache.handle,
                self.workspace,
                h_q,
                h_k,
                h_v,
                h_out,
                self.n_heads,
                ptr::null(),
                &position,
                1,
                windows.as_ptr(),
                self.routing.attn_scale,
                self.routing.softcap,
                0,
                stream,
                &mut ticket,
            )
        })?;
        Ok(ticket)
    }

    /// wait_and_read_logits (forward/decode.rs:169-259) for this path: blocks until the token's
    /// outputs are in its host buffer, then commits the position.
    pub fn wait_token(&mut self, dev: &CudaDevice, ticket: u64, position: u32) -> Result<(), String> {
        dev.check(unsafe { sys::vfkv_decode_token_host_wait(self.workspace, ticket) })?;
        self.commit_position(position);
        Ok(())
    }

    /// After the token's GPU work has been waited for (forward/decode.rs:812).
    pub fn commit_position(&mut self, position: u32) {
        self.kv_cache.set_current_seq_len(position + 1);
    }

    pub fn destroy(self) {
        unsafe { sys::vfkv_workspace_destroy(self.workspace) };
        self.kv_cache.destroy();
    }
}
