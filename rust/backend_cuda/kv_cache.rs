//! `src/backend/cuda/kv_cache.rs` -- the KV cache of the CUDA backend.
//!
//! Same type and method names as `src/backend/vulkan/kv_cache.rs` (`KvDtype`, `KvCacheConfig`,
//! `KvCache::{new, bytes_per_buffer, head_dim_for, kv_heads_for, layer_offset_elems,
//! layer_offset_bytes, pos_offset_bytes, row_bytes, layer_size_bytes, is_fp8, is_fp16, reset,
//! zero_fill, zero_layer, destroy}`, `kv_dtype_from_env`, `guard_kv_precision`,
//! `kv_bytes_per_token`), so the forward pass keeps calling what it calls today.  Every number
//! comes from libvfkv.so; nothing is recomputed on this side.  `k_buffer` / `v_buffer` are device
//! pointers instead of `GpuBuffer`s, and `current_seq_len` is kept per slot inside the library
//! (slot 0 is the reference's single sequence).
//!
//! NOT COMPILED in the repository this file lives in (no Rust toolchain in its build image).
use std::ffi::CStr;
use std::os::raw::c_void;
use std::ptr;

use vfkv_sys as sys;

#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum KvDtype {
    F32,
    F16,
    F8,
}

impl KvDtype {
    fn raw(self) -> u32 {
        match self {
            KvDtype::F32 => sys::VFKV_F32,
            KvDtype::F16 => sys::VFKV_F16,
            KvDtype::F8 => sys::VFKV_F8,
        }
    }
    fn from_raw(v: u32) -> KvDtype {
        match v {
            sys::VFKV_F8 => KvDtype::F8,
            sys::VFKV_F16 => KvDtype::F16,
            _ => KvDtype::F32,
        }
    }
    pub fn element_size(self) -> u64 {
        unsafe { sys::vfkv_dtype_element_size(self.raw()) }
    }
    pub fn label(self) -> &'static str {
        match self {
            KvDtype::F32 => "FP32",
            KvDtype::F16 => "FP16",
            KvDtype::F8 => "FP8",
        }
    }
}

/// VULKANFORGE_KV_FP8 / VULKANFORGE_FP16_KV, read by the library exactly as the Vulkan backend does.
pub fn kv_dtype_from_env() -> KvDtype {
    KvDtype::from_raw(unsafe { sys::vfkv_dtype_from_env() })
}

pub fn guard_kv_precision(is_gemma4_moe: bool, kv_dtype: KvDtype) -> Result<(), String> {
    let force = std::env::var("VULKANFORGE_ALLOW_BROKEN_KV").as_deref() == Ok("1");
    let rc = unsafe { sys::vfkv_guard_kv_precision(is_gemma4_moe as i32, kv_dtype.raw(), force as i32) };
    if rc == sys::VFKV_OK {
        Ok(())
    } else {
        Err("gemma-4-MoE needs VULKANFORGE_KV_FP8=1: the F16/F32 KV cache is known to be broken for it".into())
    }
}

pub fn kv_bytes_per_token(
    n_layers: u32,
    n_kv_heads: u32,
    head_dim: u32,
    per_layer_head_dim: Option<&[u32]>,
    per_layer_n_kv_heads: Option<&[u32]>,
    elem_size: u64,
) -> u64 {
    unsafe {
        sys::vfkv_kv_bytes_per_token(
            n_layers,
            n_kv_heads,
            head_dim,
            per_layer_head_dim.map_or(ptr::null(), |v| v.as_ptr()),
            per_layer_n_kv_heads.map_or(ptr::null(), |v| v.as_ptr()),
            elem_size,
        )
    }
}

#[derive(Clone, Debug)]
pub struct KvCacheConfig {
    pub n_layers: u32,
    pub n_kv_heads: u32,
    pub head_dim: u32,
    pub max_seq_len: u32,
    pub per_layer_head_dim: Option<Vec<u32>>,
    pub per_layer_n_kv_heads: Option<Vec<u32>>,
}

/// One GPU's library context: the stand-in for the (device, pipeline registry) pair.
pub struct CudaDevice {
    pub(crate) ctx: *mut sys::vfkv_ctx,
}

impl CudaDevice {
    pub fn new(ordinal: i32) -> Result<CudaDevice, String> {
        let mut ctx = ptr::null_mut();
        let rc = unsafe { sys::vfkv_ctx_create(ordinal, &mut ctx) };
        if rc != sys::VFKV_OK {
            let text = unsafe { CStr::from_ptr(sys::vfkv_status_string(rc)) };
            return Err(format!("vfkv_ctx_create({ordinal}): {}", text.to_string_lossy()));
        }
        Ok(CudaDevice { ctx })
    }
    pub(crate) fn check(&self, rc: i32) -> Result<(), String> {
        if rc == sys::VFKV_OK {
            return Ok(());
        }
        let text = unsafe { CStr::from_ptr(sys::vfkv_last_error(self.ctx)) };
        Err(text.to_string_lossy().into_owned())
    }
    /// Device-side reports (a bounded wait that ran out, a row out of range); call once per token.
    pub fn poll(&self, stream: *mut c_void) -> Result<(), String> {
        self.check(unsafe { sys::vfkv_ctx_poll(self.ctx, stream) })
    }
}

impl Drop for CudaDevice {
    fn drop(&mut self) {
        unsafe { sys::vfkv_ctx_destroy(self.ctx) };
    }
}

pub struct KvCache {
    pub k_buffer: *mut c_void,
    pub v_buffer: *mut c_void,
    pub config: KvCacheConfig,
    pub kv_dtype: KvDtype,
    pub(crate) handle: *mut sys::vfkv_cache,
}

impl KvCache {
    /// As the reference: the element type is chosen here from the environment.
    pub fn new(device: &CudaDevice, config: KvCacheConfig) -> Result<KvCache, Box<dyn std::error::Error>> {
        let kv_dtype = kv_dtype_from_env();
        let raw = sys::vfkv_cache_config {
            n_layers: config.n_layers,
            n_kv_heads: config.n_kv_heads,
            head_dim: config.head_dim,
            max_seq_len: config.max_seq_len,
            dtype: kv_dtype.raw(),
            per_layer_head_dim: config.per_layer_head_dim.as_ref().map_or(ptr::null(), |v| v.as_ptr()),
            per_layer_n_kv_heads: config.per_layer_n_kv_heads.as_ref().map_or(ptr::null(), |v| v.as_ptr()),
            n_slots: 1,
            scale_mode: sys::VFKV_SCALE_NONE,
        };
        let mut handle = ptr::null_mut();
        device.check(unsafe { sys::vfkv_cache_create(device.ctx, &raw, &mut handle) })?;
        let (k_buffer, v_buffer) = unsafe { (sys::vfkv_cache_k_ptr(handle), sys::vfkv_cache_v_ptr(handle)) };
        eprintln!(
            "KV cache: {} x2 buffers of {} MB ({} layers, max_seq {})",
            kv_dtype.label(),
            unsafe { sys::vfkv_cache_bytes_per_buffer(handle) } >> 20,
            config.n_layers,
            config.max_seq_len
        );
        Ok(KvCache { k_buffer, v_buffer, config, kv_dtype, handle })
    }

    pub fn current_seq_len(&self) -> u32 {
        let mut n = 0u32;
        unsafe { sys::vfkv_cache_seq_len(self.handle, 0, &mut n) };
        n
    }
    /// `kv_cache.current_seq_len = n` of forward/decode.rs:812, forward/prefill.rs:277, state.rs:215-227.
    pub fn set_current_seq_len(&mut self, n: u32) {
        unsafe { sys::vfkv_cache_set_seq_len(self.handle, 0, n) };
    }
    pub fn bytes_per_buffer(&self) -> u64 {
        unsafe { sys::vfkv_cache_bytes_per_buffer(self.handle) }
    }
    pub fn head_dim_for(&self, layer: u32) -> u32 {
        unsafe { sys::vfkv_cache_head_dim_for(self.handle, layer) }
    }
    pub fn kv_heads_for(&self, layer: u32) -> u32 {
        unsafe { sys::vfkv_cache_kv_heads_for(self.handle, layer) }
    }
    pub fn layer_offset_elems(&self, layer: u32) -> u64 {
        unsafe { sys::vfkv_cache_layer_offset_elems(self.handle, layer) }
    }
    pub fn layer_offset_bytes(&self, layer: u32) -> u64 {
        unsafe { sys::vfkv_cache_layer_offset_bytes(self.handle, layer) }
    }
    pub fn pos_offset_bytes(&self, layer: u32, pos: u32) -> u64 {
        unsafe { sys::vfkv_cache_pos_offset_bytes(self.handle, layer, pos) }
    }
    pub fn row_bytes(&self, layer: u32) -> u64 {
        unsafe { sys::vfkv_cache_row_bytes(self.handle, layer) }
    }
    pub fn layer_size_bytes(&self, layer: u32) -> u64 {
        unsafe { sys::vfkv_cache_layer_size_bytes(self.handle, layer) }
    }
    pub fn is_fp8(&self) -> bool {
        self.kv_dtype == KvDtype::F8
    }
    pub fn is_fp16(&self) -> bool {
        self.kv_dtype == KvDtype::F16
    }
    /// Zeroes the counter only; the rows stay (prefix reuse relies on that).
    pub fn reset(&mut self) {
        unsafe { sys::vfkv_cache_reset(self.handle, 0) };
    }
    pub fn zero_fill(&self, device: &CudaDevice, stream: *mut c_void) -> Result<(), String> {
        device.check(unsafe { sys::vfkv_cache_zero_fill(self.handle, stream) })
    }
    pub fn zero_layer(&self, device: &CudaDevice, layer: u32, stream: *mut c_void) -> Result<(), String> {
        device.check(unsafe { sys::vfkv_cache_zero_layer(self.handle, layer, stream) })
    }
    pub fn destroy(self) {
        unsafe { sys::vfkv_cache_destroy(self.handle) };
    }
}
