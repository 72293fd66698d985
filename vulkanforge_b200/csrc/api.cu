// extern "C" surface of libvfkv.so (declared in include/vfkv.h): argument
// validation, cache / workspace objects, and routing to the kernel launchers.
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>

#include "attn_params.cuh"

using namespace vfkv;

namespace vfkv {

int32_t set_error(vfkv_ctx *ctx, int32_t status, const std::string &msg)
{
    if (ctx) ctx->last_error = msg;
    return status;
}

int32_t check_cuda(vfkv_ctx *ctx, cudaError_t e, const char *what)
{
    if (e == cudaSuccess) return VFKV_OK;
    int32_t st = e == cudaErrorMemoryAllocation ? VFKV_ERR_OOM : VFKV_ERR_CUDA;
    return set_error(ctx, st, std::string(what) + ": " + cudaGetErrorString(e));
}

}  // namespace vfkv

namespace {

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev)
    {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
        else prev = -1;
    }
    ~DeviceGuard()
    {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

inline cudaStream_t as_stream(void *s) { return static_cast<cudaStream_t>(s); }

// Views of one layer for the kernels.
KvView make_view(vfkv_cache *c, uint32_t kv_layer)
{
    const KvCache &kv = c->kv;
    KvView v;
    const uint64_t off = kv.layer_offset_bytes(kv_layer);
    v.k = static_cast<const uint8_t *>(kv.k_buffer) + off;
    v.v = static_cast<const uint8_t *>(kv.v_buffer) + off;
    v.slot_stride_bytes = kv.layer_size_bytes(kv_layer);
    v.max_seq = kv.config.max_seq_len;
    v.n_slots = kv.config.n_slots;
    v.dtype = uint32_t(kv.kv_dtype);
    v.n_kv_heads = kv.kv_heads_for(kv_layer);
    v.head_dim = kv.head_dim_for(kv_layer);
    if (kv.k_scales) {
        v.k_scales = kv.k_scales + kv.scale_offset(kv_layer, 0, 0);
        v.v_scales = kv.v_scales + kv.scale_offset(kv_layer, 0, 0);
        v.slot_stride_scales = uint64_t(kv.config.max_seq_len) * v.n_kv_heads;
    }
    // TMA descriptors are encoded once per layer and reused by every attention call
    if (c->tm_state.empty()) {
        c->tm_state.assign(kv.config.n_layers, 0);
        c->tm_k.resize(kv.config.n_layers);
        c->tm_v.resize(kv.config.n_layers);
    }
    if (c->tm_state[kv_layer] == 0)
        c->tm_state[kv_layer] = encode_layer_maps(c->ctx, v, c->tm_k[kv_layer].b, c->tm_v[kv_layer].b) ? 1 : 2;
    if (c->tm_state[kv_layer] == 1) {
        v.tm_k = c->tm_k[kv_layer].b;
        v.tm_v = c->tm_v[kv_layer].b;
    }
    return v;
}

int32_t check_layer(vfkv_cache *c, uint32_t layer, const char *fn)
{
    if (!c) return VFKV_ERR_INVALID;
    if (layer >= c->kv.config.n_layers)
        return set_error(c->ctx, VFKV_ERR_INVALID, std::string(fn) + ": layer out of range");
    return VFKV_OK;
}

}  // namespace

static void prof_clear(vfkv_ctx *ctx)
{
    for (auto &r : ctx->prof) { cudaEventDestroy(r.e0); cudaEventDestroy(r.e1); }
    ctx->prof.clear();
}

extern "C" {

uint32_t vfkv_abi_version(void) { return VFKV_ABI_VERSION; }

const char *vfkv_status_string(int32_t s)
{
    switch (s) {
    case VFKV_OK: return "ok";
    case VFKV_ERR_INVALID: return "invalid argument";
    case VFKV_ERR_OVERFLOW: return "size overflow";
    case VFKV_ERR_OOM: return "out of device memory";
    case VFKV_ERR_CUDA: return "CUDA error";
    case VFKV_ERR_UNSUPPORTED: return "unsupported shape or dtype";
    case VFKV_ERR_TIMEOUT: return "device-side wait timed out or a row was out of range";
    case VFKV_ERR_PRECISION: return "KV precision refused for this model";
    }
    return "unknown status";
}

int32_t vfkv_ctx_create(int32_t device_ordinal, vfkv_ctx **out)
{
    if (!out) return VFKV_ERR_INVALID;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) return VFKV_ERR_CUDA;
    if (device_ordinal < 0 || device_ordinal >= n) return VFKV_ERR_INVALID;
    vfkv_ctx *ctx = new (std::nothrow) vfkv_ctx();
    if (!ctx) return VFKV_ERR_OOM;
    ctx->device = device_ordinal;
    DeviceGuard g(device_ordinal);
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device_ordinal) != cudaSuccess) { delete ctx; return VFKV_ERR_CUDA; }
    if (prop.major != 10) {
        // the library is built for sm_100a only; refuse early instead of failing at first launch
        delete ctx;
        return VFKV_ERR_UNSUPPORTED;
    }
    ctx->sm_count = prop.multiProcessorCount;
    if (cudaMalloc(&ctx->d_status, sizeof(uint32_t)) != cudaSuccess) { delete ctx; return VFKV_ERR_OOM; }
    cudaMemset(ctx->d_status, 0, sizeof(uint32_t));
    cudaDriverEntryPointQueryResult qres;
    void *fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
        ctx->encode_tiled = fn;
    *out = ctx;
    return VFKV_OK;
}

int32_t vfkv_ctx_destroy(vfkv_ctx *ctx)
{
    if (!ctx) return VFKV_OK;
    DeviceGuard g(ctx->device);
    cudaFree(ctx->d_status);
    cudaFree(ctx->d_prefill_scratch);
    prof_clear(ctx);
    delete ctx;
    return VFKV_OK;
}

const char *vfkv_last_error(const vfkv_ctx *ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }

int32_t vfkv_ctx_poll(vfkv_ctx *ctx, void *stream)
{
    if (!ctx) return VFKV_ERR_INVALID;
    DeviceGuard g(ctx->device);
    uint32_t h = 0;
    cudaError_t e = cudaMemcpyAsync(&h, ctx->d_status, 4, cudaMemcpyDeviceToHost, as_stream(stream));
    if (e == cudaSuccess) e = cudaMemsetAsync(ctx->d_status, 0, 4, as_stream(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(as_stream(stream));
    if (e != cudaSuccess) return check_cuda(ctx, e, "vfkv_ctx_poll");
    if (h == 0) return VFKV_OK;
    return set_error(ctx, VFKV_ERR_TIMEOUT,
                     std::string("device status word = ") + std::to_string(h) +
                         " (1: bounded wait gave up, 2: append row out of range, 4: attend slot/length out of range, "
                         "8: a peer's partial did not arrive in time)");
}

int32_t vfkv_ctx_set_attn_impl(vfkv_ctx *ctx, uint32_t impl)
{
    if (!ctx || impl > 3) return VFKV_ERR_INVALID;
    ctx->attn_impl = impl;
    return VFKV_OK;
}

int32_t vfkv_ctx_set_attn_tuning(vfkv_ctx *ctx, uint32_t warps, uint32_t stages)
{
    if (!ctx) return VFKV_ERR_INVALID;
    const bool ok = (warps == 0 && stages == 0) || (warps == 4 && stages >= 1 && stages <= 3) ||
                    (warps == 8 && (stages == 1 || stages == 3));
    if (!ok) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_ctx_set_attn_tuning: warps x stages must be 0x0, 4x1, 4x2, 4x3, 8x1 or 8x3");
    ctx->tune_warps = warps;
    ctx->tune_stages = stages;
    return VFKV_OK;
}

int32_t vfkv_ctx_set_dependent_launch(vfkv_ctx *ctx, uint32_t mode)
{
    if (!ctx || mode > 2) return VFKV_ERR_INVALID;
    ctx->pdl = mode;
    return VFKV_OK;
}

int32_t vfkv_ctx_set_merge_wait_ms(vfkv_ctx *ctx, uint32_t ms)
{
    if (!ctx || ms == 0 || ms > 10000) return VFKV_ERR_INVALID;
    ctx->merge_wait_ns = uint64_t(ms) * 1000000ull;
    return VFKV_OK;
}

int32_t vfkv_ctx_debug_fail_split(vfkv_ctx *ctx, uint32_t split)
{
    if (!ctx) return VFKV_ERR_INVALID;
    ctx->debug_fail_split = split;
    return VFKV_OK;
}

int32_t vfkv_ctx_set_trace_buffer(vfkv_ctx *ctx, void *d_buffer)
{
    if (!ctx) return VFKV_ERR_INVALID;
    ctx->d_trace = static_cast<unsigned long long *>(d_buffer);
    ctx->trace_seq = 0;
    return VFKV_OK;
}

int32_t vfkv_ctx_set_trace_ring(vfkv_ctx *ctx, uint32_t n_blocks)
{
    if (!ctx || n_blocks == 0) return VFKV_ERR_INVALID;
    ctx->trace_ring = n_blocks;
    ctx->trace_seq = 0;
    return VFKV_OK;
}

uint64_t vfkv_ctx_launch_count(const vfkv_ctx *ctx) { return ctx ? ctx->launches : 0; }

int32_t vfkv_profile_enable(vfkv_ctx *ctx, int32_t on)
{
    if (!ctx) return VFKV_ERR_INVALID;
    DeviceGuard g(ctx->device);
    ctx->profiling = on != 0;
    if (!on) prof_clear(ctx);
    return VFKV_OK;
}

int32_t vfkv_profile_collect(vfkv_ctx *ctx, uint32_t label, uint64_t *count, double *total_ms, double *min_ms,
                             int32_t reset)
{
    if (!ctx || label >= VFKV_PROF_LABELS) return VFKV_ERR_INVALID;
    DeviceGuard g(ctx->device);
    uint64_t n = 0;
    double tot = 0.0, mn = 0.0;
    for (auto &r : ctx->prof) {
        if (r.label != label) continue;
        cudaError_t e = cudaEventSynchronize(r.e1);
        float ms = 0.f;
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, r.e0, r.e1);
        if (e != cudaSuccess) return check_cuda(ctx, e, "vfkv_profile_collect");
        tot += ms;
        mn = (n == 0 || ms < mn) ? ms : mn;
        ++n;
    }
    if (count) *count = n;
    if (total_ms) *total_ms = tot;
    if (min_ms) *min_ms = mn;
    if (reset) prof_clear(ctx);
    return VFKV_OK;
}

/* ---- cache --------------------------------------------------------------- */

int32_t vfkv_cache_create(vfkv_ctx *ctx, const vfkv_cache_config *cfg, vfkv_cache **out)
{
    if (!ctx || !cfg || !out) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_cache_create: null argument");
    *out = nullptr;
    if (cfg->dtype > VFKV_F8) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_cache_create: unknown dtype");
    KvCacheConfig c;
    c.n_layers = cfg->n_layers; c.n_kv_heads = cfg->n_kv_heads; c.head_dim = cfg->head_dim;
    c.max_seq_len = cfg->max_seq_len; c.n_slots = cfg->n_slots ? cfg->n_slots : 1;
    c.scale_mode = cfg->scale_mode;
    if (cfg->per_layer_head_dim)
        c.per_layer_head_dim = std::vector<uint32_t>(cfg->per_layer_head_dim, cfg->per_layer_head_dim + cfg->n_layers);
    if (cfg->per_layer_n_kv_heads)
        c.per_layer_n_kv_heads = std::vector<uint32_t>(cfg->per_layer_n_kv_heads, cfg->per_layer_n_kv_heads + cfg->n_layers);
    vfkv_cache *cache = new (std::nothrow) vfkv_cache();
    if (!cache) return set_error(ctx, VFKV_ERR_OOM, "host allocation failed");
    cache->ctx = ctx;
    std::string err;
    if (!KvCache::plan(c, KvDtype(cfg->dtype), &cache->kv, &err)) {
        delete cache;
        const bool ovf = err.find("overflow") != std::string::npos;
        return set_error(ctx, ovf ? VFKV_ERR_OVERFLOW : VFKV_ERR_INVALID, "vfkv_cache_create: " + err);
    }
    DeviceGuard g(ctx->device);
    KvCache &kv = cache->kv;
    const uint64_t bytes = kv.bytes ? kv.bytes : 16;
    cudaError_t e = cudaMalloc(&kv.k_buffer, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&kv.v_buffer, bytes);
    if (e == cudaSuccess && kv.scale_floats) {
        e = cudaMalloc(reinterpret_cast<void **>(&kv.k_scales), kv.scale_floats * 4);
        if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&kv.v_scales), kv.scale_floats * 4);
    }
    if (e != cudaSuccess) {
        cudaFree(kv.k_buffer); cudaFree(kv.v_buffer); cudaFree(kv.k_scales); cudaFree(kv.v_scales);
        cudaGetLastError();
        delete cache;
        return check_cuda(ctx, e, "vfkv_cache_create: cudaMalloc");
    }
    *out = cache;
    return VFKV_OK;
}

int32_t vfkv_cache_destroy(vfkv_cache *cache)
{
    if (!cache) return VFKV_OK;
    DeviceGuard g(cache->ctx->device);
    cudaFree(cache->kv.k_buffer); cudaFree(cache->kv.v_buffer);
    cudaFree(cache->kv.k_scales); cudaFree(cache->kv.v_scales);
    delete cache;
    return VFKV_OK;
}

int32_t vfkv_cache_zero_fill(vfkv_cache *cache, void *stream)
{
    if (!cache) return VFKV_ERR_INVALID;
    DeviceGuard g(cache->ctx->device);
    KvCache &kv = cache->kv;
    cudaError_t e = cudaMemsetAsync(kv.k_buffer, 0, kv.bytes, as_stream(stream));
    if (e == cudaSuccess) e = cudaMemsetAsync(kv.v_buffer, 0, kv.bytes, as_stream(stream));
    if (e == cudaSuccess && kv.k_scales) {
        e = cudaMemsetAsync(kv.k_scales, 0, kv.scale_floats * 4, as_stream(stream));
        if (e == cudaSuccess) e = cudaMemsetAsync(kv.v_scales, 0, kv.scale_floats * 4, as_stream(stream));
    }
    return check_cuda(cache->ctx, e, "vfkv_cache_zero_fill");
}

int32_t vfkv_cache_zero_layer(vfkv_cache *cache, uint32_t layer, void *stream)
{
    int32_t rc = check_layer(cache, layer, "vfkv_cache_zero_layer");
    if (rc) return rc;
    DeviceGuard g(cache->ctx->device);
    KvCache &kv = cache->kv;
    const uint64_t off = kv.layer_offset_bytes(layer), size = kv.layer_size_bytes(layer) * kv.config.n_slots;
    cudaError_t e = cudaMemsetAsync(static_cast<uint8_t *>(kv.k_buffer) + off, 0, size, as_stream(stream));
    if (e == cudaSuccess) e = cudaMemsetAsync(static_cast<uint8_t *>(kv.v_buffer) + off, 0, size, as_stream(stream));
    return check_cuda(cache->ctx, e, "vfkv_cache_zero_layer");
}

int32_t vfkv_cache_reset(vfkv_cache *cache, uint32_t slot)
{
    if (!cache || slot >= cache->kv.config.n_slots) return VFKV_ERR_INVALID;
    cache->kv.reset(slot);
    return VFKV_OK;
}

int32_t vfkv_cache_seq_len(const vfkv_cache *cache, uint32_t slot, uint32_t *out)
{
    if (!cache || !out || slot >= cache->kv.config.n_slots) return VFKV_ERR_INVALID;
    *out = cache->kv.current_seq_len[slot];
    return VFKV_OK;
}

int32_t vfkv_cache_set_seq_len(vfkv_cache *cache, uint32_t slot, uint32_t seq_len)
{
    if (!cache || slot >= cache->kv.config.n_slots) return VFKV_ERR_INVALID;
    if (seq_len > cache->kv.config.max_seq_len)
        return set_error(cache->ctx, VFKV_ERR_INVALID, "vfkv_cache_set_seq_len: beyond max_seq_len");
    cache->kv.current_seq_len[slot] = seq_len;
    return VFKV_OK;
}

#define VFKV_LAYER_OK(c, l) ((c) && (l) < (c)->kv.config.n_layers)
uint32_t vfkv_cache_head_dim_for(const vfkv_cache *c, uint32_t l) { return VFKV_LAYER_OK(c, l) ? c->kv.head_dim_for(l) : 0; }
uint32_t vfkv_cache_kv_heads_for(const vfkv_cache *c, uint32_t l) { return VFKV_LAYER_OK(c, l) ? c->kv.kv_heads_for(l) : 0; }
uint64_t vfkv_cache_row_bytes(const vfkv_cache *c, uint32_t l) { return VFKV_LAYER_OK(c, l) ? c->kv.row_bytes(l) : 0; }
uint64_t vfkv_cache_layer_size_bytes(const vfkv_cache *c, uint32_t l) { return VFKV_LAYER_OK(c, l) ? c->kv.layer_size_bytes(l) : 0; }
uint64_t vfkv_cache_layer_offset_bytes(const vfkv_cache *c, uint32_t l) { return VFKV_LAYER_OK(c, l) ? c->kv.layer_offset_bytes(l) : 0; }
uint64_t vfkv_cache_layer_offset_elems(const vfkv_cache *c, uint32_t l) { return VFKV_LAYER_OK(c, l) ? c->kv.layer_offset_elems(l) : 0; }
uint64_t vfkv_cache_pos_offset_bytes(const vfkv_cache *c, uint32_t l, uint32_t pos) { return VFKV_LAYER_OK(c, l) ? c->kv.pos_offset_bytes(l, pos) : 0; }
uint64_t vfkv_cache_slot_offset_bytes(const vfkv_cache *c, uint32_t l, uint32_t slot) { return VFKV_LAYER_OK(c, l) ? c->kv.slot_offset_bytes(l, slot) : 0; }
uint64_t vfkv_cache_bytes_per_buffer(const vfkv_cache *c) { return c ? c->kv.bytes_per_buffer() : 0; }
uint32_t vfkv_cache_dtype(const vfkv_cache *c) { return c ? uint32_t(c->kv.kv_dtype) : 0; }
int32_t vfkv_cache_is_fp8(const vfkv_cache *c) { return c && c->kv.is_fp8(); }
int32_t vfkv_cache_is_fp16(const vfkv_cache *c) { return c && c->kv.is_fp16(); }
void *vfkv_cache_k_ptr(const vfkv_cache *c) { return c ? c->kv.k_buffer : nullptr; }
void *vfkv_cache_v_ptr(const vfkv_cache *c) { return c ? c->kv.v_buffer : nullptr; }
float *vfkv_cache_k_scale_ptr(const vfkv_cache *c) { return c ? c->kv.k_scales : nullptr; }
float *vfkv_cache_v_scale_ptr(const vfkv_cache *c) { return c ? c->kv.v_scales : nullptr; }

uint64_t vfkv_kv_bytes_per_token(uint32_t n_layers, uint32_t n_kv_heads, uint32_t head_dim,
                                 const uint32_t *plhd, const uint32_t *plkv, uint64_t elem_size)
{
    return kv_bytes_per_token(n_layers, n_kv_heads, head_dim, plhd, plkv, elem_size);
}
uint64_t vfkv_dtype_element_size(uint32_t dtype) { return dtype <= VFKV_F8 ? element_size(KvDtype(dtype)) : 0; }
uint32_t vfkv_dtype_from_env(void) { return uint32_t(kv_dtype_from_env()); }
int32_t vfkv_guard_kv_precision(int32_t is_gemma4_moe, uint32_t dtype, int32_t force)
{
    if (dtype > VFKV_F8) return VFKV_ERR_INVALID;
    return guard_kv_precision(is_gemma4_moe != 0, KvDtype(dtype), force != 0, nullptr) ? VFKV_OK
                                                                                       : VFKV_ERR_PRECISION;
}
uint32_t vfkv_sliding_kv_start(uint32_t position, uint32_t window) { return sliding_kv_start(position, window); }

/* ---- raw ops -------------------------------------------------------------- */

static int32_t raw_store(vfkv_ctx *ctx, uint32_t dtype, const float *src, void *dst, uint32_t n,
                         uint64_t off, void *stream, const char *fn)
{
    if (!ctx) return VFKV_ERR_INVALID;
    if (!src || !dst) return set_error(ctx, VFKV_ERR_INVALID, std::string(fn) + ": null buffer");
    // src/backend/vulkan/forward/runs.rs:2400-2404,2448-2452
    if (off % 4 != 0 || reinterpret_cast<uintptr_t>(dst) % 4 != 0)
        return set_error(ctx, VFKV_ERR_INVALID, std::string(fn) + ": dst_byte_offset must be 4-byte aligned");
    DeviceGuard g(ctx->device);
    return launch_store(ctx, dtype, src, static_cast<uint8_t *>(dst) + off, n, as_stream(stream));
}

int32_t vfkv_kv_store_fp8(vfkv_ctx *ctx, const float *d_src, void *d_dst, uint32_t n, uint64_t off, void *stream)
{
    return raw_store(ctx, VFKV_F8, d_src, d_dst, n, off, stream, "vfkv_kv_store_fp8");
}

int32_t vfkv_kv_copy_fp16(vfkv_ctx *ctx, const float *d_src, void *d_dst, uint32_t n, uint64_t off, void *stream)
{
    return raw_store(ctx, VFKV_F16, d_src, d_dst, n, off, stream, "vfkv_kv_copy_fp16");
}

int32_t vfkv_kv_fp8_to_f16(vfkv_ctx *ctx, const void *d_src, void *d_dst, uint64_t n, void *stream)
{
    if (!ctx) return VFKV_ERR_INVALID;
    if (!d_src || !d_dst) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_kv_fp8_to_f16: null buffer");
    if (reinterpret_cast<uintptr_t>(d_dst) % 2 != 0)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_kv_fp8_to_f16: destination must be 2-byte aligned");
    DeviceGuard g(ctx->device);
    return launch_fp8_to_f16(ctx, d_src, d_dst, n, as_stream(stream));
}

int32_t vfkv_flash_attn_split_reduce(vfkv_ctx *ctx, vfkv_workspace *ws, const float *d_q, const void *d_k,
                                     const void *d_v, float *d_out, uint32_t dtype, uint32_t n_heads,
                                     uint32_t n_kv_heads, uint32_t head_dim, uint32_t seq_len,
                                     uint32_t max_seq, float scale, uint32_t kv_start, float softcap,
                                     uint32_t n_splits, void *stream)
{
    if (!ctx) return VFKV_ERR_INVALID;
    if (!d_q || !d_k || !d_v || !d_out) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_flash_attn_split_reduce: null buffer");
    if (dtype > VFKV_F8) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_flash_attn_split_reduce: unknown dtype");
    if (seq_len > max_seq) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_flash_attn_split_reduce: seq_len > max_seq");
    if ((reinterpret_cast<uintptr_t>(d_k) | reinterpret_cast<uintptr_t>(d_v)) % 16 != 0)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_flash_attn_split_reduce: K/V slabs must be 16-byte aligned");
    AttnArgs a;
    a.kv.k = d_k; a.kv.v = d_v; a.kv.max_seq = max_seq; a.kv.n_slots = 1; a.kv.dtype = dtype;
    a.kv.n_kv_heads = n_kv_heads; a.kv.head_dim = head_dim;
    a.seq.n_seqs = 1; a.seq.seq_len_scalar = seq_len; a.seq.kv_start_scalar = kv_start;
    a.q = d_q; a.out = d_out; a.n_q_heads = n_heads; a.scale = scale; a.softcap = softcap;
    a.n_splits = n_splits;
    DeviceGuard g(ctx->device);
    return launch_attention(ctx, ws, a, as_stream(stream));
}

/* ---- workspace ------------------------------------------------------------ */

int32_t vfkv_workspace_create(vfkv_ctx *ctx, uint32_t max_seqs, uint32_t n_q_heads, uint32_t head_dim,
                              uint32_t max_splits, vfkv_workspace **out)
{
    if (!ctx || !out) return VFKV_ERR_INVALID;
    *out = nullptr;
    if (!max_seqs || !n_q_heads || !head_dim || !max_splits)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_workspace_create: zero dimension");
    uint64_t rows, parts, ofl;
    if (__builtin_mul_overflow(uint64_t(max_seqs), uint64_t(n_q_heads), &rows) ||
        __builtin_mul_overflow(rows, uint64_t(max_splits), &parts) ||
        __builtin_mul_overflow(parts, uint64_t(head_dim) * 4, &ofl))
        return set_error(ctx, VFKV_ERR_OVERFLOW, "vfkv_workspace_create: size overflow");
    vfkv_workspace *ws = new (std::nothrow) vfkv_workspace();
    if (!ws) return set_error(ctx, VFKV_ERR_OOM, "host allocation failed");
    ws->ctx = ctx; ws->max_seqs = max_seqs; ws->n_q_heads = n_q_heads; ws->head_dim = head_dim;
    ws->max_splits = max_splits;
    DeviceGuard g(ctx->device);
    const uint64_t u32_bytes = uint64_t(max_seqs) * 4 * 4;
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&ws->part_o), ofl);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&ws->part_m), parts * 4);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&ws->part_l), parts * 4);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&ws->d_u32), u32_bytes);
    ws->n_counters = rows;
    // per (q-head row, split): the o words, and room for the {m, l} words and padding of up to sixteen
    // slices of the output (one per merging CTA; a launch takes fewer slices if that is not enough)
    ws->tag_words = parts * (uint64_t(head_dim) + 68);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&ws->tickets), rows * 256 * 8);
    if (e == cudaSuccess) e = cudaMemset(ws->tickets, 0, rows * 256 * 8);
    // tag 0 is never used by a launch, so zeroed words read as "not there yet"
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&ws->tag_part), ws->tag_words * 8);
    if (e == cudaSuccess) e = cudaMemset(ws->tag_part, 0, ws->tag_words * 8);
    if (e != cudaSuccess) {
        cudaFree(ws->part_o); cudaFree(ws->part_m); cudaFree(ws->part_l); cudaFree(ws->d_u32); cudaFree(ws->tickets);
        cudaFree(ws->tag_part);
        cudaGetLastError();
        delete ws;
        return check_cuda(ctx, e, "vfkv_workspace_create: cudaMalloc");
    }
    ws->bytes = ofl + parts * 8 + u32_bytes + rows * 256 * 8 + ws->tag_words * 8;
    *out = ws;
    return VFKV_OK;
}

int32_t vfkv_workspace_destroy(vfkv_workspace *ws)
{
    if (!ws) return VFKV_OK;
    DeviceGuard g(ws->ctx->device);
    cudaFree(ws->part_o); cudaFree(ws->part_m); cudaFree(ws->part_l); cudaFree(ws->d_u32); cudaFree(ws->tickets);
    cudaFree(ws->tag_part);
    cudaFree(ws->stage_in); cudaFree(ws->stage_out);
    for (auto gexec : ws->tok_graphs)
        if (gexec) cudaGraphExecDestroy(gexec);
    for (auto ev : ws->tok_events)
        if (ev) cudaEventDestroy(ev);
    if (ws->copy_stream) cudaStreamDestroy(ws->copy_stream);
    for (auto &hs : ws->host_slot) {
        cudaFree(hs.in); cudaFree(hs.out); cudaFree(hs.u32);
        if (hs.graph) cudaGraphExecDestroy(hs.graph);
        if (hs.ev_in) cudaEventDestroy(hs.ev_in);
        if (hs.ev_done) cudaEventDestroy(hs.ev_done);
        if (hs.ev_out) cudaEventDestroy(hs.ev_out);
    }
    if (ws->h2d_stream) cudaStreamDestroy(ws->h2d_stream);
    if (ws->d2h_stream) cudaStreamDestroy(ws->d2h_stream);
    cudaGetLastError();
    delete ws;
    return VFKV_OK;
}

int32_t vfkv_workspace_reset(vfkv_workspace *ws, void *stream)
{
    if (!ws) return VFKV_ERR_INVALID;
    DeviceGuard g(ws->ctx->device);
    cudaError_t e = cudaMemsetAsync(ws->tickets, 0, ws->n_counters * 256 * 8, as_stream(stream));
    if (e == cudaSuccess) e = cudaMemsetAsync(ws->tag_part, 0, ws->tag_words * 8, as_stream(stream));
    return check_cuda(ws->ctx, e, "vfkv_workspace_reset");
}

uint64_t vfkv_workspace_bytes(const vfkv_workspace *ws) { return ws ? ws->bytes + ws->stage_in_bytes + ws->stage_out_bytes : 0; }

/* ---- cache-level ops ------------------------------------------------------- */

static AppendArgs make_append(vfkv_cache *cache, uint32_t layer, const float *k, const float *v)
{
    KvCache &kv = cache->kv;
    AppendArgs a;
    a.k = k; a.v = v;
    const uint64_t off = kv.layer_offset_bytes(layer);
    a.k_dst = static_cast<uint8_t *>(kv.k_buffer) + off;
    a.v_dst = static_cast<uint8_t *>(kv.v_buffer) + off;
    a.slot_stride_bytes = kv.layer_size_bytes(layer);
    a.n_kv_heads = kv.kv_heads_for(layer);
    a.head_dim = kv.head_dim_for(layer);
    a.row_elems = a.n_kv_heads * a.head_dim;
    a.dtype = uint32_t(kv.kv_dtype);
    a.max_seq = kv.config.max_seq_len;
    a.n_slots = kv.config.n_slots;
    if (kv.k_scales) {
        a.k_scales = kv.k_scales + kv.scale_offset(layer, 0, 0);
        a.v_scales = kv.v_scales + kv.scale_offset(layer, 0, 0);
        a.slot_stride_scales = uint64_t(kv.config.max_seq_len) * a.n_kv_heads;
    }
    return a;
}

int32_t vfkv_append(vfkv_cache *cache, uint32_t layer, const float *d_k, const float *d_v, uint32_t n_tokens,
                    uint32_t slot, uint32_t base_pos, void *stream)
{
    int32_t rc = check_layer(cache, layer, "vfkv_append");
    if (rc) return rc;
    vfkv_ctx *ctx = cache->ctx;
    if (!d_k || !d_v) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_append: null K or V");
    if ((reinterpret_cast<uintptr_t>(d_k) | reinterpret_cast<uintptr_t>(d_v)) % 16 != 0)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_append: K and V inputs must be 16-byte aligned");
    if (slot >= cache->kv.config.n_slots) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_append: slot out of range");
    // the context-overflow check of src/backend/vulkan/decode.rs:523-533, at the cache
    if (uint64_t(base_pos) + n_tokens > cache->kv.config.max_seq_len)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_append: base_pos + n_tokens exceeds max_seq_len");
    AppendArgs a = make_append(cache, layer, d_k, d_v);
    a.n_rows = n_tokens; a.slot = slot; a.base_pos = base_pos;
    DeviceGuard g(ctx->device);
    return launch_append(ctx, a, as_stream(stream));
}

int32_t vfkv_append_sharded(vfkv_cache *cache, uint32_t layer, const float *d_k, const float *d_v, uint32_t n_tokens,
                            uint32_t slot, uint32_t base_pos, uint32_t world, uint32_t page, uint32_t rank, void *stream)
{
    int32_t rc = check_layer(cache, layer, "vfkv_append_sharded");
    if (rc) return rc;
    vfkv_ctx *ctx = cache->ctx;
    if (!d_k || !d_v) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_append_sharded: null K or V");
    if ((reinterpret_cast<uintptr_t>(d_k) | reinterpret_cast<uintptr_t>(d_v)) % 16 != 0)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_append_sharded: K and V inputs must be 16-byte aligned");
    if (slot >= cache->kv.config.n_slots) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_append_sharded: slot out of range");
    if (world == 0 || rank >= world || page == 0) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_append_sharded: bad sharding plan");
    if (uint64_t(base_pos) + n_tokens > 0xFFFFFFFFull)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_append_sharded: base_pos + n_tokens overflows");
    // the context-overflow check of src/backend/vulkan/decode.rs:523-533, on this rank's share
    if (n_tokens && vfkv_shard_local_len(world, page, uint64_t(base_pos) + n_tokens, rank) > cache->kv.config.max_seq_len)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_append_sharded: this rank's rows exceed max_seq_len");
    AppendArgs a = make_append(cache, layer, d_k, d_v);
    a.n_rows = n_tokens; a.slot = slot; a.base_pos = base_pos;
    a.shard_world = world; a.shard_rank = rank; a.shard_page = page;
    DeviceGuard g(ctx->device);
    return launch_append(ctx, a, as_stream(stream));
}

int32_t vfkv_append_batch(vfkv_cache *cache, uint32_t layer, const float *d_k, const float *d_v,
                          const uint32_t *d_slot_ids, const uint32_t *d_positions, uint32_t n_seqs, void *stream)
{
    int32_t rc = check_layer(cache, layer, "vfkv_append_batch");
    if (rc) return rc;
    vfkv_ctx *ctx = cache->ctx;
    if (!d_k || !d_v || !d_positions) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_append_batch: null argument");
    if ((reinterpret_cast<uintptr_t>(d_k) | reinterpret_cast<uintptr_t>(d_v)) % 16 != 0)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_append_batch: K and V inputs must be 16-byte aligned");
    AppendArgs a = make_append(cache, layer, d_k, d_v);
    a.n_rows = n_seqs; a.slot_ids = d_slot_ids; a.positions = d_positions;
    DeviceGuard g(ctx->device);
    return launch_append(ctx, a, as_stream(stream));
}

int32_t vfkv_fp8_to_f16(vfkv_cache *cache, uint32_t slot, uint32_t layer, uint32_t n_positions, void *d_k_out,
                        void *d_v_out, void *stream)
{
    int32_t rc = check_layer(cache, layer, "vfkv_fp8_to_f16");
    if (rc) return rc;
    vfkv_ctx *ctx = cache->ctx;
    KvCache &kv = cache->kv;
    if (!kv.is_fp8()) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_fp8_to_f16: cache is not FP8");
    if (slot >= kv.config.n_slots || n_positions > kv.config.max_seq_len)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_fp8_to_f16: slot or n_positions out of range");
    if (!d_k_out || !d_v_out) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_fp8_to_f16: null output");
    const uint64_t off = kv.slot_offset_bytes(layer, slot);
    const uint64_t n = uint64_t(n_positions) * kv.kv_heads_for(layer) * kv.head_dim_for(layer);
    DeviceGuard g(ctx->device);
    rc = launch_fp8_to_f16(ctx, static_cast<uint8_t *>(kv.k_buffer) + off, d_k_out, n, as_stream(stream));
    if (rc) return rc;
    return launch_fp8_to_f16(ctx, static_cast<uint8_t *>(kv.v_buffer) + off, d_v_out, n, as_stream(stream));
}

static int32_t attend_common(vfkv_cache *cache, uint32_t layer, uint32_t kv_layer, uint32_t n_q_heads,
                             const char *fn)
{
    int32_t rc = check_layer(cache, layer, fn);
    if (rc) return rc;
    rc = check_layer(cache, kv_layer, fn);
    if (rc) return rc;
    KvCache &kv = cache->kv;
    // run_scalar_attn takes head_dim from `layer` and the slab from `kv_layer`
    // (runs.rs:734-741); a publisher and its subscribers share one shape.
    if (kv.head_dim_for(layer) != kv.head_dim_for(kv_layer) || kv.kv_heads_for(layer) != kv.kv_heads_for(kv_layer))
        return set_error(cache->ctx, VFKV_ERR_INVALID, std::string(fn) + ": layer and kv_layer differ in shape");
    if (n_q_heads == 0 || kv.kv_heads_for(layer) == 0 || n_q_heads % kv.kv_heads_for(layer) != 0)
        return set_error(cache->ctx, VFKV_ERR_INVALID, std::string(fn) + ": n_q_heads must be a multiple of the layer's kv heads");
    return VFKV_OK;
}

int32_t vfkv_attend(vfkv_cache *cache, vfkv_workspace *ws, uint32_t layer, uint32_t kv_layer, const float *d_q,
                    float *d_out, uint32_t n_q_heads, uint32_t slot, uint32_t seq_len, uint32_t kv_start,
                    float scale, float softcap, uint32_t n_splits, void *stream)
{
    int32_t rc = attend_common(cache, layer, kv_layer, n_q_heads, "vfkv_attend");
    if (rc) return rc;
    vfkv_ctx *ctx = cache->ctx;
    if (!d_q || !d_out) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_attend: null Q or output");
    if (slot >= cache->kv.config.n_slots) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_attend: slot out of range");
    if (seq_len > cache->kv.config.max_seq_len) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_attend: seq_len exceeds max_seq_len");
    if (kv_start > seq_len) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_attend: kv_start exceeds seq_len");
    AttnArgs a;
    a.kv = make_view(cache, kv_layer);
    a.seq.n_seqs = 1; a.seq.slot0 = slot; a.seq.seq_len_scalar = seq_len; a.seq.kv_start_scalar = kv_start;
    a.q = d_q; a.out = d_out; a.n_q_heads = n_q_heads; a.scale = scale; a.softcap = softcap; a.n_splits = n_splits;
    DeviceGuard g(ctx->device);
    return launch_attention(ctx, ws, a, as_stream(stream));
}

int32_t vfkv_attend_batch(vfkv_cache *cache, vfkv_workspace *ws, uint32_t layer, uint32_t kv_layer,
                          const float *d_q, float *d_out, uint32_t n_q_heads, const uint32_t *d_slot_ids,
                          const uint32_t *d_seq_lens, const uint32_t *d_kv_starts, uint32_t n_seqs,
                          uint32_t max_seq_len_hint, float scale, float softcap, uint32_t n_splits, void *stream)
{
    int32_t rc = attend_common(cache, layer, kv_layer, n_q_heads, "vfkv_attend_batch");
    if (rc) return rc;
    vfkv_ctx *ctx = cache->ctx;
    if (!d_q || !d_out || !d_seq_lens) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_attend_batch: null argument");
    AttnArgs a;
    a.kv = make_view(cache, kv_layer);
    a.seq.n_seqs = n_seqs; a.seq.slot_ids = d_slot_ids; a.seq.seq_lens = d_seq_lens; a.seq.kv_starts = d_kv_starts;
    a.seq.max_len_hint = max_seq_len_hint;
    a.q = d_q; a.out = d_out; a.n_q_heads = n_q_heads; a.scale = scale; a.softcap = softcap; a.n_splits = n_splits;
    DeviceGuard g(ctx->device);
    return launch_attention(ctx, ws, a, as_stream(stream));
}

int32_t vfkv_decode_step(vfkv_cache *cache, vfkv_workspace *ws, uint32_t layer, const float *d_q, const float *d_k,
                         const float *d_v, float *d_out, uint32_t n_q_heads, const uint32_t *d_slot_ids,
                         const uint32_t *d_positions, uint32_t n_seqs, uint32_t max_seq_len_hint, uint32_t window,
                         float scale, float softcap, uint32_t n_splits, void *stream)
{
    int32_t rc = attend_common(cache, layer, layer, n_q_heads, "vfkv_decode_step");
    if (rc) return rc;
    vfkv_ctx *ctx = cache->ctx;
    if (!d_q || !d_k || !d_v || !d_out || !d_positions)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_decode_step: null argument");
    if ((reinterpret_cast<uintptr_t>(d_k) | reinterpret_cast<uintptr_t>(d_v)) % 16 != 0)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_decode_step: K and V inputs must be 16-byte aligned");
    AttnArgs a;
    a.kv = make_view(cache, layer);
    a.seq.n_seqs = n_seqs; a.seq.slot_ids = d_slot_ids; a.seq.positions = d_positions; a.seq.window = window;
    a.seq.max_len_hint = max_seq_len_hint;
    a.q = d_q; a.out = d_out; a.n_q_heads = n_q_heads; a.scale = scale; a.softcap = softcap; a.n_splits = n_splits;
    // The tensor-core kernel stores the new rows itself (one launch per layer); otherwise the
    // append runs first, as KvWrite precedes Attention in the reference's layer plan.
    const bool fused = ctx->attn_impl != 1 && attn_mma_supported(a);
    if (fused) {
        a.k_new = d_k;
        a.v_new = d_v;
    } else {
        rc = vfkv_append_batch(cache, layer, d_k, d_v, d_slot_ids, d_positions, n_seqs, stream);
        if (rc) return rc;
    }
    DeviceGuard g(ctx->device);
    return launch_attention(ctx, ws, a, as_stream(stream));
}

int32_t vfkv_decode_token(vfkv_cache *cache, vfkv_workspace *ws, const float *d_q, const float *d_k, const float *d_v,
                          float *d_out, uint32_t n_q_heads, const uint32_t *d_slot_ids, const uint32_t *d_positions,
                          uint32_t n_seqs, uint32_t max_seq_len_hint, const uint32_t *windows, float scale,
                          float softcap, uint32_t n_splits, void *stream)
{
    if (!cache) return VFKV_ERR_INVALID;
    vfkv_ctx *ctx = cache->ctx;
    KvCache &kv = cache->kv;
    if (kv.layer_byte_offsets) return set_error(ctx, VFKV_ERR_UNSUPPORTED, "vfkv_decode_token: uniform-shape caches only");
    const uint32_t L = kv.config.n_layers, D = kv.config.head_dim, Hkv = kv.config.n_kv_heads;
    const uint64_t q_stride = uint64_t(n_seqs) * n_q_heads * D, kv_stride = uint64_t(n_seqs) * Hkv * D;
    for (uint32_t l = 0; l < L; ++l) {
        int32_t rc = vfkv_decode_step(cache, ws, l, d_q + l * q_stride, d_k + l * kv_stride, d_v + l * kv_stride,
                                      d_out + l * q_stride, n_q_heads, d_slot_ids, d_positions, n_seqs,
                                      max_seq_len_hint, windows ? windows[l] : 0, scale, softcap, n_splits, stream);
        if (rc) return rc;
    }
    return VFKV_OK;
}

int32_t vfkv_decode_token_host(vfkv_cache *cache, vfkv_workspace *ws, const float *h_q, const float *h_k,
                               const float *h_v, float *h_out, uint32_t n_q_heads, const uint32_t *h_slot_ids,
                               const uint32_t *h_positions, uint32_t n_seqs, const uint32_t *windows, float scale,
                               float softcap, uint32_t n_splits, void *stream)
{
    if (!cache || !ws) return VFKV_ERR_INVALID;
    vfkv_ctx *ctx = cache->ctx;
    KvCache &kv = cache->kv;
    if (!h_q || !h_k || !h_v || !h_out || !h_positions)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_decode_token_host: null argument");
    if (kv.layer_byte_offsets) return set_error(ctx, VFKV_ERR_UNSUPPORTED, "vfkv_decode_token_host: uniform-shape caches only");
    if (n_seqs == 0 || n_seqs > ws->max_seqs) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_decode_token_host: n_seqs outside the workspace");
    uint32_t max_pos = 0;
    for (uint32_t i = 0; i < n_seqs; ++i) {
        if (h_positions[i] >= kv.config.max_seq_len) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_decode_token_host: position exceeds max_seq_len");
        if (h_slot_ids && h_slot_ids[i] >= kv.config.n_slots) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_decode_token_host: slot out of range");
        if (!h_slot_ids && i >= kv.config.n_slots) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_decode_token_host: more sequences than slots");
        max_pos = h_positions[i] > max_pos ? h_positions[i] : max_pos;
    }
    const uint32_t L = kv.config.n_layers, D = kv.config.head_dim, Hkv = kv.config.n_kv_heads;
    const uint64_t q_elems = uint64_t(L) * n_seqs * n_q_heads * D, kv_elems = uint64_t(L) * n_seqs * Hkv * D;
    const uint64_t in_bytes = (q_elems + 2 * kv_elems) * 4, out_bytes = q_elems * 4;
    DeviceGuard g(ctx->device);
    cudaStream_t st = as_stream(stream);
    if (ws->stage_in_bytes < in_bytes) {
        cudaStreamSynchronize(st);
        cudaFree(ws->stage_in);
        ws->stage_in = nullptr; ws->stage_in_bytes = 0;
        cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&ws->stage_in), in_bytes);
        if (e != cudaSuccess) return check_cuda(ctx, e, "vfkv_decode_token_host: staging");
        ws->stage_in_bytes = in_bytes;
    }
    if (ws->stage_out_bytes < out_bytes) {
        cudaStreamSynchronize(st);
        cudaFree(ws->stage_out);
        ws->stage_out = nullptr; ws->stage_out_bytes = 0;
        cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&ws->stage_out), out_bytes);
        if (e != cudaSuccess) return check_cuda(ctx, e, "vfkv_decode_token_host: staging");
        ws->stage_out_bytes = out_bytes;
    }
    float *dq = ws->stage_in, *dk = dq + q_elems, *dv = dk + kv_elems;
    uint32_t *d_pos = ws->d_u32, *d_slots = ws->d_u32 + ws->max_seqs;
    cudaError_t e = cudaMemcpyAsync(d_pos, h_positions, n_seqs * 4, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess && h_slot_ids) e = cudaMemcpyAsync(d_slots, h_slot_ids, n_seqs * 4, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return check_cuda(ctx, e, "vfkv_decode_token_host: H2D");
    const uint64_t q_stride = uint64_t(n_seqs) * n_q_heads * D, kv_stride = uint64_t(n_seqs) * Hkv * D;
    // The launches of one token depend on the host only through the configuration below
    // (positions and slots are device-side inputs; the length hint is rounded up so that it
    // changes rarely): capture them once, replay afterwards.
    uint32_t hint = (max_pos + 1 + 1023u) / 1024u * 1024u;
    if (hint > kv.config.max_seq_len) hint = kv.config.max_seq_len;
    uint64_t wh = 1469598103934665603ull;
    auto mix = [&](uint64_t x) { wh = (wh ^ x) * 1099511628211ull; };
    for (uint32_t l = 0; windows && l < L; ++l) mix(windows[l]);
    // a cache object re-created at the same address must not find the old graphs
    mix(reinterpret_cast<uint64_t>(kv.k_buffer)); mix(reinterpret_cast<uint64_t>(kv.v_buffer));
    mix(L); mix(D); mix(Hkv); mix(uint64_t(kv.kv_dtype)); mix(kv.config.max_seq_len); mix(kv.config.n_slots);
    mix(reinterpret_cast<uint64_t>(ws->part_o)); mix(reinterpret_cast<uint64_t>(dk));
    uint32_t fs, fc;
    memcpy(&fs, &scale, 4); memcpy(&fc, &softcap, 4);
    const uint64_t key[8] = {reinterpret_cast<uint64_t>(cache), reinterpret_cast<uint64_t>(dq),
                             reinterpret_cast<uint64_t>(ws->stage_out),
                             uint64_t(n_q_heads) << 32 | n_seqs, uint64_t(hint) << 32 | n_splits,
                             uint64_t(fs) << 32 | fc, wh ^ (h_slot_ids ? 1u : 0u),
                             uint64_t(ctx->pdl) | uint64_t(ctx->tune_warps) << 8 | uint64_t(ctx->tune_stages) << 16 |
                                 uint64_t(ctx->attn_impl) << 24 | uint64_t(ctx->cluster_merge) << 32 |
                                 uint64_t(reinterpret_cast<uintptr_t>(st) & 0xffffffu) << 40};
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(st, &cap);
    bool graphable = cap == cudaStreamCaptureStatusNone && !ctx->profiling && !ctx->d_trace && st != nullptr;
    // The layers are cut into up to four groups, one graph each: the inputs of group c + 1 cross
    // the bus on a second stream while group c computes, and the outputs of group c go back while
    // group c + 1 computes.  Only the first group's inputs and the last group's outputs are exposed.
    const uint32_t n_chunks = L < vfkv_workspace::kTokChunks ? L : vfkv_workspace::kTokChunks;
    auto chunk_begin = [&](uint32_t c) { return uint32_t(uint64_t(L) * c / n_chunks); };
    auto run_layers = [&](uint32_t l0, uint32_t l1, uint32_t len_hint) -> int32_t {
        for (uint32_t l = l0; l < l1; ++l) {
            int32_t rc = vfkv_decode_step(cache, ws, l, dq + l * q_stride, dk + l * kv_stride, dv + l * kv_stride,
                                          ws->stage_out + l * q_stride, n_q_heads, h_slot_ids ? d_slots : nullptr,
                                          d_pos, n_seqs, len_hint, windows ? windows[l] : 0, scale, softcap,
                                          n_splits, stream);
            if (rc) return rc;
        }
        return VFKV_OK;
    };
    if (graphable && !ws->copy_stream) {
        bool ok = cudaStreamCreateWithFlags(&ws->copy_stream, cudaStreamNonBlocking) == cudaSuccess;
        for (uint32_t i = 0; ok && i < 2 * vfkv_workspace::kTokChunks; ++i)
            ok = cudaEventCreateWithFlags(&ws->tok_events[i], cudaEventDisableTiming) == cudaSuccess;
        if (!ok) { cudaGetLastError(); graphable = false; }
    }
    if (graphable && (!ws->tok_graphs[0] || memcmp(key, ws->tok_key, sizeof(key)) != 0)) {
        for (auto &gexec : ws->tok_graphs)
            if (gexec) { cudaGraphExecDestroy(gexec); gexec = nullptr; }
        for (uint32_t c = 0; c < n_chunks; ++c) {
            cudaGraph_t graph = nullptr;
            if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { cudaGetLastError(); break; }
            const uint64_t launches = ctx->launches;
            int32_t rc = run_layers(chunk_begin(c), chunk_begin(c + 1), hint);
            cudaError_t ce = cudaStreamEndCapture(st, &graph);
            ctx->launches = launches;                           // recorded, not run
            const bool ok = rc == VFKV_OK && ce == cudaSuccess && graph &&
                            cudaGraphInstantiate(&ws->tok_graphs[c], graph, 0) == cudaSuccess;
            if (graph) cudaGraphDestroy(graph);
            cudaGetLastError();
            if (rc) return rc;
            if (!ok) { ws->tok_graphs[c] = nullptr; break; }
        }
        bool all = true;
        for (uint32_t c = 0; c < n_chunks; ++c) all = all && ws->tok_graphs[c];
        if (all) memcpy(ws->tok_key, key, sizeof(key));
        else {
            for (auto &gexec : ws->tok_graphs)
                if (gexec) { cudaGraphExecDestroy(gexec); gexec = nullptr; }
        }
    }
    if (graphable && ws->tok_graphs[0]) {
        cudaStream_t cs = ws->copy_stream;
        cudaEvent_t *ev_in = ws->tok_events, *ev_done = ws->tok_events + vfkv_workspace::kTokChunks;
        // The staging buffers belong to the workspace and every earlier call drained both streams,
        // so the first copies need not wait for the caller's stream.  Each group's launch is issued
        // as soon as its own copies are queued: the host calls for the later groups then run while
        // the first group computes.  On the copy stream the order is in(0) in(1) out(0) in(2) out(1)
        // ..., so an input copy never waits for a group that has not started.
        auto copy_in = [&](uint32_t c) {
            const uint32_t l0 = chunk_begin(c), nl = chunk_begin(c + 1) - l0;
            cudaError_t ce = cudaMemcpyAsync(dq + l0 * q_stride, h_q + l0 * q_stride, nl * q_stride * 4, cudaMemcpyHostToDevice, cs);
            if (ce == cudaSuccess) ce = cudaMemcpyAsync(dk + l0 * kv_stride, h_k + l0 * kv_stride, nl * kv_stride * 4, cudaMemcpyHostToDevice, cs);
            if (ce == cudaSuccess) ce = cudaMemcpyAsync(dv + l0 * kv_stride, h_v + l0 * kv_stride, nl * kv_stride * 4, cudaMemcpyHostToDevice, cs);
            if (ce == cudaSuccess) ce = cudaEventRecord(ev_in[c], cs);
            return ce;
        };
        e = copy_in(0);
        for (uint32_t c = 0; c < n_chunks && e == cudaSuccess; ++c) {
            const uint32_t l0 = chunk_begin(c), nl = chunk_begin(c + 1) - l0;
            e = cudaStreamWaitEvent(st, ev_in[c], 0);
            if (e == cudaSuccess) e = cudaGraphLaunch(ws->tok_graphs[c], st);
            if (e == cudaSuccess) e = cudaEventRecord(ev_done[c], st);
            if (e == cudaSuccess) ctx->launches += nl;
            if (e == cudaSuccess && c + 1 < n_chunks) e = copy_in(c + 1);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(cs, ev_done[c], 0);
            if (e == cudaSuccess) e = cudaMemcpyAsync(h_out + l0 * q_stride, ws->stage_out + l0 * q_stride, nl * q_stride * 4, cudaMemcpyDeviceToHost, cs);
        }
        // The last output copy follows the last group, so the copy stream finishing means the step
        // is complete; the caller's stream is drained as well, also after an error, so that
        // nothing of this call is left in flight.
        cudaError_t e2 = cudaStreamSynchronize(cs);
        cudaError_t e3 = cudaStreamSynchronize(st);
        if (e == cudaSuccess) e = e2 != cudaSuccess ? e2 : e3;
        return check_cuda(ctx, e, "vfkv_decode_token_host: pipelined step");
    }
    // stream order only (inside a capture, under the profiler or with the phase trace on)
    e = cudaMemcpyAsync(dq, h_q, q_elems * 4, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dk, h_k, kv_elems * 4, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dv, h_v, kv_elems * 4, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return check_cuda(ctx, e, "vfkv_decode_token_host: H2D");
    if (int32_t rc = run_layers(0, L, max_pos + 1)) return rc;
    e = cudaMemcpyAsync(h_out, ws->stage_out, out_bytes, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    return check_cuda(ctx, e, "vfkv_decode_token_host: D2H");
}

/* ---- the same step without waiting: two tokens in flight ------------------------------------- */

int32_t vfkv_decode_token_host_submit(vfkv_cache *cache, vfkv_workspace *ws, const float *h_q, const float *h_k,
                                      const float *h_v, float *h_out, uint32_t n_q_heads, const uint32_t *h_slot_ids,
                                      const uint32_t *h_positions, uint32_t n_seqs, const uint32_t *windows,
                                      float scale, float softcap, uint32_t n_splits, void *stream, uint64_t *ticket)
{
    if (!cache || !ws) return VFKV_ERR_INVALID;
    vfkv_ctx *ctx = cache->ctx;
    KvCache &kv = cache->kv;
    if (!h_q || !h_k || !h_v || !h_out || !h_positions || !ticket)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_decode_token_host_submit: null argument");
    *ticket = 0;
    if (!stream) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_decode_token_host_submit: needs a stream of its own, not the default stream");
    if (kv.layer_byte_offsets) return set_error(ctx, VFKV_ERR_UNSUPPORTED, "vfkv_decode_token_host_submit: uniform-shape caches only");
    if (n_seqs == 0 || n_seqs > ws->max_seqs) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_decode_token_host_submit: n_seqs outside the workspace");
    if (ctx->profiling || ctx->d_trace)
        return set_error(ctx, VFKV_ERR_UNSUPPORTED, "vfkv_decode_token_host_submit: not while profiling or tracing");
    uint32_t max_pos = 0;
    for (uint32_t i = 0; i < n_seqs; ++i) {
        if (h_positions[i] >= kv.config.max_seq_len) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_decode_token_host_submit: position exceeds max_seq_len");
        if (h_slot_ids && h_slot_ids[i] >= kv.config.n_slots) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_decode_token_host_submit: slot out of range");
        if (!h_slot_ids && i >= kv.config.n_slots) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_decode_token_host_submit: more sequences than slots");
        max_pos = h_positions[i] > max_pos ? h_positions[i] : max_pos;
    }
    vfkv_workspace::HostSlot *hs = nullptr;
    for (auto &cand : ws->host_slot)
        if (cand.ticket == 0) { hs = &cand; break; }
    if (!hs) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_decode_token_host_submit: two tokens are in flight; wait for one first");
    const uint32_t L = kv.config.n_layers, D = kv.config.head_dim, Hkv = kv.config.n_kv_heads;
    const uint64_t q_elems = uint64_t(L) * n_seqs * n_q_heads * D, kv_elems = uint64_t(L) * n_seqs * Hkv * D;
    const uint64_t in_bytes = (q_elems + 2 * kv_elems) * 4, out_bytes = q_elems * 4;
    DeviceGuard g(ctx->device);
    cudaStream_t st = as_stream(stream);
    cudaError_t e = cudaSuccess;
    if (!ws->h2d_stream) {
        e = cudaStreamCreateWithFlags(&ws->h2d_stream, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ws->d2h_stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) return check_cuda(ctx, e, "vfkv_decode_token_host_submit: streams");
    }
    if (!hs->ev_in) {
        e = cudaEventCreateWithFlags(&hs->ev_in, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&hs->ev_done, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&hs->ev_out, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&hs->u32), uint64_t(ws->max_seqs) * 2 * 4);
        if (e != cudaSuccess) return check_cuda(ctx, e, "vfkv_decode_token_host_submit: events");
    }
    // staging grows on first use (a free slot has nothing in flight, so this cannot pull memory from
    // under a running step)
    if (hs->in_bytes < in_bytes) {
        cudaFree(hs->in); hs->in = nullptr; hs->in_bytes = 0;
        e = cudaMalloc(reinterpret_cast<void **>(&hs->in), in_bytes);
        if (e != cudaSuccess) return check_cuda(ctx, e, "vfkv_decode_token_host_submit: staging");
        hs->in_bytes = in_bytes;
    }
    if (hs->out_bytes < out_bytes) {
        cudaFree(hs->out); hs->out = nullptr; hs->out_bytes = 0;
        e = cudaMalloc(reinterpret_cast<void **>(&hs->out), out_bytes);
        if (e != cudaSuccess) return check_cuda(ctx, e, "vfkv_decode_token_host_submit: staging");
        hs->out_bytes = out_bytes;
    }
    float *dq = hs->in, *dk = dq + q_elems, *dv = dk + kv_elems;
    uint32_t *d_pos = hs->u32, *d_slots = hs->u32 + ws->max_seqs;
    const uint64_t q_stride = uint64_t(n_seqs) * n_q_heads * D, kv_stride = uint64_t(n_seqs) * Hkv * D;
    uint32_t hint = (max_pos + 1 + 1023u) / 1024u * 1024u;
    if (hint > kv.config.max_seq_len) hint = kv.config.max_seq_len;
    uint64_t wh = 1469598103934665603ull;
    auto mix = [&](uint64_t x) { wh = (wh ^ x) * 1099511628211ull; };
    for (uint32_t l = 0; windows && l < L; ++l) mix(windows[l]);
    mix(reinterpret_cast<uint64_t>(kv.k_buffer)); mix(reinterpret_cast<uint64_t>(kv.v_buffer));
    mix(L); mix(D); mix(Hkv); mix(uint64_t(kv.kv_dtype)); mix(kv.config.max_seq_len); mix(kv.config.n_slots);
    mix(reinterpret_cast<uint64_t>(ws->tag_part));
    uint32_t fs, fc;
    memcpy(&fs, &scale, 4); memcpy(&fc, &softcap, 4);
    const uint64_t key[8] = {reinterpret_cast<uint64_t>(cache), reinterpret_cast<uint64_t>(dq),
                             reinterpret_cast<uint64_t>(hs->out), uint64_t(n_q_heads) << 32 | n_seqs,
                             uint64_t(hint) << 32 | n_splits, uint64_t(fs) << 32 | fc, wh ^ (h_slot_ids ? 1u : 0u),
                             uint64_t(ctx->pdl) | uint64_t(ctx->tune_warps) << 8 | uint64_t(ctx->tune_stages) << 16 |
                                 uint64_t(ctx->attn_impl) << 24 | uint64_t(ctx->cluster_merge) << 32 |
                                 uint64_t(reinterpret_cast<uintptr_t>(st) & 0xffffffu) << 40};
    if (!hs->graph || memcmp(key, hs->key, sizeof(key)) != 0) {
        if (hs->graph) { cudaGraphExecDestroy(hs->graph); hs->graph = nullptr; }
        cudaGraph_t graph = nullptr;
        e = cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal);
        if (e != cudaSuccess) return check_cuda(ctx, e, "vfkv_decode_token_host_submit: capture");
        const uint64_t launches = ctx->launches;
        int32_t rc = VFKV_OK;
        for (uint32_t l = 0; l < L && rc == VFKV_OK; ++l)
            rc = vfkv_decode_step(cache, ws, l, dq + l * q_stride, dk + l * kv_stride, dv + l * kv_stride,
                                  hs->out + l * q_stride, n_q_heads, h_slot_ids ? d_slots : nullptr, d_pos, n_seqs, hint,
                                  windows ? windows[l] : 0, scale, softcap, n_splits, stream);
        hs->launches = uint32_t(ctx->launches - launches);
        ctx->launches = launches;                               // recorded, not run
        cudaError_t ce = cudaStreamEndCapture(st, &graph);
        if (rc == VFKV_OK && ce == cudaSuccess && graph) ce = cudaGraphInstantiate(&hs->graph, graph, 0);
        if (graph) cudaGraphDestroy(graph);
        if (rc != VFKV_OK) return rc;
        if (ce != cudaSuccess || !hs->graph) { hs->graph = nullptr; return check_cuda(ctx, ce != cudaSuccess ? ce : cudaErrorUnknown, "vfkv_decode_token_host_submit: graph"); }
        memcpy(hs->key, key, sizeof(key));
    }
    // inputs on their own stream, the layers on the caller's, the outputs on a third: the copies of
    // one token run beside the layers of the other
    e = cudaMemcpyAsync(d_pos, h_positions, n_seqs * 4, cudaMemcpyHostToDevice, ws->h2d_stream);
    if (e == cudaSuccess && h_slot_ids) e = cudaMemcpyAsync(d_slots, h_slot_ids, n_seqs * 4, cudaMemcpyHostToDevice, ws->h2d_stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dq, h_q, q_elems * 4, cudaMemcpyHostToDevice, ws->h2d_stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dk, h_k, kv_elems * 4, cudaMemcpyHostToDevice, ws->h2d_stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dv, h_v, kv_elems * 4, cudaMemcpyHostToDevice, ws->h2d_stream);
    if (e == cudaSuccess) e = cudaEventRecord(hs->ev_in, ws->h2d_stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(st, hs->ev_in, 0);
    if (e == cudaSuccess) e = cudaGraphLaunch(hs->graph, st);
    if (e == cudaSuccess) e = cudaEventRecord(hs->ev_done, st);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(ws->d2h_stream, hs->ev_done, 0);
    if (e == cudaSuccess) e = cudaMemcpyAsync(h_out, hs->out, out_bytes, cudaMemcpyDeviceToHost, ws->d2h_stream);
    if (e == cudaSuccess) e = cudaEventRecord(hs->ev_out, ws->d2h_stream);
    if (e != cudaSuccess) {
        // leave nothing of this call in flight
        cudaStreamSynchronize(ws->h2d_stream); cudaStreamSynchronize(st); cudaStreamSynchronize(ws->d2h_stream);
        return check_cuda(ctx, e, "vfkv_decode_token_host_submit");
    }
    ctx->launches += hs->launches;
    hs->ticket = ws->next_ticket++;
    *ticket = hs->ticket;
    return VFKV_OK;
}

int32_t vfkv_decode_token_host_wait(vfkv_workspace *ws, uint64_t ticket)
{
    if (!ws || ticket == 0) return VFKV_ERR_INVALID;
    for (auto &hs : ws->host_slot) {
        if (hs.ticket != ticket) continue;
        DeviceGuard g(ws->ctx->device);
        cudaError_t e = cudaEventSynchronize(hs.ev_out);
        hs.ticket = 0;
        return check_cuda(ws->ctx, e, "vfkv_decode_token_host_wait");
    }
    return set_error(ws->ctx, VFKV_ERR_INVALID, "vfkv_decode_token_host_wait: no such ticket in flight");
}

/* ---- sequence-dimension sharding ------------------------------------------ */

int32_t vfkv_attend_partial(vfkv_cache *cache, vfkv_workspace *ws, uint32_t layer, uint32_t kv_layer,
                            const float *d_q, uint32_t n_q_heads, uint32_t slot, uint32_t pos_begin,
                            uint32_t pos_end, float scale, float softcap, uint32_t n_splits, float *d_m,
                            float *d_l, float *d_o, void *stream)
{
    int32_t rc = attend_common(cache, layer, kv_layer, n_q_heads, "vfkv_attend_partial");
    if (rc) return rc;
    vfkv_ctx *ctx = cache->ctx;
    if (!d_q || !d_m || !d_l || !d_o) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_attend_partial: null argument");
    if (slot >= cache->kv.config.n_slots || pos_end > cache->kv.config.max_seq_len || pos_begin > pos_end)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_attend_partial: slot or position range out of bounds");
    AttnArgs a;
    a.kv = make_view(cache, kv_layer);
    a.seq.n_seqs = 1; a.seq.slot0 = slot; a.seq.seq_len_scalar = pos_end; a.seq.kv_start_scalar = pos_begin;
    a.q = d_q; a.out_m = d_m; a.out_l = d_l; a.out_o = d_o; a.n_q_heads = n_q_heads; a.scale = scale;
    a.softcap = softcap; a.n_splits = n_splits;
    DeviceGuard g(ctx->device);
    return launch_attention(ctx, ws, a, as_stream(stream));
}

// ---- the same exchange through a collective library -----------------------------------------------
// ncclAllGather is looked up in the NCCL that the process has loaded (or can load) the first time
// it is needed; the library itself links no collective library.
namespace {
typedef int (*NcclAllGatherFn)(const void *, void *, size_t, int, void *, cudaStream_t);
NcclAllGatherFn find_nccl_all_gather()
{
    static std::mutex mu;
    static bool looked = false;
    static NcclAllGatherFn fn = nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!looked) {
        looked = true;
        void *sym = dlsym(RTLD_DEFAULT, "ncclAllGather");
        if (!sym) {
            void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
            if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
            if (h) sym = dlsym(h, "ncclAllGather");
        }
        fn = reinterpret_cast<NcclAllGatherFn>(sym);
    }
    return fn;
}
}  // namespace

int32_t vfkv_attend_allgather(vfkv_cache *cache, vfkv_workspace *ws, void *nccl_comm, uint32_t world, uint32_t rank,
                              uint32_t layer, uint32_t kv_layer, const float *d_q, uint32_t n_q_heads, uint32_t slot,
                              uint32_t pos_begin, uint32_t pos_end, float scale, float softcap, uint32_t n_splits,
                              float *d_packed, float *d_out, void *stream)
{
    int32_t rc = attend_common(cache, layer, kv_layer, n_q_heads, "vfkv_attend_allgather");
    if (rc) return rc;
    vfkv_ctx *ctx = cache->ctx;
    if (!nccl_comm || !d_packed || !d_out) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_attend_allgather: null argument");
    if (world == 0 || rank >= world) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_attend_allgather: rank outside the world");
    NcclAllGatherFn all_gather = find_nccl_all_gather();
    if (!all_gather) return set_error(ctx, VFKV_ERR_UNSUPPORTED, "vfkv_attend_allgather: no NCCL library in this process (ncclAllGather not found)");
    const uint32_t D = cache->kv.head_dim_for(kv_layer);
    const uint64_t block = uint64_t(n_q_heads) * (D + 2);        // m[rows], l[rows], o[rows][D] of one rank
    float *mine = d_packed + uint64_t(rank) * block;
    rc = vfkv_attend_partial(cache, ws, layer, kv_layer, d_q, n_q_heads, slot, pos_begin, pos_end, scale, softcap,
                             n_splits, mine, mine + n_q_heads, mine + 2ull * n_q_heads, stream);
    if (rc) return rc;
    DeviceGuard g(ctx->device);
    const int nrc = all_gather(mine, d_packed, size_t(block), /* ncclFloat32 */ 7, nccl_comm, as_stream(stream));
    if (nrc != 0) return set_error(ctx, VFKV_ERR_CUDA, "vfkv_attend_allgather: ncclAllGather failed with code " + std::to_string(nrc));
    return launch_merge_partials_packed(ctx, d_packed, world, n_q_heads, D, d_out, as_stream(stream));
}

// Shared by vfkv_attend_push (fused = false) and vfkv_attend_exchange (fused = true).
static int32_t attend_push_impl(vfkv_cache *cache, vfkv_workspace *ws, vfkv_exchange *ex, uint32_t layer,
                                uint32_t kv_layer, const float *d_q, const float *d_k_new, const float *d_v_new,
                                uint32_t n_q_heads, uint32_t slot, uint32_t pos_begin, uint32_t pos_end, float scale,
                                float softcap, uint32_t n_splits, float *d_out, bool fused, bool *did_fuse,
                                void *stream, const char *fn)
{
    if (did_fuse) *did_fuse = false;
    int32_t rc = attend_common(cache, layer, kv_layer, n_q_heads, fn);
    if (rc) return rc;
    vfkv_ctx *ctx = cache->ctx;
    const std::string name(fn);
    if (!d_q || !ex) return set_error(ctx, VFKV_ERR_INVALID, name + ": null argument");
    if (ex->ctx != ctx) return set_error(ctx, VFKV_ERR_INVALID, name + ": exchange belongs to another context");
    if (!vfkv_exchange_ready(ex)) return set_error(ctx, VFKV_ERR_INVALID, name + ": not every rank's buffer is set");
    if (slot >= cache->kv.config.n_slots || pos_end > cache->kv.config.max_seq_len || pos_begin > pos_end)
        return set_error(ctx, VFKV_ERR_INVALID, name + ": slot or position range out of bounds");
    const bool has_new = d_k_new || d_v_new;
    if (has_new && (!d_k_new || !d_v_new || pos_end == 0 || pos_begin == pos_end || kv_layer != layer))
        return set_error(ctx, VFKV_ERR_INVALID, name + ": a new token needs both K and V, a non-empty range and kv_layer == layer");
    if ((reinterpret_cast<uintptr_t>(d_k_new) | reinterpret_cast<uintptr_t>(d_v_new)) % 16 != 0)
        return set_error(ctx, VFKV_ERR_INVALID, name + ": K and V inputs must be 16-byte aligned");
    AttnArgs a;
    a.kv = make_view(cache, kv_layer);
    if (ex->fan.n_rows != n_q_heads || ex->head_dim != a.kv.head_dim)
        return set_error(ctx, VFKV_ERR_INVALID, name + ": exchange was created for another shape");
    a.seq.n_seqs = 1; a.seq.slot0 = slot; a.seq.seq_len_scalar = pos_end; a.seq.kv_start_scalar = pos_begin;
    a.q = d_q; a.n_q_heads = n_q_heads; a.scale = scale; a.softcap = softcap; a.n_splits = n_splits;
    // the staged block has the layout of one exchange block, in plain floats
    a.out_m = ex->staging;
    a.out_l = ex->staging + n_q_heads;
    a.out_o = ex->staging + 2ull * n_q_heads;
    if (attn_mma_supported(a) && ctx->attn_impl != 1) {
        a.out_m = a.out_l = a.out_o = nullptr;          // the kernel stores into the exchange buffers itself,
        a.fan = ex->d_fan;                              // and writes the new token's cache row as well
        a.k_new = d_k_new;
        a.v_new = d_v_new;
        if (fused && reinterpret_cast<uintptr_t>(d_out) % 16 == 0) {
            // one launch per layer: the same kernel waits for the other ranks' blocks and writes the rows
            a.out = d_out;
            a.fan_merge = true;
            if (did_fuse) *did_fuse = true;
        }
        DeviceGuard g(ctx->device);
        rc = launch_attention(ctx, ws, a, as_stream(stream));
        if (rc == VFKV_ERR_UNSUPPORTED && a.fan_merge) {      // shape too large for the one-launch form: two launches
            a.out = nullptr;
            a.fan_merge = false;
            if (did_fuse) *did_fuse = false;
            rc = launch_attention(ctx, ws, a, as_stream(stream));
        }
        return rc;
    }
    if (has_new) {
        rc = vfkv_append(cache, layer, d_k_new, d_v_new, 1, slot, pos_end - 1, stream);
        if (rc) return rc;
    }
    DeviceGuard g(ctx->device);
    rc = launch_attention(ctx, ws, a, as_stream(stream));
    if (rc) return rc;
    return launch_fanout_push(ctx, ex->fan, ex->staging, ex->head_dim, as_stream(stream));
}

int32_t vfkv_attend_push(vfkv_cache *cache, vfkv_workspace *ws, vfkv_exchange *ex, uint32_t layer, uint32_t kv_layer,
                         const float *d_q, const float *d_k_new, const float *d_v_new, uint32_t n_q_heads,
                         uint32_t slot, uint32_t pos_begin, uint32_t pos_end, float scale, float softcap,
                         uint32_t n_splits, void *stream)
{
    return attend_push_impl(cache, ws, ex, layer, kv_layer, d_q, d_k_new, d_v_new, n_q_heads, slot, pos_begin, pos_end,
                            scale, softcap, n_splits, nullptr, false, nullptr, stream, "vfkv_attend_push");
}

int32_t vfkv_attend_exchange(vfkv_cache *cache, vfkv_workspace *ws, vfkv_exchange *ex, uint32_t layer,
                             uint32_t kv_layer, const float *d_q, const float *d_k_new, const float *d_v_new,
                             uint32_t n_q_heads, uint32_t slot, uint32_t pos_begin, uint32_t pos_end, float scale,
                             float softcap, uint32_t n_splits, float *d_out, void *stream)
{
    if (!d_out) return VFKV_ERR_INVALID;
    bool fused = false;
    int32_t rc = attend_push_impl(cache, ws, ex, layer, kv_layer, d_q, d_k_new, d_v_new, n_q_heads, slot, pos_begin,
                                  pos_end, scale, softcap, n_splits, d_out, true, &fused, stream,
                                  "vfkv_attend_exchange");
    if (rc || fused) return rc;
    return vfkv_exchange_merge(ex, d_out, stream);
}

int32_t vfkv_merge_partials(vfkv_ctx *ctx, const float *d_m, const float *d_l, const float *d_o, uint32_t n_parts,
                            uint32_t n_rows, uint32_t head_dim, float *d_out, void *stream)
{
    if (!ctx) return VFKV_ERR_INVALID;
    if (!d_m || !d_l || !d_o || !d_out) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_merge_partials: null argument");
    if (head_dim == 0 || head_dim > 512) return set_error(ctx, VFKV_ERR_UNSUPPORTED, "vfkv_merge_partials: head_dim must be 1..512");
    DeviceGuard g(ctx->device);
    return launch_merge_partials(ctx, d_m, d_l, d_o, n_parts, n_rows, head_dim, d_out, as_stream(stream));
}

int32_t vfkv_merge_partials_packed(vfkv_ctx *ctx, const float *d_packed, uint32_t n_parts, uint32_t n_rows,
                                   uint32_t head_dim, float *d_out, void *stream)
{
    if (!ctx) return VFKV_ERR_INVALID;
    if (!d_packed || !d_out) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_merge_partials_packed: null argument");
    if (head_dim == 0 || head_dim > 512) return set_error(ctx, VFKV_ERR_UNSUPPORTED, "vfkv_merge_partials_packed: head_dim must be 1..512");
    DeviceGuard g(ctx->device);
    return launch_merge_partials_packed(ctx, d_packed, n_parts, n_rows, head_dim, d_out, as_stream(stream));
}

/* ---- device-memory helpers -------------------------------------------------- */

int32_t vfkv_malloc(vfkv_ctx *ctx, uint64_t bytes, void **d_out)
{
    if (!ctx || !d_out) return VFKV_ERR_INVALID;
    DeviceGuard g(ctx->device);
    *d_out = nullptr;
    cudaError_t e = cudaMalloc(d_out, bytes ? bytes : 1);
    if (e != cudaSuccess) cudaGetLastError();
    return check_cuda(ctx, e, "vfkv_malloc");
}
int32_t vfkv_free(vfkv_ctx *ctx, void *d_ptr)
{
    if (!ctx) return VFKV_ERR_INVALID;
    DeviceGuard g(ctx->device);
    return check_cuda(ctx, cudaFree(d_ptr), "vfkv_free");
}
int32_t vfkv_malloc_host(vfkv_ctx *ctx, uint64_t bytes, void **h_out)
{
    if (!ctx || !h_out) return VFKV_ERR_INVALID;
    DeviceGuard g(ctx->device);
    *h_out = nullptr;
    return check_cuda(ctx, cudaMallocHost(h_out, bytes ? bytes : 1), "vfkv_malloc_host");
}
int32_t vfkv_free_host(vfkv_ctx *ctx, void *h_ptr)
{
    if (!ctx) return VFKV_ERR_INVALID;
    DeviceGuard g(ctx->device);
    return check_cuda(ctx, cudaFreeHost(h_ptr), "vfkv_free_host");
}
int32_t vfkv_memcpy_h2d(vfkv_ctx *ctx, void *d_dst, const void *h_src, uint64_t bytes, void *stream)
{
    if (!ctx) return VFKV_ERR_INVALID;
    DeviceGuard g(ctx->device);
    return check_cuda(ctx, cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, as_stream(stream)), "vfkv_memcpy_h2d");
}
int32_t vfkv_memcpy_d2h(vfkv_ctx *ctx, void *h_dst, const void *d_src, uint64_t bytes, void *stream)
{
    if (!ctx) return VFKV_ERR_INVALID;
    DeviceGuard g(ctx->device);
    return check_cuda(ctx, cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)), "vfkv_memcpy_d2h");
}
int32_t vfkv_memset(vfkv_ctx *ctx, void *d_dst, int32_t byte, uint64_t bytes, void *stream)
{
    if (!ctx) return VFKV_ERR_INVALID;
    DeviceGuard g(ctx->device);
    return check_cuda(ctx, cudaMemsetAsync(d_dst, byte, bytes, as_stream(stream)), "vfkv_memset");
}
int32_t vfkv_stream_synchronize(vfkv_ctx *ctx, void *stream)
{
    if (!ctx) return VFKV_ERR_INVALID;
    DeviceGuard g(ctx->device);
    return check_cuda(ctx, cudaStreamSynchronize(as_stream(stream)), "vfkv_stream_synchronize");
}

}  // extern "C"
