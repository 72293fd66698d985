// RoPE-NeoX fused with the KV append, and the same rotation for Q rows.
//
// In the reference one layer's K goes through a rope dispatch (run_rope_neox*, host
// src/backend/vulkan/forward/runs.rs:647-720, math vk_shaders/rope_funcs.glsl:73-107), a pipeline
// barrier, and then kv_store_fp8 / kv_copy_fp16 (executor/attention.rs:435-530, :546-596): the
// rotated row makes a round trip through memory in f32.  Here the rotation happens in the
// registers of the thread that encodes the cache bytes, and K and V share one launch.
//
// The angle follows the CPU form the reference grades against (tests/correctness.rs:827-838):
// theta_i = pos * theta_scale^i with theta_scale = freq_base^(-2 / n_dims) computed once in f32
// and the powers taken by repeated multiplication.
#include <cmath>

#include "../../include/vfkv_next.h"
#include "common.cuh"
#include "fp8_codec.cuh"

namespace vfkv {

struct RopeAppendParams {
    const float *k, *v;
    uint8_t *k_dst, *v_dst;                // layer base (slot 0)
    float *k_rot;                          // optional f32 copy of the rotated K rows
    const uint32_t *slot_ids, *positions;  // batch mode when positions != null
    uint64_t slot_stride_bytes;
    uint32_t row_elems, head_dim, n_kv_heads, max_seq, n_slots, n_rows, slot, base_pos;
    uint32_t n_dims;
    float theta_scale, freq_scale;
    uint32_t *status;
};

template <int DT> struct Pack;
template <> struct Pack<VFKV_F8> {
    static constexpr int kElems = 16, kBytes = 1;
    __device__ static uint4 run(const float *x)
    {
        return make_uint4(f32x4_to_e4m3x4(x[0], x[1], x[2], x[3]), f32x4_to_e4m3x4(x[4], x[5], x[6], x[7]),
                          f32x4_to_e4m3x4(x[8], x[9], x[10], x[11]), f32x4_to_e4m3x4(x[12], x[13], x[14], x[15]));
    }
};
template <> struct Pack<VFKV_F16> {
    static constexpr int kElems = 8, kBytes = 2;
    __device__ static uint4 run(const float *x)
    {
        return make_uint4(f32x2_to_f16x2(x[0], x[1]), f32x2_to_f16x2(x[2], x[3]), f32x2_to_f16x2(x[4], x[5]),
                          f32x2_to_f16x2(x[6], x[7]));
    }
};
template <> struct Pack<VFKV_F32> {
    static constexpr int kElems = 4, kBytes = 4;
    __device__ static uint4 run(const float *x)
    {
        return make_uint4(__float_as_uint(x[0]), __float_as_uint(x[1]), __float_as_uint(x[2]), __float_as_uint(x[3]));
    }
};

// Rotates E consecutive elements starting at dim d0 of one head (x points at the head's dim 0).
// Requires n_dims / 2 to be a multiple of E, so that a piece lies wholly in one half.
template <int E>
__device__ __forceinline__ void rotate_piece(const float *__restrict__ x, uint32_t d0, uint32_t n_dims,
                                             float theta_scale, float pos_f, float *out)
{
    const uint32_t half = n_dims / 2;
    if (d0 >= n_dims) {
#pragma unroll
        for (int j = 0; j < E; ++j) out[j] = x[d0 + j];
        return;
    }
    const bool upper = d0 >= half;
    const uint32_t i0 = upper ? d0 - half : d0;
    // both halves of the pairs as 16-byte loads (x, i0 and half are multiples of four elements)
    float lo[E], hi[E];
#pragma unroll
    for (int j = 0; j < E; j += 4) {
        const float4 u = __ldg(reinterpret_cast<const float4 *>(x + i0 + j));
        const float4 w = __ldg(reinterpret_cast<const float4 *>(x + i0 + half + j));
        lo[j] = u.x; lo[j + 1] = u.y; lo[j + 2] = u.z; lo[j + 3] = u.w;
        hi[j] = w.x; hi[j + 1] = w.y; hi[j + 2] = w.z; hi[j + 3] = w.w;
    }
    float freq = 1.0f;
    for (uint32_t i = 0; i < i0; ++i) freq = __fmul_rn(freq, theta_scale);
#pragma unroll
    for (int j = 0; j < E; ++j) {
        const float theta = __fmul_rn(pos_f, freq);
        float s, c;
        sincosf(theta, &s, &c);
        const float a = lo[j], b = hi[j];
        // (x_i, x_{i+half}) <- (a c - b s, a s + b c), products rounded separately as on the CPU
        out[j] = upper ? __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c)) : __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
        freq = __fmul_rn(freq, theta_scale);
    }
}

// grid.y: 0 = K (rotated), 1 = V (stored as it is).  One 16-byte cache store per thread.
template <int DT>
__global__ void __launch_bounds__(256) rope_append_kernel(const RopeAppendParams p)
{
    constexpr int E = Pack<DT>::kElems;
    const uint32_t which = blockIdx.y;
    const uint32_t pieces_per_row = p.row_elems / E;
    const uint64_t total = uint64_t(p.n_rows) * pieces_per_row;
    const uint64_t row_bytes = uint64_t(p.row_elems) * Pack<DT>::kBytes;
    for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < total; i += uint64_t(gridDim.x) * blockDim.x) {
        const uint32_t row = uint32_t(i / pieces_per_row), c = uint32_t(i % pieces_per_row);
        uint32_t slot, pos;
        if (p.positions) { slot = p.slot_ids ? p.slot_ids[row] : row; pos = p.positions[row]; }
        else { slot = p.slot; pos = p.base_pos + row; }
        if (slot >= p.n_slots || pos >= p.max_seq) { atomicOr(p.status, 2u); continue; }
        float x[E];
        const uint32_t e0 = c * E;
        if (which == 0) {
            const uint32_t head = e0 / p.head_dim, d0 = e0 % p.head_dim;
            const float *src = p.k + uint64_t(row) * p.row_elems + uint64_t(head) * p.head_dim;
            rotate_piece<E>(src, d0, p.n_dims, p.theta_scale, __fmul_rn(float(pos), p.freq_scale), x);
            if (p.k_rot) {
                float *o = p.k_rot + uint64_t(row) * p.row_elems + e0;
#pragma unroll
                for (int j = 0; j < E; j += 4) *reinterpret_cast<float4 *>(o + j) = make_float4(x[j], x[j + 1], x[j + 2], x[j + 3]);
            }
        } else {
            const float4 *s = reinterpret_cast<const float4 *>(p.v + uint64_t(row) * p.row_elems + e0);
#pragma unroll
            for (int j = 0; j < E / 4; ++j) { float4 t = s[j]; x[4 * j] = t.x; x[4 * j + 1] = t.y; x[4 * j + 2] = t.z; x[4 * j + 3] = t.w; }
        }
        uint8_t *d = (which ? p.v_dst : p.k_dst) + uint64_t(slot) * p.slot_stride_bytes + uint64_t(pos) * row_bytes;
        reinterpret_cast<uint4 *>(d)[c] = Pack<DT>::run(x);
    }
}

// Q rows (or any [rows][heads][head_dim] f32): one thread per pair.
__global__ void __launch_bounds__(256)
rope_neox_kernel(const float *__restrict__ x, float *__restrict__ out, uint64_t n_rows, uint32_t n_heads,
                 uint32_t head_dim, const uint32_t *__restrict__ positions, uint32_t base_pos, uint32_t n_dims,
                 float theta_scale, float freq_scale)
{
    const uint32_t half = n_dims / 2, tail = head_dim - n_dims;
    const uint32_t per_head = half + tail;              // work items per head: pairs, then pass-through dims
    const uint64_t total = n_rows * n_heads * per_head;
    for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < total; i += uint64_t(gridDim.x) * blockDim.x) {
        const uint32_t w = uint32_t(i % per_head);
        const uint64_t rh = i / per_head, row = rh / n_heads;
        const float *src = x + rh * head_dim;
        float *dst = out + rh * head_dim;
        if (w >= half) { dst[n_dims + (w - half)] = src[n_dims + (w - half)]; continue; }
        const uint32_t pos = positions ? positions[row] : base_pos + uint32_t(row);
        float freq = 1.0f;
        for (uint32_t k = 0; k < w; ++k) freq = __fmul_rn(freq, theta_scale);
        const float theta = __fmul_rn(__fmul_rn(float(pos), freq_scale), freq);
        float s, c;
        sincosf(theta, &s, &c);
        const float a = src[w], b = src[w + half];
        dst[w] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
        dst[w + half] = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
    }
}

static float theta_scale_of(const vfkv_rope_params &r)
{
    return powf(1.0f / r.freq_base, 2.0f / float(r.n_dims));     // setup.rs:786-788 in f32
}

template <int DT>
static int32_t launch_rope_append_t(vfkv_ctx *ctx, const RopeAppendParams &p, cudaStream_t st)
{
    constexpr int E = Pack<DT>::kElems;
    const uint64_t total = uint64_t(p.n_rows) * (p.row_elems / E);
    uint64_t blocks = (total + 255) / 256;
    const uint64_t cap = uint64_t(ctx->sm_count) * 16;
    if (blocks > cap) blocks = cap;
    ProfScope ps(ctx, VFKV_PROF_KV_STORE, st);
    rope_append_kernel<DT><<<dim3(unsigned(blocks), 2), 256, 0, st>>>(p);
    ctx->launches++;
    ctx->last_written_slab = p.k_dst;
    return check_cuda(ctx, cudaGetLastError(), "rope_append launch");
}

}  // namespace vfkv

using namespace vfkv;

namespace {

struct Guard {
    int prev = -1;
    explicit Guard(int dev) { cudaGetDevice(&prev); if (prev != dev) cudaSetDevice(dev); else prev = -1; }
    ~Guard() { if (prev >= 0) cudaSetDevice(prev); }
};

int32_t check_rope(vfkv_ctx *ctx, const vfkv_rope_params *r, uint32_t head_dim, const char *fn)
{
    if (!r) return set_error(ctx, VFKV_ERR_INVALID, std::string(fn) + ": null rope parameters");
    if (r->n_dims == 0 || r->n_dims % 2 != 0 || r->n_dims > head_dim)
        return set_error(ctx, VFKV_ERR_INVALID, std::string(fn) + ": n_dims must be even and at most head_dim");
    if (!(r->freq_base > 0.f) || !(r->freq_scale > 0.f))
        return set_error(ctx, VFKV_ERR_INVALID, std::string(fn) + ": freq_base and freq_scale must be positive");
    return VFKV_OK;
}

int32_t rope_append_common(vfkv_cache *cache, uint32_t layer, const float *d_k, const float *d_v, uint32_t n_rows,
                           uint32_t slot, uint32_t base_pos, const uint32_t *d_slot_ids, const uint32_t *d_positions,
                           const vfkv_rope_params *rope, float *d_k_rot, void *stream, const char *fn)
{
    if (!cache) return VFKV_ERR_INVALID;
    vfkv_ctx *ctx = cache->ctx;
    KvCache &kv = cache->kv;
    if (layer >= kv.config.n_layers) return set_error(ctx, VFKV_ERR_INVALID, std::string(fn) + ": layer out of range");
    if (!d_k || !d_v) return set_error(ctx, VFKV_ERR_INVALID, std::string(fn) + ": null K or V");
    if ((reinterpret_cast<uintptr_t>(d_k) | reinterpret_cast<uintptr_t>(d_v) | reinterpret_cast<uintptr_t>(d_k_rot)) % 16 != 0)
        return set_error(ctx, VFKV_ERR_INVALID, std::string(fn) + ": K, V and the rotated-K output must be 16-byte aligned");
    const uint32_t hd = kv.head_dim_for(layer), hkv = kv.kv_heads_for(layer);
    int32_t rc = check_rope(ctx, rope, hd, fn);
    if (rc) return rc;
    if (n_rows == 0) return VFKV_OK;
    const uint32_t dt = uint32_t(kv.kv_dtype);
    const uint32_t E = dt == VFKV_F8 ? 16 : dt == VFKV_F16 ? 8 : 4;
    const bool fusable = !kv.k_scales && (rope->n_dims / 2) % E == 0 && hd % E == 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!fusable) {
        // shapes the fused kernel does not tile (or a cache with scale planes): rotate into the
        // caller's buffer, then the ordinary append
        if (!d_k_rot) return set_error(ctx, VFKV_ERR_UNSUPPORTED, std::string(fn) + ": this shape needs the d_k_rot buffer");
        rc = vfkv_rope_neox(ctx, d_k, d_k_rot, n_rows, hkv, hd, d_positions, base_pos, rope, stream);
        if (rc) return rc;
        return d_positions ? vfkv_append_batch(cache, layer, d_k_rot, d_v, d_slot_ids, d_positions, n_rows, stream)
                           : vfkv_append(cache, layer, d_k_rot, d_v, n_rows, slot, base_pos, stream);
    }
    RopeAppendParams p{};
    p.k = d_k; p.v = d_v; p.k_rot = d_k_rot;
    const uint64_t off = kv.layer_offset_bytes(layer);
    p.k_dst = static_cast<uint8_t *>(kv.k_buffer) + off;
    p.v_dst = static_cast<uint8_t *>(kv.v_buffer) + off;
    p.slot_ids = d_slot_ids; p.positions = d_positions;
    p.slot_stride_bytes = kv.layer_size_bytes(layer);
    p.row_elems = hkv * hd; p.head_dim = hd; p.n_kv_heads = hkv;
    p.max_seq = kv.config.max_seq_len; p.n_slots = kv.config.n_slots;
    p.n_rows = n_rows; p.slot = slot; p.base_pos = base_pos;
    p.n_dims = rope->n_dims; p.theta_scale = theta_scale_of(*rope); p.freq_scale = rope->freq_scale;
    p.status = ctx->d_status;
    Guard g(ctx->device);
    switch (dt) {
    case VFKV_F8: return launch_rope_append_t<VFKV_F8>(ctx, p, st);
    case VFKV_F16: return launch_rope_append_t<VFKV_F16>(ctx, p, st);
    case VFKV_F32: return launch_rope_append_t<VFKV_F32>(ctx, p, st);
    }
    return set_error(ctx, VFKV_ERR_INVALID, "unknown dtype");
}

}  // namespace

extern "C" {

int32_t vfkv_rope_append(vfkv_cache *cache, uint32_t layer, const float *d_k, const float *d_v, uint32_t n_tokens,
                         uint32_t slot, uint32_t base_pos, const vfkv_rope_params *rope, float *d_k_rot, void *stream)
{
    if (!cache) return VFKV_ERR_INVALID;
    if (slot >= cache->kv.config.n_slots)
        return set_error(cache->ctx, VFKV_ERR_INVALID, "vfkv_rope_append: slot out of range");
    if (uint64_t(base_pos) + n_tokens > cache->kv.config.max_seq_len)
        return set_error(cache->ctx, VFKV_ERR_INVALID, "vfkv_rope_append: base_pos + n_tokens exceeds max_seq_len");
    return rope_append_common(cache, layer, d_k, d_v, n_tokens, slot, base_pos, nullptr, nullptr, rope, d_k_rot, stream,
                              "vfkv_rope_append");
}

int32_t vfkv_rope_append_batch(vfkv_cache *cache, uint32_t layer, const float *d_k, const float *d_v,
                               const uint32_t *d_slot_ids, const uint32_t *d_positions, uint32_t n_seqs,
                               const vfkv_rope_params *rope, float *d_k_rot, void *stream)
{
    if (!cache) return VFKV_ERR_INVALID;
    if (!d_positions) return set_error(cache->ctx, VFKV_ERR_INVALID, "vfkv_rope_append_batch: null positions");
    return rope_append_common(cache, layer, d_k, d_v, n_seqs, 0, 0, d_slot_ids, d_positions, rope, d_k_rot, stream,
                              "vfkv_rope_append_batch");
}

int32_t vfkv_rope_neox(vfkv_ctx *ctx, const float *d_x, float *d_out, uint32_t n_rows, uint32_t n_heads,
                       uint32_t head_dim, const uint32_t *d_positions, uint32_t base_pos, const vfkv_rope_params *rope,
                       void *stream)
{
    if (!ctx) return VFKV_ERR_INVALID;
    if (!d_x || !d_out) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_rope_neox: null argument");
    if (head_dim == 0 || n_heads == 0) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_rope_neox: empty shape");
    int32_t rc = check_rope(ctx, rope, head_dim, "vfkv_rope_neox");
    if (rc) return rc;
    if (n_rows == 0) return VFKV_OK;
    Guard g(ctx->device);
    const uint64_t total = uint64_t(n_rows) * n_heads * (rope->n_dims / 2 + head_dim - rope->n_dims);
    uint64_t blocks = (total + 255) / 256;
    const uint64_t cap = uint64_t(ctx->sm_count) * 16;
    if (blocks > cap) blocks = cap;
    rope_neox_kernel<<<unsigned(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        d_x, d_out, n_rows, n_heads, head_dim, d_positions, base_pos, rope->n_dims, theta_scale_of(*rope),
        rope->freq_scale);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "rope_neox launch");
}

}  // extern "C"
