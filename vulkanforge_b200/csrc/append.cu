// KV append and the FP8 -> F16 cache read.
//
// Replaces, on B200:
//   vk_shaders/kv_store_fp8.comp   (f32 -> E4M3, 4 codes per 32-bit word)
//   vk_shaders/kv_copy_fp16.comp   (f32 -> binary16 pairs)
//   the vkCmdCopyBuffer of the F32 cache (executor/attention.rs:576-581)
//   vk_shaders/kv_fp8_to_f16.comp  (E4M3 -> binary16, identity index)
// and their host halves Forward::run_kv_store_fp8 / run_kv_copy_fp16
// (src/backend/vulkan/forward/runs.rs:2389-2478).
//
// The reference converts 4 (or 2) elements per thread and issues K and V as two
// dispatches; here each thread produces one 16-byte store and K and V share a
// launch.  The work is a few KB per token, so the only lever that matters is
// launch count; the vector width keeps the prefill-chunk case at full HBM rate.
#include "common.cuh"
#include "fp8_codec.cuh"

namespace vfkv {

template <int DT> struct Enc;
template <> struct Enc<VFKV_F8> {   // 16 elements -> 16 bytes
    static constexpr int kElems = 16;
    __device__ static uint4 run(const float4 *s)
    {
        float4 a = s[0], b = s[1], c = s[2], d = s[3];
        return make_uint4(f32x4_to_e4m3x4(a.x, a.y, a.z, a.w), f32x4_to_e4m3x4(b.x, b.y, b.z, b.w),
                          f32x4_to_e4m3x4(c.x, c.y, c.z, c.w), f32x4_to_e4m3x4(d.x, d.y, d.z, d.w));
    }
};
template <> struct Enc<VFKV_F16> {  // 8 elements -> 16 bytes
    static constexpr int kElems = 8;
    __device__ static uint4 run(const float4 *s)
    {
        float4 a = s[0], b = s[1];
        return make_uint4(f32x2_to_f16x2(a.x, a.y), f32x2_to_f16x2(a.z, a.w),
                          f32x2_to_f16x2(b.x, b.y), f32x2_to_f16x2(b.z, b.w));
    }
};
template <> struct Enc<VFKV_F32> {  // 4 elements -> 16 bytes
    static constexpr int kElems = 4;
    __device__ static uint4 run(const float4 *s)
    {
        float4 a = s[0];
        return make_uint4(__float_as_uint(a.x), __float_as_uint(a.y), __float_as_uint(a.z),
                          __float_as_uint(a.w));
    }
};

// ---- raw store: n f32 -> dst, 16-byte vector body + word-sized tail -------
template <int DT>
__global__ void __launch_bounds__(256) store_vec_kernel(const float *__restrict__ src,
                                                        uint8_t *__restrict__ dst, uint64_t n)
{
    constexpr int E = Enc<DT>::kElems;
    const uint64_t n_vec = n / E;
    for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < n_vec;
         i += uint64_t(gridDim.x) * blockDim.x) {
        uint4 r = Enc<DT>::run(reinterpret_cast<const float4 *>(src + i * E));
        reinterpret_cast<uint4 *>(dst)[i] = r;
    }
}

// One 32-bit word per thread, exactly the reference's granularity, with its
// zero padding of a ragged tail (kv_store_fp8.comp:58-66, kv_copy_fp16.comp:46-50).
template <int DT>
__global__ void __launch_bounds__(256) store_word_kernel(const float *__restrict__ src,
                                                         uint32_t *__restrict__ dst,
                                                         uint64_t first, uint64_t n)
{
    constexpr int W = DT == VFKV_F8 ? 4 : DT == VFKV_F16 ? 2 : 1;
    uint64_t w = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
    uint64_t e = first + w * W;
    if (e >= n) return;
    float x[4];
#pragma unroll
    for (int j = 0; j < W; ++j) x[j] = (e + j < n) ? src[e + j] : 0.0f;
    uint32_t r;
    if (DT == VFKV_F8) r = f32x4_to_e4m3x4(x[0], x[1], x[2], x[3]);
    else if (DT == VFKV_F16) r = f32x2_to_f16x2(x[0], x[1]);
    else r = __float_as_uint(x[0]);
    dst[e / W] = r;
}

template <int DT>
static int32_t launch_store_t(vfkv_ctx *ctx, const float *src, void *dst, uint64_t n, cudaStream_t st)
{
    constexpr int E = Enc<DT>::kElems;
    constexpr int W = DT == VFKV_F8 ? 4 : DT == VFKV_F16 ? 2 : 1;
    const bool aligned = (reinterpret_cast<uintptr_t>(src) % 16 == 0) &&
                         (reinterpret_cast<uintptr_t>(dst) % 16 == 0);
    uint64_t done = 0;
    if (aligned && n >= uint64_t(E)) {
        uint64_t n_vec = n / E;
        uint64_t blocks = (n_vec + 255) / 256;
        uint64_t cap = uint64_t(ctx->sm_count) * 16;
        if (blocks > cap) blocks = cap;
        ProfScope ps(ctx, VFKV_PROF_KV_STORE, st);
        store_vec_kernel<DT><<<unsigned(blocks), 256, 0, st>>>(src, static_cast<uint8_t *>(dst), n);
        ctx->launches++;
        done = n_vec * E;
    }
    if (done < n) {
        uint64_t words = (n - done + W - 1) / W;
        ProfScope ps(ctx, VFKV_PROF_KV_STORE, st);
        store_word_kernel<DT><<<unsigned((words + 255) / 256), 256, 0, st>>>(
            src, static_cast<uint32_t *>(dst), done, n);
        ctx->launches++;
    }
    ctx->last_written_slab = vfkv::kAnySlab;        // a raw destination may lie in any layer
    return check_cuda(ctx, cudaGetLastError(), "store kernel launch");
}

int32_t launch_store(vfkv_ctx *ctx, uint32_t dtype, const float *src, void *dst, uint64_t n,
                     cudaStream_t st)
{
    if (n == 0) return VFKV_OK;
    switch (dtype) {
    case VFKV_F8: return launch_store_t<VFKV_F8>(ctx, src, dst, n, st);
    case VFKV_F16: return launch_store_t<VFKV_F16>(ctx, src, dst, n, st);
    case VFKV_F32: return launch_store_t<VFKV_F32>(ctx, src, dst, n, st);
    }
    return set_error(ctx, VFKV_ERR_INVALID, "unknown dtype");
}

// ---- cache-level append: K and V rows of many tokens in one launch ----------
struct AppendParams {
    const float *src[2];
    uint8_t *dst[2];
    float *scales[2];
    const uint32_t *slot_ids;
    const uint32_t *positions;
    uint64_t slot_stride_bytes, slot_stride_scales;
    uint32_t row_elems, head_dim, n_kv_heads, max_seq, n_slots, n_rows, slot, base_pos;
    uint32_t shard_world, shard_rank, shard_page;   // world > 1: base_pos + row is a global position dealt out in pages
    uint32_t *status;
};

__device__ __forceinline__ bool row_target(const AppendParams &p, uint32_t row, uint32_t *slot,
                                           uint32_t *pos)
{
    if (p.positions) {
        *slot = p.slot_ids ? p.slot_ids[row] : row;
        *pos = p.positions[row];
    } else {
        *slot = p.slot;
        *pos = p.base_pos + row;
        if (p.shard_world > 1u) {        // pages of positions dealt round-robin: rows of other ranks are not stored here
            const uint32_t page = *pos / p.shard_page;
            if (page % p.shard_world != p.shard_rank) return false;
            *pos = (page / p.shard_world) * p.shard_page + *pos % p.shard_page;
        }
    }
    if (*slot >= p.n_slots || *pos >= p.max_seq) {
        atomicOr(p.status, 2u);   // out-of-range row: skipped, reported through vfkv_ctx_poll
        return false;
    }
    return true;
}

// grid.y selects K (0) or V (1); each thread emits one 16-byte piece of a row.
template <int DT>
__global__ void __launch_bounds__(256) append_kernel(const AppendParams p)
{
    constexpr int E = Enc<DT>::kElems;
    const uint32_t which = blockIdx.y;
    const uint32_t chunks_per_row = p.row_elems / E;
    const uint64_t total = uint64_t(p.n_rows) * chunks_per_row;
    const uint64_t row_bytes = uint64_t(p.row_elems) * (DT == VFKV_F8 ? 1 : DT == VFKV_F16 ? 2 : 4);
    for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < total;
         i += uint64_t(gridDim.x) * blockDim.x) {
        uint32_t row = uint32_t(i / chunks_per_row), c = uint32_t(i % chunks_per_row);
        uint32_t slot, pos;
        if (!row_target(p, row, &slot, &pos)) continue;
        const float4 *s = reinterpret_cast<const float4 *>(p.src[which] + uint64_t(row) * p.row_elems +
                                                           uint64_t(c) * E);
        uint4 r = Enc<DT>::run(s);
        uint8_t *d = p.dst[which] + uint64_t(slot) * p.slot_stride_bytes + uint64_t(pos) * row_bytes;
        reinterpret_cast<uint4 *>(d)[c] = r;
    }
}

// Extension: per-(token, kv-head) absmax scale.  One warp per (row, head, K|V).
// scale = max(absmax * (1/448), 1e-12); inv = 1/scale; code = e4m3(clamp(x*inv, +-448)):
// the recipe of vk_shaders/mul_coopmat_fp8_native_bn32.comp:149-152,214.
__global__ void __launch_bounds__(256) append_scaled_kernel(const AppendParams p)
{
    const uint32_t warps_per_block = blockDim.x / 32;
    const uint32_t which = blockIdx.y;
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t total = uint64_t(p.n_rows) * p.n_kv_heads;
    for (uint64_t w = blockIdx.x * uint64_t(warps_per_block) + threadIdx.x / 32; w < total;
         w += uint64_t(gridDim.x) * warps_per_block) {
        uint32_t row = uint32_t(w / p.n_kv_heads), head = uint32_t(w % p.n_kv_heads);
        uint32_t slot, pos;
        if (!row_target(p, row, &slot, &pos)) continue;
        const float *x = p.src[which] + uint64_t(row) * p.row_elems + uint64_t(head) * p.head_dim;
        float amax = 0.f;
        for (uint32_t d = lane * 4; d < p.head_dim; d += 128) {
            float4 v = *reinterpret_cast<const float4 *>(x + d);
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float sc = fmaxf(__fmul_rn(amax, 1.0f / 448.0f), 1e-12f);
        const float inv = __fdiv_rn(1.0f, sc);
        uint8_t *drow = p.dst[which] + uint64_t(slot) * p.slot_stride_bytes +
                        uint64_t(pos) * p.row_elems + uint64_t(head) * p.head_dim;
        for (uint32_t d = lane * 4; d < p.head_dim; d += 128) {
            float4 v = *reinterpret_cast<const float4 *>(x + d);
            float y[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float t = fminf(fmaxf(__fmul_rn(y[j], inv), -448.f), 448.f);
                y[j] = (y[j] != y[j]) ? y[j] : t;
            }
            *reinterpret_cast<uint32_t *>(drow + d) = f32x4_to_e4m3x4(y[0], y[1], y[2], y[3]);
        }
        if (lane == 0)
            p.scales[which][uint64_t(slot) * p.slot_stride_scales + uint64_t(pos) * p.n_kv_heads + head] = sc;
    }
}

int32_t launch_append(vfkv_ctx *ctx, const AppendArgs &a, cudaStream_t st)
{
    if (a.n_rows == 0) return VFKV_OK;
    AppendParams p;
    p.src[0] = a.k; p.src[1] = a.v;
    p.dst[0] = static_cast<uint8_t *>(a.k_dst); p.dst[1] = static_cast<uint8_t *>(a.v_dst);
    p.scales[0] = a.k_scales; p.scales[1] = a.v_scales;
    p.slot_ids = a.slot_ids; p.positions = a.positions;
    p.slot_stride_bytes = a.slot_stride_bytes; p.slot_stride_scales = a.slot_stride_scales;
    p.row_elems = a.row_elems; p.head_dim = a.head_dim; p.n_kv_heads = a.n_kv_heads;
    p.max_seq = a.max_seq; p.n_slots = a.n_slots; p.n_rows = a.n_rows; p.slot = a.slot;
    p.base_pos = a.base_pos; p.status = ctx->d_status;
    p.shard_world = a.shard_world; p.shard_rank = a.shard_rank; p.shard_page = a.shard_page ? a.shard_page : 1u;

    if (a.k_scales) {
        if (a.head_dim % 4 != 0) return set_error(ctx, VFKV_ERR_UNSUPPORTED, "scaled append needs head_dim % 4 == 0");
        uint64_t warps = uint64_t(a.n_rows) * a.n_kv_heads;
        uint64_t blocks = (warps + 7) / 8, cap = uint64_t(ctx->sm_count) * 8;
        if (blocks > cap) blocks = cap;
        {
            ProfScope ps(ctx, VFKV_PROF_KV_STORE, st);
            append_scaled_kernel<<<dim3(unsigned(blocks), 2), 256, 0, st>>>(p);
        }
        ctx->launches++;
        ctx->last_written_slab = a.k_dst;
        return check_cuda(ctx, cudaGetLastError(), "append_scaled launch");
    }
    const int E = a.dtype == VFKV_F8 ? 16 : a.dtype == VFKV_F16 ? 8 : 4;
    uint64_t chunks = uint64_t(a.n_rows) * (a.row_elems / E);
    uint64_t blocks = (chunks + 255) / 256, cap = uint64_t(ctx->sm_count) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    dim3 grid(unsigned(blocks), 2);
    ProfScope ps(ctx, VFKV_PROF_KV_STORE, st);
    switch (a.dtype) {
    case VFKV_F8: append_kernel<VFKV_F8><<<grid, 256, 0, st>>>(p); break;
    case VFKV_F16: append_kernel<VFKV_F16><<<grid, 256, 0, st>>>(p); break;
    case VFKV_F32: append_kernel<VFKV_F32><<<grid, 256, 0, st>>>(p); break;
    default: return set_error(ctx, VFKV_ERR_INVALID, "unknown dtype");
    }
    ctx->launches++;
    ctx->last_written_slab = a.k_dst;
    return check_cuda(ctx, cudaGetLastError(), "append launch");
}

// ---- E4M3 -> binary16 (vk_shaders/kv_fp8_to_f16.comp:28-34) ----------------
__global__ void __launch_bounds__(256) fp8_to_f16_vec_kernel(const uint4 *__restrict__ src,
                                                             uint4 *__restrict__ dst, uint64_t n_vec)
{
    for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < n_vec;
         i += uint64_t(gridDim.x) * blockDim.x) {
        uint4 s = src[i];
        uint32_t w[4] = {s.x, s.y, s.z, s.w};
        uint32_t o[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            __half2 lo = e4m3x2_to_half2(w[j] & 0xFFFFu), hi = e4m3x2_to_half2(w[j] >> 16);
            o[2 * j] = *reinterpret_cast<uint32_t *>(&lo);
            o[2 * j + 1] = *reinterpret_cast<uint32_t *>(&hi);
        }
        dst[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
}

__global__ void __launch_bounds__(256) fp8_to_f16_scalar_kernel(const uint8_t *__restrict__ src,
                                                                __half *__restrict__ dst,
                                                                uint64_t first, uint64_t n)
{
    uint64_t i = first + blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
    if (i >= n) return;
    dst[i] = __low2half(e4m3x2_to_half2(src[i]));
}

int32_t launch_fp8_to_f16(vfkv_ctx *ctx, const void *src, void *dst, uint64_t n, cudaStream_t st)
{
    if (n == 0) return VFKV_OK;
    const bool aligned = (reinterpret_cast<uintptr_t>(src) % 16 == 0) &&
                         (reinterpret_cast<uintptr_t>(dst) % 16 == 0);
    uint64_t done = 0;
    if (aligned && n >= 16) {
        uint64_t n_vec = n / 16, blocks = (n_vec + 255) / 256, cap = uint64_t(ctx->sm_count) * 16;
        if (blocks > cap) blocks = cap;
        ProfScope ps(ctx, VFKV_PROF_FP8_TO_F16, st);
        fp8_to_f16_vec_kernel<<<unsigned(blocks), 256, 0, st>>>(
            static_cast<const uint4 *>(src), static_cast<uint4 *>(dst), n_vec);
        ctx->launches++;
        done = n_vec * 16;
    }
    if (done < n) {
        uint64_t rem = n - done;
        ProfScope ps(ctx, VFKV_PROF_FP8_TO_F16, st);
        fp8_to_f16_scalar_kernel<<<unsigned((rem + 255) / 256), 256, 0, st>>>(
            static_cast<const uint8_t *>(src), static_cast<__half *>(dst), done, n);
        ctx->launches++;
    }
    return check_cuda(ctx, cudaGetLastError(), "fp8_to_f16 launch");
}

}  // namespace vfkv
