// Chunked-prefill causal attention over the KV cache: m queries of one sequence against the
// positions the cache already holds.
//
// Replaces vk_shaders/flash_attn_batch.comp:105-208 (+ FP16_KV / FP8_KV variants) and
// Forward::run_flash_attn_batch (src/backend/vulkan/forward/runs.rs:933-1010).  The reference
// runs one 64-thread workgroup per (head, query) and streams the causal K/V range once per
// query and head; here one CTA owns 64 rows = (64 / g) consecutive queries x the g q-heads of
// one kv-head, so a K/V tile is fetched once per 64 rows, widened to half precision once
// (FP8 caches; the kv_fp8_to_f16.comp step) and consumed by m16n8k16 tensor-core MMAs with the
// usual online softmax.  Shapes outside that kernel use a CUDA-core kernel with the reference's
// work split (one CTA per (query, head)).
#include <cmath>

#include "../../include/vfkv_next.h"
#include "common.cuh"
#include "fp8_codec.cuh"

namespace vfkv {
namespace {

constexpr float kLog2e = 1.4426950408889634f;

struct PrefillParams {
    const uint8_t *k, *v;              // rows of the slot: [pos][kv_head][dim]
    const float *k_scales, *v_scales;  // [pos][kv_head] or null
    const float *q;                    // [m][n_q_heads][dim]
    float *out;                        // [m][n_q_heads][dim]
    uint64_t row_bytes;
    uint32_t n_q_heads, n_kv_heads, group, head_dim, m, q_start, n_kv, kv_start, window;
    float scale, softcap;
};

// Visible range [lo, hi) of query i (flash_attn_batch.comp:116-119,141-144; window: per-query bound).
__device__ __forceinline__ void query_range(const PrefillParams &p, uint32_t i, uint32_t *lo, uint32_t *hi)
{
    uint32_t c = p.q_start + i + 1u;
    if (c > p.n_kv) c = p.n_kv;
    uint32_t l = p.kv_start;
    if (p.window != 0u && c > p.window && c - p.window > l) l = c - p.window;
    if (l > c) l = c;
    *lo = l; *hi = c;
}

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool valid)
{
    const uint32_t n = valid ? 16u : 0u;          // 0 source bytes: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi)
{
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

constexpr int BM = 64;     // rows per CTA (4 warps x 16)
constexpr int BN = 64;     // positions per tile

// Byte offset of 16-byte chunk c of row r in a half-precision tile with D dims per row; the
// XOR spreads the eight rows an ldmatrix reads over all banks.
template <int D> __device__ __forceinline__ uint32_t tile_off(uint32_t r, uint32_t c)
{
    return r * (D * 2) + ((c ^ (r & 7u)) << 4);
}

template <int DT, int D> struct PrefillSmem {
    static constexpr int ES = DT == VFKV_F8 ? 1 : 2;
    static constexpr int TILE16 = BN * D * 2;                       // one half-precision tile
    static constexpr int RAW = DT == VFKV_F8 ? BN * D : 0;          // one raw FP8 tile
    // F16 cache: two (K, V) half tiles, filled by cp.async directly.
    // FP8 cache: two raw (K, V) tiles for cp.async plus one (K, V) half tile for the MMAs.
    static constexpr int BYTES = DT == VFKV_F8 ? 4 * RAW + 2 * TILE16 : 4 * TILE16;
};

// QSPLIT: Q is fed as hi + lo half-precision parts (two MMAs per K block); used for F16 caches,
// whose error budget is that of the reference's f32 shader rather than of FP8 storage.
// QSMEM: the Q fragments live in shared memory and are re-read per k-step (head_dim 256, where
// they would not fit in registers beside the accumulators).
template <int DT, int D, bool CAP, bool QSPLIT, bool QSMEM>
__global__ void __launch_bounds__(128) prefill_mma_kernel(const PrefillParams p)
{
    using S = PrefillSmem<DT, D>;
    constexpr bool FP8 = DT == VFKV_F8;
    constexpr int KSTEPS = D / 16, NB = BN / 8, DB = D / 8, CPR = D * S::ES / 16;   // CPR: 16-byte chunks per cache row
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sbase = smem_addr(smem);
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gid = lane >> 2, tig = lane & 3;
    const uint32_t kvh = blockIdx.y, g = p.group;
    const uint32_t n_rows = p.m * g;
    // heaviest row blocks (latest queries) first
    const uint32_t rb = gridDim.x - 1u - blockIdx.x;
    const uint32_t row0 = rb * BM;

    // this thread's two rows: (query, head in group)
    uint32_t r_lo[2], r_hi[2];
    bool r_ok[2];
    uint32_t q_idx[2], hj[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t r = row0 + warp * 16 + gid + 8 * h;
        r_ok[h] = r < n_rows;
        q_idx[h] = r_ok[h] ? r / g : 0u;
        hj[h] = r_ok[h] ? r % g : 0u;
        query_range(p, q_idx[h], &r_lo[h], &r_hi[h]);
        if (!r_ok[h]) { r_lo[h] = 0u; r_hi[h] = 0u; }
    }
    // CTA-wide tile range: queries row0 / g .. (row0 + BM - 1) / g
    uint32_t c_lo, c_hi;
    {
        const uint32_t qa = row0 / g;
        uint32_t qb = (row0 + BM - 1) / g;
        if (qb >= p.m) qb = p.m - 1;
        uint32_t lo_a, hi_a, lo_b, hi_b;
        query_range(p, qa, &lo_a, &hi_a);
        query_range(p, qb, &lo_b, &hi_b);
        c_lo = lo_a / BN * BN;           // ranges are monotone in the query index
        c_hi = hi_b;
    }
    const uint32_t n_tiles = c_hi > c_lo ? (c_hi - c_lo + BN - 1) / BN : 0u;

    // Q fragments, scaled, in half precision (hi and, with QSPLIT, the residual lo)
    uint32_t qa_hi[QSMEM ? 1 : KSTEPS][4], qa_lo[QSPLIT && !QSMEM ? KSTEPS : 1][4];
    const uint32_t q_hi0 = sbase + S::BYTES, q_lo0 = q_hi0 + BM * D * 2;    // QSMEM: [64 rows][D] halves each
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float *qp = p.q + (uint64_t(q_idx[h]) * p.n_q_heads + kvh * g + hj[h]) * D + 16 * ks + 2 * tig;
            float2 a = r_ok[h] ? *reinterpret_cast<const float2 *>(qp) : make_float2(0.f, 0.f);
            float2 b = r_ok[h] ? *reinterpret_cast<const float2 *>(qp + 8) : make_float2(0.f, 0.f);
            a.x *= p.scale; a.y *= p.scale; b.x *= p.scale; b.y *= p.scale;
            const uint32_t ha = pack_half2(a.x, a.y), hb = pack_half2(b.x, b.y);
            uint32_t la = 0u, lb = 0u;
            if constexpr (QSPLIT) {
                const float2 fa = __half22float2(*reinterpret_cast<const __half2 *>(&ha));
                const float2 fb = __half22float2(*reinterpret_cast<const __half2 *>(&hb));
                la = pack_half2(a.x - fa.x, a.y - fa.y);
                lb = pack_half2(b.x - fb.x, b.y - fb.y);
            }
            if constexpr (QSMEM) {
                const uint32_t r = warp * 16 + gid + 8 * h;
                const uint32_t oa = tile_off<D>(r, 2 * ks) + 4 * tig, ob = tile_off<D>(r, 2 * ks + 1) + 4 * tig;
                *reinterpret_cast<uint32_t *>(smem + (q_hi0 - sbase) + oa) = ha;
                *reinterpret_cast<uint32_t *>(smem + (q_hi0 - sbase) + ob) = hb;
                if constexpr (QSPLIT) {
                    *reinterpret_cast<uint32_t *>(smem + (q_lo0 - sbase) + oa) = la;
                    *reinterpret_cast<uint32_t *>(smem + (q_lo0 - sbase) + ob) = lb;
                }
            } else {
                qa_hi[ks][h] = ha; qa_hi[ks][2 + h] = hb;
                if constexpr (QSPLIT) { qa_lo[ks][h] = la; qa_lo[ks][2 + h] = lb; }
            }
        }
    }

    if constexpr (QSMEM) __syncwarp();          // a warp reads back only the 16 rows it wrote
    float acc[DB][4];
#pragma unroll
    for (int i = 0; i < DB; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
    float mrow[2] = {kMaskedScore, kMaskedScore}, lrow[2] = {0.f, 0.f};

    const uint8_t *kg = p.k + uint64_t(kvh) * D * S::ES;
    const uint8_t *vg = p.v + uint64_t(kvh) * D * S::ES;
    // shared-memory map
    const uint32_t raw_k0 = sbase, raw_v0 = sbase + 2 * S::RAW;                    // FP8: raw[2] K, raw[2] V
    const uint32_t t16_k0 = sbase + 4 * S::RAW, t16_v0 = t16_k0 + (FP8 ? 1 : 2) * S::TILE16;

    auto issue = [&](uint32_t it) {
        const uint32_t t0 = c_lo + it * BN, buf = it & 1u;
        for (uint32_t i = threadIdx.x; i < uint32_t(BN * CPR); i += 128) {
            const uint32_t r = i / CPR, c = i % CPR;
            const uint32_t pos = t0 + r;
            const bool ok = pos < p.n_kv;
            const uint64_t goff = uint64_t(ok ? pos : 0u) * p.row_bytes + c * 16;
            uint32_t dk, dv;
            if constexpr (FP8) {
                dk = raw_k0 + buf * S::RAW + r * D + c * 16;
                dv = raw_v0 + buf * S::RAW + r * D + c * 16;
            } else {
                dk = t16_k0 + buf * S::TILE16 + tile_off<D>(r, c);
                dv = t16_v0 + buf * S::TILE16 + tile_off<D>(r, c);
            }
            cp_async16(dk, kg + goff, ok);
            cp_async16(dv, vg + goff, ok);
        }
    };

    if (n_tiles) issue(0);
    cp_async_commit();

    for (uint32_t it = 0; it < n_tiles; ++it) {
        __syncthreads();                               // every warp is done with tile it - 1
        if (it + 1 < n_tiles) issue(it + 1);
        cp_async_commit();
        cp_async_wait<1>();                            // tile `it` of this thread has landed
        __syncthreads();                               // ... and of every thread
        uint32_t tk, tv;
        if constexpr (FP8) {
            // widen the raw tile to half precision (exact), 16 codes per thread and step
            const uint8_t *rk = smem + (raw_k0 - sbase) + (it & 1u) * S::RAW;
            const uint8_t *rv = smem + (raw_v0 - sbase) + (it & 1u) * S::RAW;
            for (uint32_t i = threadIdx.x; i < uint32_t(BN * CPR); i += 128) {
                const uint32_t r = i / CPR, c = i % CPR;
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    const uint4 x = *reinterpret_cast<const uint4 *>((w ? rv : rk) + r * D + c * 16);
                    uint4 lo, hi;
                    {
                        __half2 h0 = e4m3x2_to_half2(x.x & 0xffffu), h1 = e4m3x2_to_half2(x.x >> 16);
                        __half2 h2 = e4m3x2_to_half2(x.y & 0xffffu), h3 = e4m3x2_to_half2(x.y >> 16);
                        lo = make_uint4(*reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1),
                                        *reinterpret_cast<uint32_t *>(&h2), *reinterpret_cast<uint32_t *>(&h3));
                        __half2 h4 = e4m3x2_to_half2(x.z & 0xffffu), h5 = e4m3x2_to_half2(x.z >> 16);
                        __half2 h6 = e4m3x2_to_half2(x.w & 0xffffu), h7 = e4m3x2_to_half2(x.w >> 16);
                        hi = make_uint4(*reinterpret_cast<uint32_t *>(&h4), *reinterpret_cast<uint32_t *>(&h5),
                                        *reinterpret_cast<uint32_t *>(&h6), *reinterpret_cast<uint32_t *>(&h7));
                    }
                    uint8_t *dst = smem + ((w ? t16_v0 : t16_k0) - sbase);
                    *reinterpret_cast<uint4 *>(dst + tile_off<D>(r, 2 * c)) = lo;
                    *reinterpret_cast<uint4 *>(dst + tile_off<D>(r, 2 * c + 1)) = hi;
                }
            }
            __syncthreads();
            tk = t16_k0; tv = t16_v0;
        } else {
            tk = t16_k0 + (it & 1u) * S::TILE16;
            tv = t16_v0 + (it & 1u) * S::TILE16;
        }

        const uint32_t t0 = c_lo + it * BN;
        // a warp whose rows all end before this tile, or start after it, has nothing to add
        const uint32_t w_hi = __reduce_max_sync(0xffffffffu, max(r_hi[0], r_hi[1]));
        const uint32_t w_lo = __reduce_min_sync(0xffffffffu, min(r_ok[0] ? r_lo[0] : 0xffffffffu, r_ok[1] ? r_lo[1] : 0xffffffffu));
        if (t0 >= w_hi || t0 + BN <= w_lo) continue;

        // ---- S = Q K^T -------------------------------------------------------------------
        float sc[NB][4];
#pragma unroll
        for (int i = 0; i < NB; ++i) { sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f; }
        {
            const uint32_t mi = lane >> 3, lr = lane & 7;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                uint32_t ah[4], al[4];
                if constexpr (QSMEM) {
                    const uint32_t qo = tile_off<D>(warp * 16 + (mi & 1u) * 8 + lr, 2 * ks + (mi >> 1));
                    ldsm_x4(q_hi0 + qo, ah[0], ah[1], ah[2], ah[3]);
                    if constexpr (QSPLIT) ldsm_x4(q_lo0 + qo, al[0], al[1], al[2], al[3]);
                } else {
#pragma unroll
                    for (int x = 0; x < 4; ++x) { ah[x] = qa_hi[ks][x]; al[x] = QSPLIT ? qa_lo[ks][x] : 0u; }
                }
#pragma unroll
                for (int jp = 0; jp < NB / 2; ++jp) {
                    const uint32_t r = 16 * jp + (mi >> 1) * 8 + lr, c = 2 * ks + (mi & 1u);
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(tk + tile_off<D>(r, c), b0, b1, b2, b3);
                    mma16816(sc[2 * jp], ah, b0, b1);
                    mma16816(sc[2 * jp + 1], ah, b2, b3);
                    if constexpr (QSPLIT) {
                        mma16816(sc[2 * jp], al, b0, b1);
                        mma16816(sc[2 * jp + 1], al, b2, b3);
                    }
                }
            }
        }
        // ---- mask, online softmax ------------------------------------------------------------
        const uint32_t c_min_hi = __reduce_min_sync(0xffffffffu, min(r_ok[0] ? r_hi[0] : 0xffffffffu, r_ok[1] ? r_hi[1] : 0xffffffffu));
        const uint32_t c_max_lo = __reduce_max_sync(0xffffffffu, max(r_lo[0], r_lo[1]));
        const bool all_ok = __all_sync(0xffffffffu, r_ok[0] && r_ok[1]);
        const bool full = all_ok && t0 + BN <= c_min_hi && t0 >= c_max_lo;   // no masking needed in this tile
        float alpha[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float mx = kMaskedScore;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float s = sc[nb][2 * h + e];
                    if constexpr (CAP) s = p.softcap * tanhf(s / p.softcap);
                    s *= kLog2e;
                    if (!full) {
                        const uint32_t pos = t0 + 8 * nb + 2 * tig + e;
                        if (pos < r_lo[h] || pos >= r_hi[h]) s = kMaskedScore;
                    }
                    sc[nb][2 * h + e] = s;
                    mx = fmaxf(mx, s);
                }
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float mnew = fmaxf(mrow[h], mx);
            alpha[h] = fast_exp2(mrow[h] - mnew);
            float sum = 0.f;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float s = sc[nb][2 * h + e];
                    // a masked position contributes nothing, also while the row's maximum is still the sentinel
                    const float pr = (full || s > 0.5f * kMaskedScore) ? fast_exp2(s - mnew) : 0.f;
                    sc[nb][2 * h + e] = pr;
                    sum += pr;
                }
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            lrow[h] = lrow[h] * alpha[h] + sum;
            mrow[h] = mnew;
        }
#pragma unroll
        for (int i = 0; i < DB; ++i) {
            acc[i][0] *= alpha[0]; acc[i][1] *= alpha[0];
            acc[i][2] *= alpha[1]; acc[i][3] *= alpha[1];
        }
        // ---- O += P V ------------------------------------------------------------------------
        {
            const uint32_t mi = lane >> 3, lr = lane & 7;
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk) {
                uint32_t pa[4];
                pa[0] = pack_half2(sc[2 * kk][0], sc[2 * kk][1]);
                pa[1] = pack_half2(sc[2 * kk][2], sc[2 * kk][3]);
                pa[2] = pack_half2(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
                pa[3] = pack_half2(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
                for (int dp = 0; dp < DB / 2; ++dp) {
                    const uint32_t r = 16 * kk + (mi & 1u) * 8 + lr, c = 2 * dp + (mi >> 1);
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_t(tv + tile_off<D>(r, c), b0, b1, b2, b3);
                    mma16816(acc[2 * dp], pa, b0, b1);
                    mma16816(acc[2 * dp + 1], pa, b2, b3);
                }
            }
        }
    }
    cp_async_wait<0>();

    // ---- normalise and store ---------------------------------------------------------------------
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (!r_ok[h]) continue;
        const float inv = lrow[h] > 0.f ? 1.0f / lrow[h] : 0.f;      // an empty range yields zeros
        float *o = p.out + (uint64_t(q_idx[h]) * p.n_q_heads + kvh * g + hj[h]) * D + 2 * tig;
#pragma unroll
        for (int nb = 0; nb < DB; ++nb)
            *reinterpret_cast<float2 *>(o + 8 * nb) = make_float2(acc[nb][2 * h] * inv, acc[nb][2 * h + 1] * inv);
    }
}

// ---- CUDA-core kernel: one CTA of 4 warps per (query, head), warps interleave positions -----------
__device__ __forceinline__ float load_elem(const uint8_t *base, uint32_t dt, uint64_t idx)
{
    if (dt == VFKV_F32) return reinterpret_cast<const float *>(base)[idx];
    if (dt == VFKV_F16) return __half2float(reinterpret_cast<const __half *>(base)[idx]);
    const uint32_t b = base[idx];
    return e4m3x2_to_float2(b).x;
}

__global__ void __launch_bounds__(128) prefill_simple_kernel(const PrefillParams p, uint32_t dt)
{
    constexpr int kMaxPerLane = 16;                    // head_dim <= 512
    __shared__ float s_m[4], s_l[4];
    __shared__ float s_o[4][512];
    const uint32_t h = blockIdx.y, qi = blockIdx.x;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t kvh = h / p.group, D = p.head_dim;
    uint32_t lo, hi;
    query_range(p, qi, &lo, &hi);
    float qv[kMaxPerLane], o[kMaxPerLane];
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
        const uint32_t d = lane + 32 * j;
        qv[j] = d < D ? p.q[(uint64_t(qi) * p.n_q_heads + h) * D + d] : 0.f;
        o[j] = 0.f;
    }
    float m = kMaskedScore, l = 0.f;
    const uint32_t es = dt == VFKV_F32 ? 4 : dt == VFKV_F16 ? 2 : 1;
    for (uint32_t pos = lo + warp; pos < hi; pos += 4) {
        const uint64_t e0 = (uint64_t(pos) * p.row_bytes) / es + uint64_t(kvh) * D;
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j) {
            const uint32_t d = lane + 32 * j;
            if (d < D) s = fmaf(qv[j], load_elem(p.k, dt, e0 + d), s);
        }
#pragma unroll
        for (int x = 16; x > 0; x >>= 1) s += __shfl_xor_sync(0xffffffffu, s, x);
        if (p.k_scales) s *= p.k_scales[uint64_t(pos) * p.n_kv_heads + kvh];
        s *= p.scale;
        if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
        const float mn = fmaxf(m, s);
        const float ko = __expf(m - mn), pn = __expf(s - mn);
        const float vs = p.v_scales ? p.v_scales[uint64_t(pos) * p.n_kv_heads + kvh] : 1.0f;
        l = l * ko + pn;
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j) {
            const uint32_t d = lane + 32 * j;
            if (d < D) o[j] = o[j] * ko + pn * vs * load_elem(p.v, dt, e0 + d);
        }
        m = mn;
    }
    if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
        const uint32_t d = lane + 32 * j;
        if (d < D) s_o[warp][d] = o[j];
    }
    __syncthreads();
    float gm = fmaxf(fmaxf(s_m[0], s_m[1]), fmaxf(s_m[2], s_m[3]));
    float gl = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) gl += s_l[w] * __expf(s_m[w] - gm);
    const float inv = gl > 0.f ? 1.0f / gl : 0.f;
    for (uint32_t d = threadIdx.x; d < D; d += 128) {
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) a += s_o[w][d] * __expf(s_m[w] - gm);
        p.out[(uint64_t(qi) * p.n_q_heads + h) * D + d] = a * inv;
    }
}

template <int DT, int D, bool CAP, bool QSPLIT>
int32_t launch_mma_t(vfkv_ctx *ctx, const PrefillParams &p, cudaStream_t st)
{
    using S = PrefillSmem<DT, D>;
    constexpr bool QSMEM = D > 128;
    constexpr int kSmem = S::BYTES + (QSMEM ? (QSPLIT ? 2 : 1) * BM * D * 2 : 0);
    auto kern = prefill_mma_kernel<DT, D, CAP, QSPLIT, QSMEM>;
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
        if (e != cudaSuccess) return check_cuda(ctx, e, "cudaFuncSetAttribute(prefill attention)");
        configured[ctx->device & 63] = true;
    }
    const uint32_t row_blocks = (p.m * p.group + BM - 1) / BM;
    kern<<<dim3(row_blocks, p.n_kv_heads), 128, kSmem, st>>>(p);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "prefill attention launch");
}

template <int DT, int D>
int32_t launch_mma_d(vfkv_ctx *ctx, const PrefillParams &p, cudaStream_t st)
{
    constexpr bool QS = DT == VFKV_F16;
    return p.softcap > 0.f ? launch_mma_t<DT, D, true, QS>(ctx, p, st) : launch_mma_t<DT, D, false, QS>(ctx, p, st);
}

struct Guard {
    int prev = -1;
    explicit Guard(int dev) { cudaGetDevice(&prev); if (prev != dev) cudaSetDevice(dev); else prev = -1; }
    ~Guard() { if (prev >= 0) cudaSetDevice(prev); }
};

}  // namespace
}  // namespace vfkv

using namespace vfkv;

extern "C" int32_t vfkv_attend_prefill(vfkv_cache *cache, uint32_t layer, uint32_t kv_layer, const float *d_q,
                                       float *d_out, uint32_t n_q_heads, uint32_t slot, uint32_t m, uint32_t q_start,
                                       uint32_t n_kv, uint32_t kv_start, uint32_t window, float scale, float softcap,
                                       void *stream)
{
    if (!cache) return VFKV_ERR_INVALID;
    vfkv_ctx *ctx = cache->ctx;
    KvCache &kv = cache->kv;
    if (layer >= kv.config.n_layers || kv_layer >= kv.config.n_layers)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_attend_prefill: layer out of range");
    const uint32_t D = kv.head_dim_for(layer), hkv = kv.kv_heads_for(layer);
    if (kv.head_dim_for(kv_layer) != D || kv.kv_heads_for(kv_layer) != hkv)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_attend_prefill: layer and kv_layer differ in shape");
    if (n_q_heads == 0 || hkv == 0 || n_q_heads % hkv != 0)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_attend_prefill: n_q_heads must be a multiple of the layer's kv heads");
    if (!d_q || !d_out) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_attend_prefill: null Q or output");
    if (slot >= kv.config.n_slots) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_attend_prefill: slot out of range");
    if (n_kv > kv.config.max_seq_len) return set_error(ctx, VFKV_ERR_INVALID, "vfkv_attend_prefill: n_kv exceeds max_seq_len");
    if (uint64_t(q_start) + m > 0xffffffffull) return set_error(ctx, VFKV_ERR_OVERFLOW, "vfkv_attend_prefill: q_start + m overflows");
    if (D > 512) return set_error(ctx, VFKV_ERR_UNSUPPORTED, "vfkv_attend_prefill: head_dim above 512");
    if (m == 0) return VFKV_OK;
    if (uint64_t(m) * n_q_heads > 0x7fffffffull || m > 65535u * 64u)
        return set_error(ctx, VFKV_ERR_UNSUPPORTED, "vfkv_attend_prefill: chunk too large");

    const uint32_t dt = uint32_t(kv.kv_dtype);
    const uint32_t es = dt == VFKV_F32 ? 4 : dt == VFKV_F16 ? 2 : 1;
    PrefillParams p{};
    const uint64_t off = kv.layer_offset_bytes(kv_layer) + uint64_t(slot) * kv.layer_size_bytes(kv_layer);
    p.k = static_cast<const uint8_t *>(kv.k_buffer) + off;
    p.v = static_cast<const uint8_t *>(kv.v_buffer) + off;
    if (kv.k_scales) {
        const uint64_t so = kv.scale_offset(kv_layer, 0, 0) + uint64_t(slot) * kv.config.max_seq_len * hkv;
        p.k_scales = kv.k_scales + so;
        p.v_scales = kv.v_scales + so;
    }
    p.q = d_q; p.out = d_out;
    p.row_bytes = uint64_t(hkv) * D * es;
    p.n_q_heads = n_q_heads; p.n_kv_heads = hkv; p.group = n_q_heads / hkv; p.head_dim = D;
    p.m = m; p.q_start = q_start; p.n_kv = n_kv; p.kv_start = kv_start; p.window = window;
    p.scale = scale; p.softcap = softcap;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    Guard g(ctx->device);
    const bool aligned = (reinterpret_cast<uintptr_t>(d_q) | reinterpret_cast<uintptr_t>(d_out) |
                          reinterpret_cast<uintptr_t>(p.k) | reinterpret_cast<uintptr_t>(p.v)) % 16 == 0;
    const bool mma_ok = ctx->attn_impl != 1 && aligned && !kv.k_scales && BM % p.group == 0 &&
                        (dt == VFKV_F8 || dt == VFKV_F16) && (D == 64 || D == 128 || D == 256);
    if (ctx->attn_impl == 2 && !mma_ok)
        return set_error(ctx, VFKV_ERR_UNSUPPORTED, "vfkv_attend_prefill: shape outside the tensor-core kernel");
    // The tcgen05 kernel works on 256-row blocks, one CTA per SM: it pays once those fill most of
    // the GPU, or the context is long enough for it to cut the blocks' K/V tiles into even shares
    // for all SMs (256 queries at position 60 000: 1955 us on the mma.sync kernel, 332 us), or
    // for its faster tiles to outweigh its fixed cost; short chunks at short contexts keep the
    // 64-row mma.sync kernel (four times the CTAs).  attn_impl 2 forces it.
    // F16 caches carry the error budget of the reference's f32 shader (2e-3 absolute): the tcgen05
    // kernel feeds Q as one half-precision value, which holds it (1e-4 .. 5e-4 measured) with the usual
    // 1/sqrt(head_dim) scale but not with scale 1.0 (1e-2: the Gemma-4 rule); those keep the
    // mma.sync kernel and its hi + lo split of Q.
    const bool tc5_accurate = dt == VFKV_F8 || scale * sqrtf(float(D)) <= 1.5f;
    if (mma_ok && ctx->attn_impl != 3 && prefill_tc5_supported(dt, D, p.group, kv.k_scales != nullptr) && tc5_accurate &&
        (ctx->attn_impl == 2 || prefill_tc5_pays(ctx, n_q_heads, hkv, m, q_start, n_kv, kv_start, window)))
        return launch_prefill_tc5(ctx, dt, p.k, p.v, d_q, d_out, p.row_bytes, n_q_heads, hkv, m, q_start, n_kv, kv_start,
                                  window, scale, softcap, st);
    if (mma_ok) {
        if (dt == VFKV_F8) {
            if (D == 64) return launch_mma_d<VFKV_F8, 64>(ctx, p, st);
            if (D == 128) return launch_mma_d<VFKV_F8, 128>(ctx, p, st);
            return launch_mma_d<VFKV_F8, 256>(ctx, p, st);
        }
        if (D == 64) return launch_mma_d<VFKV_F16, 64>(ctx, p, st);
        if (D == 128) return launch_mma_d<VFKV_F16, 128>(ctx, p, st);
        return launch_mma_d<VFKV_F16, 256>(ctx, p, st);
    }
    prefill_simple_kernel<<<dim3(m, n_q_heads), 128, 0, st>>>(p, dt);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "prefill attention launch");
}
