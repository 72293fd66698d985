// Chunked-prefill causal attention over the cache on the 5th-generation tensor cores
// (tcgen05.mma with accumulators in tensor memory).  Same function as prefill_mma_kernel in
// attn_prefill.cu (flash_attn_batch.comp:105-208); used for head_dim 128, FP8 caches and, with the
// usual attention scale, F16 caches.
//
// One CTA = two Q tiles of 128 rows (256 / g consecutive queries x the g q-heads of one kv-head),
// one warpgroup per Q tile, x K/V tiles of 128 positions shared by both.  While one warpgroup does
// the softmax of its tile the tensor core works for the other.  Per tile:
//   1. all threads fetch the K and V rows of the tile, widen the FP8 codes to half precision
//      (exact; the kv_fp8_to_f16.comp step) and store them in the 128-byte-swizzled K-major /
//      MN-major layouts the MMA descriptors describe;
//   2. one thread issues S = Q K^T as 8 tcgen05.mma (M 128, N 128, K 16) into tensor memory;
//   3. thread t owns row t: it reads its row of S from tensor memory (tcgen05.ld 32x32b), applies
//      the causal / kv_start / window mask and the online softmax, and writes P in half
//      precision into shared memory (over the K tile, which is dead by then);
//   4. one thread issues O += P V as 8 tcgen05.mma into a second tensor-memory region, which holds
//      the running output for the whole kernel.  The exponents of a row refer to a reference
//      maximum that is moved (and O rescaled in tensor memory) only when the true maximum has
//      outgrown it by more than 2^8, so most tiles cost no rescale at all.
// Every wait on an MMA completion is bounded; a wait that runs out sets status bit 0, the CTA
// leaves the tile loop, frees its tensor memory and returns.
#include "../../include/vfkv_next.h"
#include "common.cuh"
#include "fp8_codec.cuh"

#include <algorithm>
#include <cstring>

namespace vfkv {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int BM = 128, BN = 128, HD = 128;
constexpr int SLAB = 128 * 128;                 // bytes of one [128 rows][64 halves] slab
constexpr int TILE = 2 * SLAB;                  // a [128][128] half-precision tile
constexpr int CTA_ROWS = 2 * BM;                // two Q tiles per CTA, one per warpgroup
constexpr uint32_t kMaxRowBlocks = 512;         // row blocks of 256 rows a launch can spread evenly over the CTAs
constexpr uint32_t TMEM_COLS = 512;             // S of tile 0 and 1: columns 0..255; O of tile 0 and 1: 256..511

struct Tc5Params {
    const uint8_t *k, *v;              // rows of the slot: [pos][kv_head][128] FP8
    const float *q;                    // [m][n_q_heads][128]
    float *out;
    uint64_t row_bytes;
    uint32_t n_q_heads, n_kv_heads, group, m, q_start, n_kv, kv_start, window;
    float scale, softcap;
    uint32_t *status;
    unsigned long long *trace;         // null, or 16 timestamps per warpgroup (phase analysis)
    // specialised form, work spread evenly over the CTAs (n_cta != 0): the K/V tiles of all
    // (row block, kv-head) items in launch order form one line of total_tiles tiles, CTA c takes
    // tiles [c * total / n_cta, (c + 1) * total / n_cta); pieces of items cut by that go to scratch
    uint32_t n_rb, total_tiles, n_cta;
    float *scratch;                    // [n_cta][2] pieces of {O [256][128], reference maximum [256], sum [256]}
    // inline_merge: the CTA that holds the head of a cut item puts it together itself (at most
    // three more pieces, each the first segment of one of the next CTAs, announced by
    // flags[cta] = epoch); the launch is cooperative, so the CTAs it waits for are resident
    uint32_t inline_merge, epoch;
    uint32_t *flags;
    uint32_t use_tma;                  // F16 rows, specialised form: K/V tiles by TMA through the two tensor maps
    uint64_t wait_ns;                  // time limit of the head CTA's wait for the other pieces
    uint32_t fail_cta;                 // failure injection (tests): this CTA never announces its piece
};

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ uint64_t timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
// One box of a byte-typed 2-D tensor map (x bytes into the row, row y) into 128-byte-swizzled shared memory.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int32_t x, int32_t y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 :: "r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// One look at the phase with the given parity.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0u;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
// Bounded wait for the phase with the given parity; false after one second.  The hint lets the
// hardware park the thread for up to that long instead of returning for another look (a waiting
// warp that spins takes issue slots from the warps of its scheduler that work).
constexpr uint32_t kSuspendNs = 20000u;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity)
{
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity), "r"(kSuspendNs) : "memory");
        if (done) return true;
        // the timer is slow to read: look at it only now and then
        if ((it & 255u) == 255u) {
            if (t0 == 0) t0 = timer_ns();
            else if (timer_ns() - t0 > 1000000000ull) return false;
        }
    }
}

// Shared-memory matrix descriptor, 128-byte swizzle, version 1 (sm_100).
// K-major: 8-row groups 1024 B apart (SBO), LBO unused.  MN-major: 64-element groups along
// MN `lbo` bytes apart, 8-row groups along K 1024 B apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    return uint64_t((addr >> 4) & 0x3fffu) | (uint64_t((lbo_bytes >> 4) & 0x3fffu) << 16) |
           (uint64_t((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::f16: F32 accumulate, F16 x F16, M 128, N 128; bit 16 = B is MN-major.
__host__ __device__ constexpr uint32_t idesc_f16(bool b_mn_major)
{
    return (1u << 4) | (uint32_t(b_mn_major) << 16) | (uint32_t(128 >> 3) << 17) | (uint32_t(128 >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32])
{
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// The same load without the wait, into 32 consecutive floats (wait once after a batch of loads).
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, float *v)
{
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float *v)
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 :: "r"(taddr),
                    "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
                    "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
                    "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
                    "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
                    "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
                    "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
                    "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
                    "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
                 : "memory");
}
__device__ __forceinline__ float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi)
{
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
// byte offset of 16-byte chunk c (0..15, 8 halves each) of row r in a [128][128] half tile
__device__ __forceinline__ uint32_t tile_off(uint32_t r, uint32_t c)
{
    return (c >> 3) * SLAB + r * 128 + (((c & 7u) ^ (r & 7u)) << 4);
}

__host__ __device__ __forceinline__ void query_range(const Tc5Params &p, uint32_t i, uint32_t *lo, uint32_t *hi)
{
    uint32_t c = p.q_start + i + 1u;
    if (c > p.n_kv) c = p.n_kv;
    uint32_t l = p.kv_start;
    if (p.window != 0u && c > p.window && c - p.window > l) l = c - p.window;
    if (l > c) l = c;
    *lo = l; *hi = c;
}

// Row block rb (0 = the latest queries, the most K/V tiles) of any kv-head: its first row, the
// first position of its first K/V tile and the number of tiles.
__host__ __device__ __forceinline__ void item_extent(const Tc5Params &p, uint32_t rb, uint32_t *row0, uint32_t *c_lo, uint32_t *n_tiles)
{
    const uint32_t r0 = (p.n_rb - 1u - rb) * uint32_t(CTA_ROWS);
    const uint32_t qa = r0 / p.group;
    uint32_t qb = (r0 + uint32_t(CTA_ROWS) - 1u) / p.group;
    if (qb >= p.m) qb = p.m - 1u;
    uint32_t lo_a, hi_a, lo_b, hi_b;
    query_range(p, qa, &lo_a, &hi_a);
    query_range(p, qb, &lo_b, &hi_b);
    const uint32_t lo = lo_a / uint32_t(BN) * uint32_t(BN);
    *row0 = r0;
    *c_lo = lo;
    *n_tiles = hi_b > lo ? (hi_b - lo + uint32_t(BN) - 1u) / uint32_t(BN) : 0u;
}

template <int DT, bool CAP>
__global__ void __launch_bounds__(256) prefill_tc5_kernel(const Tc5Params p)
{
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_bar[4];
    __shared__ uint32_t s_tmem, s_abort;
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;          // descriptors assume 1024-byte alignment
    uint8_t *sm = smem_raw + (base - smem_addr(smem_raw));
    // shared memory: Q tile 0, Q tile 1, K, V, P of tile 0, P of tile 1
    const uint32_t q_sm = base, k_sm = base + 2 * TILE, v_sm = base + 3 * TILE, p_sm = base + 4 * TILE;
    const uint32_t tid = threadIdx.x, warp = tid >> 5;
    const uint32_t wg = tid >> 7, t = tid & 127u;                           // warpgroup = Q tile, row inside it
    const uint32_t bar_s = smem_addr(&s_bar[wg]), bar_o = smem_addr(&s_bar[2 + wg]);
    const uint32_t kvh = blockIdx.y, g = p.group;
    const uint32_t n_rows = p.m * g;
    const uint32_t row0 = (gridDim.x - 1u - blockIdx.x) * CTA_ROWS;         // heaviest row blocks first

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) mbar_init(smem_addr(&s_bar[i]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_abort = 0u;
    }
    if (warp == 0) {
        __syncwarp();                      // the .sync.aligned instructions need the warp converged
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_addr(&s_tmem)), "n"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    // this thread's row
    const uint32_t r = row0 + wg * BM + t;
    const bool r_ok = r < n_rows;
    const uint32_t q_idx = r_ok ? r / g : 0u, hj = r_ok ? r % g : 0u;
    uint32_t r_lo, r_hi;
    query_range(p, q_idx, &r_lo, &r_hi);
    if (!r_ok) { r_lo = 0u; r_hi = 0u; }
    uint32_t c_lo, c_hi;
    {
        const uint32_t qa = row0 / g;
        uint32_t qb = (row0 + CTA_ROWS - 1) / g;
        if (qb >= p.m) qb = p.m - 1;
        uint32_t lo_a, hi_a, lo_b, hi_b;
        query_range(p, qa, &lo_a, &hi_a);
        query_range(p, qb, &lo_b, &hi_b);
        c_lo = lo_a / BN * BN;
        c_hi = hi_b;
    }
    const uint32_t n_tiles = c_hi > c_lo ? (c_hi - c_lo + BN - 1) / BN : 0u;

    // Q: f32 -> scaled half precision, two K-major swizzled tiles.  Without a soft-cap the factor
    // log2(e) of the exponentials is folded into the scale, so S arrives in log2 units.
    const float qs = CAP ? p.scale : p.scale * kLog2e;
    for (uint32_t i = tid; i < uint32_t(CTA_ROWS * 16); i += 256) {
        const uint32_t row = i >> 4, c = i & 15u;
        const uint32_t rr = row0 + row;
        uint4 hv = make_uint4(0u, 0u, 0u, 0u);
        if (rr < n_rows) {
            const float *qp = p.q + (uint64_t(rr / g) * p.n_q_heads + kvh * g + rr % g) * HD + 8 * c;
            const float4 a = *reinterpret_cast<const float4 *>(qp), b = *reinterpret_cast<const float4 *>(qp + 4);
            hv = make_uint4(pack_half2(a.x * qs, a.y * qs), pack_half2(a.z * qs, a.w * qs),
                            pack_half2(b.x * qs, b.y * qs), pack_half2(b.z * qs, b.w * qs));
        }
        *reinterpret_cast<uint4 *>(sm + (q_sm - base) + (row >> 7) * TILE + tile_off(row & 127u, c)) = hv;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    const uint32_t t_lane = ((warp & 3u) * 32u) << 16;      // this warp's 32 lanes of tensor memory
    const uint32_t tm_s = tmem + wg * 128u, tm_o = tmem + 256u + wg * 128u;   // S and O of this warpgroup's Q tile
    const uint32_t my_p = p_sm + wg * TILE;

    float mref = kMaskedScore, lrow = 0.f;       // reference maximum of the exponents (log2 units), running sum
    constexpr uint32_t ES = DT == VFKV_F8 ? 1u : 2u;           // bytes per cache element
    const uint8_t *kg = p.k + uint64_t(kvh) * HD * ES, *vg = p.v + uint64_t(kvh) * HD * ES;
    uint32_t ph_s = 0, ph_o = 0;

#define TC5_TRACE(i)                                                                                 \
    do {                                                                                             \
        if (p.trace != nullptr && t == 0 && it == 3)                                                 \
            p.trace[((blockIdx.y * gridDim.x + blockIdx.x) * 2 + wg) * 16 + (i)] = timer_ns();       \
    } while (0)
    for (uint32_t it = 0; it < n_tiles; ++it) {
        const uint32_t t0 = c_lo + it * BN;
        // ---- 1. K and V rows of this tile -> half precision in shared memory (all 256 threads) --------
        TC5_TRACE(0);
        if constexpr (DT == VFKV_F8) {
                uint4 raw[8];                                  // 4 pieces of K, 4 of V
    #pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t idx = tid + 256 * (i & 3), pos = idx >> 3, c16 = idx & 7u;
                    const bool ok = t0 + pos < p.n_kv;
                    const uint64_t off = uint64_t(ok ? t0 + pos : 0u) * p.row_bytes + c16 * 16;
                    raw[i] = ok ? __ldg(reinterpret_cast<const uint4 *>((i < 4 ? kg : vg) + off)) : make_uint4(0u, 0u, 0u, 0u);
                }
                auto widen = [&](int i) {
                    const uint32_t idx = tid + 256 * (i & 3), pos = idx >> 3, c16 = idx & 7u;
                    uint8_t *dst = sm + ((i < 4 ? k_sm : v_sm) - base);
                    const uint4 x = raw[i];
                    __half2 h0 = e4m3x2_to_half2(x.x & 0xffffu), h1 = e4m3x2_to_half2(x.x >> 16);
                    __half2 h2 = e4m3x2_to_half2(x.y & 0xffffu), h3 = e4m3x2_to_half2(x.y >> 16);
                    __half2 h4 = e4m3x2_to_half2(x.z & 0xffffu), h5 = e4m3x2_to_half2(x.z >> 16);
                    __half2 h6 = e4m3x2_to_half2(x.w & 0xffffu), h7 = e4m3x2_to_half2(x.w >> 16);
                    *reinterpret_cast<uint4 *>(dst + tile_off(pos, 2 * c16)) =
                        make_uint4(*reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1),
                                   *reinterpret_cast<uint32_t *>(&h2), *reinterpret_cast<uint32_t *>(&h3));
                    *reinterpret_cast<uint4 *>(dst + tile_off(pos, 2 * c16 + 1)) =
                        make_uint4(*reinterpret_cast<uint32_t *>(&h4), *reinterpret_cast<uint32_t *>(&h5),
                                   *reinterpret_cast<uint32_t *>(&h6), *reinterpret_cast<uint32_t *>(&h7));
                };
                // K is free already (both S products of the previous tile were waited for before its
                // softmax): it is widened while the previous tile's P V products still run.  V and P
                // are read by those products, so V waits for them.
                // (this thread waited for its own warpgroup's S product only; the other one's is long
                // complete, the wait makes that a guarantee)
                if (it > 0 && !mbar_wait(smem_addr(&s_bar[wg ^ 1u]), ph_s ^ 1u)) atomicOr(&s_abort, 1u);
    #pragma unroll
                for (int i = 0; i < 4; ++i) widen(i);
                if (it > 0) {
                    if (!mbar_wait(smem_addr(&s_bar[2]), ph_o) || !mbar_wait(smem_addr(&s_bar[3]), ph_o)) atomicOr(&s_abort, 1u);
                    ph_o ^= 1u;
                    __syncwarp();
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                }
                TC5_TRACE(1);
    #pragma unroll
                for (int i = 4; i < 8; ++i) widen(i);
        } else {
            // F16 cache: the rows are half precision already; 16-byte pieces go straight to their
            // swizzled places (8 pieces of K, then 8 of V, per thread)
            uint4 raw[8];
            auto fetch = [&](const uint8_t *src) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t idx = tid + 256 * i, pos = idx >> 4, c = idx & 15u;
                    const bool ok = t0 + pos < p.n_kv;
                    const uint64_t off = uint64_t(ok ? t0 + pos : 0u) * p.row_bytes + c * 16;
                    raw[i] = ok ? __ldg(reinterpret_cast<const uint4 *>(src + off)) : make_uint4(0u, 0u, 0u, 0u);
                }
            };
            auto place = [&](uint32_t tile_sm) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t idx = tid + 256 * i, pos = idx >> 4, c = idx & 15u;
                    *reinterpret_cast<uint4 *>(sm + (tile_sm - base) + tile_off(pos, c)) = raw[i];
                }
            };
            fetch(kg);
            if (it > 0 && !mbar_wait(smem_addr(&s_bar[wg ^ 1u]), ph_s ^ 1u)) atomicOr(&s_abort, 1u);
            place(k_sm);
            fetch(vg);
            if (it > 0) {
                if (!mbar_wait(smem_addr(&s_bar[2]), ph_o) || !mbar_wait(smem_addr(&s_bar[3]), ph_o)) atomicOr(&s_abort, 1u);
                ph_o ^= 1u;
                __syncwarp();
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            TC5_TRACE(1);
            place(v_sm);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic-proxy stores -> visible to the MMA
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        TC5_TRACE(2);
        __syncthreads();
        TC5_TRACE(3);
        if (s_abort) break;                                    // uniform: every writer passed a barrier since
        // ---- 2. S = Q K^T for both Q tiles ----------------------------------------------------------------
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (uint32_t qt = 0; qt < 2; ++qt) {
#pragma unroll
                for (uint32_t ks = 0; ks < HD / 16; ++ks) {
                    const uint32_t o = (ks >> 2) * SLAB + (ks & 3u) * 32;
                    umma_f16(tmem + qt * 128u, smem_desc(q_sm + qt * TILE + o, 16, 1024), smem_desc(k_sm + o, 16, 1024),
                             idesc_f16(false), ks);
                }
                umma_commit(smem_addr(&s_bar[qt]));
            }
        }
        // ---- 3. per warpgroup: this thread's row of S: mask, softmax against the reference maximum ----
        // While warpgroup 0 works on S0 the tensor core computes S1; while warpgroup 1 works on S1
        // it computes O0 += P0 V.
        TC5_TRACE(4);
        if (!mbar_wait(bar_s, ph_s)) atomicOr(&s_abort, 1u);
        ph_s ^= 1u;
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        TC5_TRACE(5);

        const bool full = t0 >= r_lo && t0 + BN <= r_hi;
        // the whole row in registers (one CTA of 256 threads per SM: 255 registers each are there)
        float s[BN];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32_nowait(tm_s + t_lane + 32 * c, &s[32 * c]);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        // tiles inside every row's range (all but the diagonal and window edges) need no mask
        const bool warp_full = __all_sync(0xffffffffu, full);
        float mx = kMaskedScore;
        if (warp_full && !CAP) {
#pragma unroll
            for (int j = 0; j < BN; j += 2) mx = fmaxf(mx, fmaxf(s[j], s[j + 1]));
        } else {
#pragma unroll
            for (int j = 0; j < BN; ++j) {
                float x = s[j];
                if constexpr (CAP) x = p.softcap * tanhf(x / p.softcap) * kLog2e;
                if (!full) {
                    const uint32_t pos = t0 + j;
                    if (pos < r_lo || pos >= r_hi) x = kMaskedScore;
                }
                s[j] = x;
                mx = fmaxf(mx, x);
            }
        }
        TC5_TRACE(6);
        // The accumulator O lives in tensor memory and is rescaled only when a row's maximum has
        // grown by more than 2^8 over the reference its exponents use (so P stays below 256 in
        // half precision); the decision is per warp because the tensor-memory accesses are.
        const bool grow = mx > mref + 8.0f;
        if (__any_sync(0xffffffffu, grow)) {
            const float mnew = grow ? mx : mref;
            const float alpha = fast_exp2(mref - mnew);
            lrow *= alpha;
            mref = mnew;
            if (it > 0) {                                      // O holds the sum of the earlier tiles
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    float o[32];
                    tmem_ld32_nowait(tm_o + t_lane + 32 * c, o);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 32; ++j) o[j] *= alpha;
                    tmem_st32(tm_o + t_lane + 32 * c, o);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
        }
        TC5_TRACE(7);
        float sum = 0.f;
#pragma unroll
        for (int c = 0; c < BN / 8; ++c) {                    // 16 chunks of 8 positions
            uint32_t h[4];
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                const float x0 = s[8 * c + j], x1 = s[8 * c + j + 1];
                float p0 = fast_exp2(x0 - mref), p1 = fast_exp2(x1 - mref);
                if (!warp_full) {                              // a masked position contributes nothing
                    p0 = x0 > 0.5f * kMaskedScore ? p0 : 0.f;
                    p1 = x1 > 0.5f * kMaskedScore ? p1 : 0.f;
                }
                sum += p0 + p1;
                h[j >> 1] = pack_half2(p0, p1);
            }
            // P is K-major over positions
            *reinterpret_cast<uint4 *>(sm + (my_p - base) + tile_off(t, c)) = make_uint4(h[0], h[1], h[2], h[3]);
        }
        lrow += sum;
        TC5_TRACE(8);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        asm volatile("bar.sync %0, 128;" :: "r"(1u + wg) : "memory");      // this warpgroup only
        // ---- 4. O += P V for this warpgroup's Q tile ----------------------------------------------------------
        if (t == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (uint32_t kk = 0; kk < BN / 16; ++kk) {
                const uint32_t ao = (kk >> 2) * SLAB + (kk & 3u) * 32;            // P: K-major, 16 positions per step
                umma_f16(tm_o, smem_desc(my_p + ao, 16, 1024), smem_desc(v_sm + kk * 2048, SLAB, 1024),
                         idesc_f16(true), (it | kk) != 0u ? 1u : 0u);
            }
            umma_commit(bar_o);
        }
        TC5_TRACE(9);
    }
    __syncthreads();
    const bool ran = n_tiles > 0 && s_abort == 0u;
    if (ran) {
        if (!mbar_wait(bar_o, ph_o)) atomicOr(&s_abort, 1u);
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    __syncthreads();
    const bool failed = s_abort != 0u;
    if (failed && tid == 0) atomicOr(p.status, 1u);

    {
        const float inv = (lrow > 0.f && !failed) ? 1.0f / lrow : 0.f;
        float *o = p.out + (uint64_t(q_idx) * p.n_q_heads + kvh * g + hj) * HD;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float v[32];
            if (ran) {
                tmem_ld32_nowait(tm_o + t_lane + 32 * c, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = 0.f;
            }
            if (r_ok) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<float4 *>(o + 32 * c + j) =
                        make_float4(inv > 0.f ? v[j] * inv : 0.f, inv > 0.f ? v[j + 1] * inv : 0.f,
                                    inv > 0.f ? v[j + 2] * inv : 0.f, inv > 0.f ? v[j + 3] * inv : 0.f);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "n"(TMEM_COLS) : "memory");
    }
}

constexpr int kSmemBytes = 6 * TILE + 1024;

// ---- pipelined form ---------------------------------------------------------------------------------
// Same tiles and the same arithmetic as prefill_tc5_kernel, with the two warpgroups running as two
// independent pipelines over the shared K/V tiles:
//   * P stays in tensor memory (half precision, two values per column, over the first 64 columns
//     of the warpgroup's S region) and is the A operand of O += P V straight from there; the two P
//     tiles leave shared memory, which pays for a second K buffer and a second V buffer;
//   * the K/V rows of tile it + 1 are fetched and widened by all threads while S of tile `it` is
//     on the tensor pipe; "tile ready" is an mbarrier with 256 arrivals per buffer, "buffer free"
//     is the completion of both warpgroups' P V products of the tile that used it;
//   * each warpgroup's first thread issues that warpgroup's MMAs, so while one warpgroup computes
//     its softmax the tensor pipe works for the other.
// Barriers: 0,1 S complete (per Q tile)   2,3 P V complete   4,5 K/V buffer 0 / 1 ready.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 :: "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" :: "r"(bar) : "memory");
}

template <int DT, bool CAP>
__global__ void __launch_bounds__(256, 1) prefill_tc5p_kernel(const Tc5Params p)
{
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_bar[6];
    __shared__ uint32_t s_tmem, s_abort[2];                      // one give-up flag per warpgroup
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - smem_addr(smem_raw));
    // shared memory: Q tile 0, Q tile 1, K buffers 0 1, V buffers 0 1
    const uint32_t q_sm = base, k_sm = base + 2 * TILE, v_sm = base + 4 * TILE;
    const uint32_t tid = threadIdx.x, warp = tid >> 5;
    const uint32_t wg = tid >> 7, t = tid & 127u;
    const uint32_t bar_s = smem_addr(&s_bar[wg]), bar_o = smem_addr(&s_bar[2 + wg]);
    const uint32_t kvh = blockIdx.y, g = p.group;
    const uint32_t n_rows = p.m * g;
    const uint32_t row0 = (gridDim.x - 1u - blockIdx.x) * CTA_ROWS;

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) mbar_init(smem_addr(&s_bar[i]), 1);
        mbar_init(smem_addr(&s_bar[4]), 256);
        mbar_init(smem_addr(&s_bar[5]), 256);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_abort[0] = 0u; s_abort[1] = 0u;
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_addr(&s_tmem)), "n"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    const uint32_t r = row0 + wg * BM + t;
    const bool r_ok = r < n_rows;
    const uint32_t q_idx = r_ok ? r / g : 0u, hj = r_ok ? r % g : 0u;
    uint32_t r_lo, r_hi;
    query_range(p, q_idx, &r_lo, &r_hi);
    if (!r_ok) { r_lo = 0u; r_hi = 0u; }
    uint32_t c_lo, c_hi;
    {
        const uint32_t qa = row0 / g;
        uint32_t qb = (row0 + CTA_ROWS - 1) / g;
        if (qb >= p.m) qb = p.m - 1;
        uint32_t lo_a, hi_a, lo_b, hi_b;
        query_range(p, qa, &lo_a, &hi_a);
        query_range(p, qb, &lo_b, &hi_b);
        c_lo = lo_a / BN * BN;
        c_hi = hi_b;
    }
    const uint32_t n_tiles = c_hi > c_lo ? (c_hi - c_lo + BN - 1) / BN : 0u;

    const float qs = CAP ? p.scale : p.scale * kLog2e;
    for (uint32_t i = tid; i < uint32_t(CTA_ROWS * 16); i += 256) {
        const uint32_t row = i >> 4, c = i & 15u;
        const uint32_t rr = row0 + row;
        uint4 hv = make_uint4(0u, 0u, 0u, 0u);
        if (rr < n_rows) {
            const float *qp = p.q + (uint64_t(rr / g) * p.n_q_heads + kvh * g + rr % g) * HD + 8 * c;
            const float4 a = *reinterpret_cast<const float4 *>(qp), b = *reinterpret_cast<const float4 *>(qp + 4);
            hv = make_uint4(pack_half2(a.x * qs, a.y * qs), pack_half2(a.z * qs, a.w * qs),
                            pack_half2(b.x * qs, b.y * qs), pack_half2(b.z * qs, b.w * qs));
        }
        *reinterpret_cast<uint4 *>(sm + (q_sm - base) + (row >> 7) * TILE + tile_off(row & 127u, c)) = hv;
    }

    constexpr uint32_t ES = DT == VFKV_F8 ? 1u : 2u;
    constexpr int NP = DT == VFKV_F8 ? 4 : 8;                 // 16-byte pieces of K (and of V) per thread and tile
    const uint8_t *kg = p.k + uint64_t(kvh) * HD * ES, *vg = p.v + uint64_t(kvh) * HD * ES;
    auto fetch = [&](const uint8_t *src, uint32_t t0, uint4 (&raw)[NP]) {
#pragma unroll
        for (int i = 0; i < NP; ++i) {
            const uint32_t idx = tid + 256 * i;
            const uint32_t pos = DT == VFKV_F8 ? idx >> 3 : idx >> 4, c = DT == VFKV_F8 ? idx & 7u : idx & 15u;
            const bool ok = t0 + pos < p.n_kv;
            const uint64_t off = uint64_t(ok ? t0 + pos : 0u) * p.row_bytes + c * 16;
            raw[i] = ok ? __ldg(reinterpret_cast<const uint4 *>(src + off)) : make_uint4(0u, 0u, 0u, 0u);
        }
    };
    auto place = [&](const uint4 (&raw)[NP], uint32_t tile_sm) {
        uint8_t *dst = sm + (tile_sm - base);
#pragma unroll
        for (int i = 0; i < NP; ++i) {
            const uint32_t idx = tid + 256 * i;
            if constexpr (DT == VFKV_F8) {
                const uint32_t pos = idx >> 3, c16 = idx & 7u;
                const uint4 x = raw[i];
                __half2 h0 = e4m3x2_to_half2(x.x & 0xffffu), h1 = e4m3x2_to_half2(x.x >> 16);
                __half2 h2 = e4m3x2_to_half2(x.y & 0xffffu), h3 = e4m3x2_to_half2(x.y >> 16);
                __half2 h4 = e4m3x2_to_half2(x.z & 0xffffu), h5 = e4m3x2_to_half2(x.z >> 16);
                __half2 h6 = e4m3x2_to_half2(x.w & 0xffffu), h7 = e4m3x2_to_half2(x.w >> 16);
                *reinterpret_cast<uint4 *>(dst + tile_off(pos, 2 * c16)) =
                    make_uint4(*reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1),
                               *reinterpret_cast<uint32_t *>(&h2), *reinterpret_cast<uint32_t *>(&h3));
                *reinterpret_cast<uint4 *>(dst + tile_off(pos, 2 * c16 + 1)) =
                    make_uint4(*reinterpret_cast<uint32_t *>(&h4), *reinterpret_cast<uint32_t *>(&h5),
                               *reinterpret_cast<uint32_t *>(&h6), *reinterpret_cast<uint32_t *>(&h7));
            } else {
                *reinterpret_cast<uint4 *>(dst + tile_off(idx >> 4, idx & 15u)) = raw[i];
            }
        }
    };

    // tile 0 into buffer 0
    if (n_tiles > 0) {
        uint4 raw[NP];
        fetch(kg, c_lo, raw);
        place(raw, k_sm);
        fetch(vg, c_lo, raw);
        place(raw, v_sm);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(smem_addr(&s_bar[4]));
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    const uint32_t t_lane = ((warp & 3u) * 32u) << 16;
    const uint32_t tm_s = tmem + wg * 128u, tm_o = tmem + 256u + wg * 128u;
    volatile uint32_t *abort_flag = &s_abort[wg];            // written and read by this warpgroup only

    float mref = kMaskedScore, lrow = 0.f;
    bool gave_up = false;
    for (uint32_t it = 0; it < n_tiles; ++it) {
        const uint32_t t0 = c_lo + it * BN, b = it & 1u, par = it & 1u;
        const bool more = it + 1 < n_tiles;
        // ---- 1. S = Q K^T of this warpgroup's Q tile.  Its region of tensor memory still holds
        //         P of the previous tile until that tile's P V product is complete.
        TC5_TRACE(0);
        if (it > 0 && !mbar_wait(bar_o, par ^ 1u)) gave_up = true;
        TC5_TRACE(1);
        if (t == 0) {
            if (!mbar_wait(smem_addr(&s_bar[4 + b]), (it >> 1) & 1u)) gave_up = true;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (uint32_t ks = 0; ks < HD / 16; ++ks) {
                const uint32_t o = (ks >> 2) * SLAB + (ks & 3u) * 32;
                umma_f16(tm_s, smem_desc(q_sm + wg * TILE + o, 16, 1024), smem_desc(k_sm + b * TILE + o, 16, 1024),
                         idesc_f16(false), ks);
            }
            umma_commit(bar_s);
        }
        TC5_TRACE(2);
        // ---- 2. K/V rows of the next tile into the other buffer, free once both warpgroups' P V
        //         products of tile it - 1 are complete (this warpgroup's was waited for above).
        if (more) {
            uint4 raw[NP];
            fetch(kg, t0 + BN, raw);
            if (it > 0 && !mbar_wait(smem_addr(&s_bar[2 + (wg ^ 1u)]), par ^ 1u)) gave_up = true;
            place(raw, k_sm + (b ^ 1u) * TILE);
            fetch(vg, t0 + BN, raw);
            place(raw, v_sm + (b ^ 1u) * TILE);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(smem_addr(&s_bar[4 + (b ^ 1u)]));
        }
        TC5_TRACE(3);
        // ---- 3. this thread's row of S: mask, softmax against the reference maximum, P -> tensor memory
        if (!mbar_wait(bar_s, par)) gave_up = true;
        TC5_TRACE(4);
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const bool full = t0 >= r_lo && t0 + BN <= r_hi;
        float s[BN];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32_nowait(tm_s + t_lane + 32 * c, &s[32 * c]);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const bool warp_full = __all_sync(0xffffffffu, full);
        float mx = kMaskedScore;
        if (warp_full && !CAP) {
#pragma unroll
            for (int j = 0; j < BN; j += 2) mx = fmaxf(mx, fmaxf(s[j], s[j + 1]));
        } else {
#pragma unroll
            for (int j = 0; j < BN; ++j) {
                float x = s[j];
                if constexpr (CAP) x = p.softcap * tanhf(x / p.softcap) * kLog2e;
                if (!full) {
                    const uint32_t pos = t0 + j;
                    if (pos < r_lo || pos >= r_hi) x = kMaskedScore;
                }
                s[j] = x;
                mx = fmaxf(mx, x);
            }
        }
        const bool grow = mx > mref + 8.0f;
        if (__any_sync(0xffffffffu, grow)) {
            const float mnew = grow ? mx : mref;
            const float alpha = fast_exp2(mref - mnew);
            lrow *= alpha;
            mref = mnew;
            if (it > 0) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    float o[32];
                    tmem_ld32_nowait(tm_o + t_lane + 32 * c, o);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 32; ++j) o[j] *= alpha;
                    tmem_st32(tm_o + t_lane + 32 * c, o);
                }
            }
        }
        float sum = 0.f;
#pragma unroll
        for (int c = 0; c < 2; ++c) {                         // 64 positions = 32 packed columns per store
            float pk[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float x0 = s[64 * c + 2 * j], x1 = s[64 * c + 2 * j + 1];
                float p0 = fast_exp2(x0 - mref), p1 = fast_exp2(x1 - mref);
                if (!warp_full) {
                    p0 = x0 > 0.5f * kMaskedScore ? p0 : 0.f;
                    p1 = x1 > 0.5f * kMaskedScore ? p1 : 0.f;
                }
                sum += p0 + p1;
                pk[j] = __uint_as_float(pack_half2(p0, p1));   // position 2j in the low half
            }
            tmem_st32(tm_s + t_lane + 32 * c, pk);
        }
        lrow += sum;
        TC5_TRACE(5);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        if (gave_up) *abort_flag = 1u;
        asm volatile("bar.sync %0, 128;" :: "r"(1u + wg) : "memory");      // this warpgroup only
        TC5_TRACE(6);
        if (*abort_flag) break;                                            // the same value for the whole warpgroup
        // ---- 4. O += P V: A from tensor memory (16 positions = 8 columns per step), B = V rows (MN-major)
        if (t == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (uint32_t kk = 0; kk < BN / 16; ++kk)
                umma_f16_ts(tm_o, tm_s + kk * 8u, smem_desc(v_sm + b * TILE + kk * 2048, SLAB, 1024), idesc_f16(true),
                            (it | kk) != 0u ? 1u : 0u);
            umma_commit(bar_o);
        }
        TC5_TRACE(7);
    }
    const bool ran = n_tiles > 0 && *abort_flag == 0u;
    if (ran) {
        if (!mbar_wait(bar_o, (n_tiles - 1u) & 1u)) *abort_flag = 1u;
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    __syncthreads();
    const bool failed = (s_abort[0] | s_abort[1]) != 0u;
    if (failed && tid == 0) atomicOr(p.status, 1u);
    {
        const float inv = (lrow > 0.f && !failed) ? 1.0f / lrow : 0.f;
        float *o = p.out + (uint64_t(q_idx) * p.n_q_heads + kvh * g + hj) * HD;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float v[32];
            if (ran && !failed) {
                tmem_ld32_nowait(tm_o + t_lane + 32 * c, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = 0.f;
            }
            if (r_ok) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<float4 *>(o + 32 * c + j) =
                        make_float4(inv > 0.f ? v[j] * inv : 0.f, inv > 0.f ? v[j + 1] * inv : 0.f,
                                    inv > 0.f ? v[j + 2] * inv : 0.f, inv > 0.f ? v[j + 3] * inv : 0.f);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "n"(TMEM_COLS) : "memory");
    }
}


// ---- specialised form ----------------------------------------------------------------------------------
// tcgen05.mma holds the thread that issues it for as long as the tensor pipe is busy (measured in
// the two forms above: 0.5-0.7 us per group of 8), and in those forms that thread also owns a row
// of the softmax, so 127 threads wait for it at every barrier.  Here the roles are separate warps:
//   warps 0-3 / 4-7   softmax of Q tile 0 / 1 (thread t = row t), in halves of 64 positions;
//   warp 8            one thread issues every MMA;
//   warps 9-11        fetch, widen and place the K/V tiles (two buffers each); F16 rows: one thread
//                     of them issues TMA copies instead.
// Twelve warps leave 168 registers a thread, which is why a row is handled 64 columns at a time;
// per Q tile and K/V tile: S = Q K^T (N = 128, one piece: two N = 64 products measured twice the
// time) -> softmax of columns 0-63 -> P half a (tensor memory) -> O += P V (K = 64) while the
// softmax of columns 64-127 runs -> P half b -> O += P V, and right behind that the S of the next
// K/V tile.  MMAs issued by the one thread execute in issue order, which is what lets the next S be
// issued behind the P V that reads P from the same tensor-memory columns; with two Q tiles the
// tensor pipe has the other tile's products to run while one is in its softmax.
// mbarriers (count): S ready [tile] (1, commit)   P ready [tile][half] (128)   P V done
// [tile][half] (1, commit)   K / V ready [buffer] (96)   K / V free [buffer] (1, commit).  Each
// completes once per K/V tile (or once per two), so a wait on a phase parity is never more than
// one phase away from the barrier's state.
__host__ __device__ constexpr uint32_t idesc_f16_n(bool b_mn_major, uint32_t n)
{
    return (1u << 4) | (uint32_t(b_mn_major) << 16) | (uint32_t(n >> 3) << 17) | (uint32_t(128 >> 4) << 24);
}

// 64 columns of this thread's lane, loaded and waited for inside one statement: the compiler may
// not touch the destination registers before the wait (it knows nothing of the load being
// asynchronous).
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&v)[64])
{
    uint32_t r[64];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n\t"
                 "tcgen05.wait::ld.sync.aligned;"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
                 : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}

// Bounded wait for a flag that another CTA of this (cooperative) launch sets; false after limit_ns.
__device__ __forceinline__ bool flag_wait(const uint32_t *flag, uint32_t want, uint64_t limit_ns)
{
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
        uint32_t v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v == want) return true;
        if ((it & 63u) == 63u) {
            if (t0 == 0) t0 = timer_ns();
            else if (timer_ns() - t0 > limit_ns) return false;
        }
    }
}

template <int DT, bool CAP>
__global__ void __launch_bounds__(384, 1) prefill_tc5h_kernel(const Tc5Params p, const __grid_constant__ CUtensorMap tm_k,
                                                              const __grid_constant__ CUtensorMap tm_v)
{
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_bar[20];
    __shared__ uint32_t s_tmem, s_abort, s_seg[7];
    __shared__ uint32_t s_tj[kMaxRowBlocks], s_cl[kMaxRowBlocks];      // tiles and first position of every row block
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - smem_addr(smem_raw));
    const uint32_t q_sm = base, k_sm = base + 2 * TILE, v_sm = base + 4 * TILE;
    const uint32_t tid = threadIdx.x, warp = tid >> 5;
    // One CTA per item (n_cta == 0): grid = (kv-heads, row blocks), the heaviest row blocks (latest
    // queries) of every kv-head start first.  Work spread evenly (n_cta != 0): grid = n_cta, this CTA
    // takes its share of the line of all items' tiles as a sequence of segments, each a run of
    // K/V tiles of one item; a segment that is a whole item writes the output rows, the first and
    // the last segment may be pieces of items and go to scratch for prefill_tc5_merge_kernel.
    const uint32_t g = p.group;
    const uint32_t n_rows = p.m * g;
#define TC5H_STAMP(slot)                                                                           \
    do {                                                                                           \
        if (p.trace != nullptr && seg_i == 0u)                                                     \
            p.trace[(blockIdx.x * gridDim.y + blockIdx.y) * 32 + (slot)] = timer_ns();             \
    } while (0)
    auto bar = [&](uint32_t i) { return smem_addr(&s_bar[i]); };
    // 0-1 S ready (tile)   4-7 P ready (tile * 2 + half)   8-11 P V done (tile * 2 + half)   12-13 K ready
    // 14-15 V ready   16-17 K free   18-19 V free
    if (tid == 0) {
        for (uint32_t i = 0; i < 4; ++i) mbar_init(bar(i), 1);
        for (uint32_t i = 4; i < 8; ++i) mbar_init(bar(i), 128);
        for (uint32_t i = 8; i < 12; ++i) mbar_init(bar(i), 1);
        for (uint32_t i = 12; i < 16; ++i) mbar_init(bar(i), p.use_tma != 0u ? 1u : 96u);
        for (uint32_t i = 16; i < 20; ++i) mbar_init(bar(i), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_abort = 0u;
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_addr(&s_tmem)), "n"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    const float qs = CAP ? p.scale : p.scale * kLog2e;
    volatile uint32_t *abort_flag = &s_abort;
    uint32_t cur = 0u, t_end = 0u;                       // this CTA's tiles on the line of all tiles
    if (p.n_cta != 0u) {
        cur = uint32_t(uint64_t(blockIdx.x) * p.total_tiles / p.n_cta);
        t_end = uint32_t(uint64_t(blockIdx.x + 1u) * p.total_tiles / p.n_cta);
    }
    const uint32_t t_begin = cur;
    if (p.n_cta != 0u) {
        // one thread walking the row blocks with item_extent (divisions, clamps) costs 0.8 us a row
        // block; all threads fill a table once, the walk then only adds
        for (uint32_t rb = tid; rb < p.n_rb; rb += 384u) {
            uint32_t r0, cl, tj;
            item_extent(p, rb, &r0, &cl, &tj);
            s_tj[rb] = tj;
            s_cl[rb] = cl;
        }
        __syncthreads();
    }
    // K/V tiles this CTA has been through: every barrier completes once per tile (K/V ready and
    // free: once per two), so all phase parities follow from this count, across segments
    uint32_t gt = 0u;
    uint32_t tmem = 0u;
    for (uint32_t seg_i = 0u;; ++seg_i) {
        if (tid == 0) {
            TC5H_STAMP(13);
            uint32_t live = 0u, kvh_ = 0u, row0_ = 0u, c_lo_ = 0u, nt_ = 0u, mode_ = 0u, more_ = 0u;
            if (p.n_cta == 0u) {
                if (seg_i == 0u) { live = 1u; kvh_ = blockIdx.x; item_extent(p, blockIdx.y, &row0_, &c_lo_, &nt_); }
            } else if (cur < t_end) {
                uint32_t acc = 0u;
                for (uint32_t rb = 0u; rb < p.n_rb; ++rb) {
                    const uint32_t tj = s_tj[rb];
                    const uint32_t blk = tj * p.n_kv_heads;
                    if (cur < acc + blk) {
                        const uint32_t rel = cur - acc;
                        kvh_ = rel / tj;
                        const uint32_t tin = rel - kvh_ * tj;
                        nt_ = min(tj - tin, t_end - cur);
                        row0_ = (p.n_rb - 1u - rb) * uint32_t(CTA_ROWS);
                        c_lo_ = s_cl[rb] + tin * BN;
                        // 0: a whole item; 1 / 2: a piece of one for the merge kernel, as this CTA's first / a
                        // later segment; 3: a piece that is not the item's head, for the CTA that holds the
                        // head; 4: the head, which waits for the more_ pieces of the next CTAs
                        if (tin == 0u && nt_ == tj) mode_ = 0u;
                        else if (p.inline_merge == 0u) mode_ = cur == t_begin ? 1u : 2u;
                        else if (tin != 0u) mode_ = 3u;
                        else {
                            mode_ = 4u;
                            const uint64_t e = uint64_t(acc) + uint64_t(kvh_ + 1u) * tj;
                            more_ = uint32_t((e * p.n_cta - 1u) / p.total_tiles) - blockIdx.x;
                        }
                        live = 1u;
                        break;
                    }
                    acc += blk;
                }
            }
            s_seg[0] = live; s_seg[1] = kvh_; s_seg[2] = row0_; s_seg[3] = c_lo_; s_seg[4] = nt_; s_seg[5] = mode_; s_seg[6] = more_;
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        tmem = s_tmem;
        if (s_seg[0] == 0u) break;
        const uint32_t kvh = s_seg[1], row0 = s_seg[2], c_lo = s_seg[3], n_tiles = s_seg[4], mode = s_seg[5], n_more = s_seg[6];

        // Q tiles -> shared memory (half precision, scale folded in), all threads
        // by the nine warps that are not fetching K/V (those start on their first tiles meanwhile);
        // eight pieces a thread in flight at a time, two rounds.  g divides 128, so it is a power of two.
        if (warp < 9u) {
            constexpr uint32_t QT = 288u, QB = 8u;
            const uint32_t g_shift = uint32_t(__ffs(int(g))) - 1u;
            for (uint32_t i0 = tid; i0 < uint32_t(CTA_ROWS * 16); i0 += QT * QB) {
                float4 qa[QB], qb[QB];
#pragma unroll
                for (uint32_t u = 0; u < QB; ++u) {
                    const uint32_t i = i0 + QT * u, row = i >> 4, c = i & 15u, rr = row0 + row;
                    const bool in = i < uint32_t(CTA_ROWS * 16) && rr < n_rows;
                    const float *qp = p.q + (uint64_t(in ? rr >> g_shift : 0u) * p.n_q_heads + kvh * g + (in ? rr & (g - 1u) : 0u)) * HD + 8 * c;
                    qa[u] = in ? __ldg(reinterpret_cast<const float4 *>(qp)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    qb[u] = in ? __ldg(reinterpret_cast<const float4 *>(qp + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (uint32_t u = 0; u < QB; ++u) {
                    const uint32_t i = i0 + QT * u, row = i >> 4, c = i & 15u;
                    if (i < uint32_t(CTA_ROWS * 16))
                        *reinterpret_cast<uint4 *>(sm + (q_sm - base) + (row >> 7) * TILE + tile_off(row & 127u, c)) =
                            make_uint4(pack_half2(qa[u].x * qs, qa[u].y * qs), pack_half2(qa[u].z * qs, qa[u].w * qs),
                                       pack_half2(qb[u].x * qs, qb[u].y * qs), pack_half2(qb[u].z * qs, qb[u].w * qs));
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("bar.sync 1, 288;" ::: "memory");
        }
        if (tid == 0) TC5H_STAMP(14);
#define TC5H_TRACE(slot)                                                                           \
    do {                                                                                           \
        if (p.trace != nullptr && it == 3u && seg_i == 0u)                                         \
            p.trace[(blockIdx.x * gridDim.y + blockIdx.y) * 32 + (slot)] = timer_ns();             \
    } while (0)

        if (warp < 8) {
            // ================= softmax warps: thread t of warpgroup wg owns row t of Q tile wg =============
            const uint32_t wg = warp >> 2, t = tid & 127u;
            const uint32_t r = row0 + wg * BM + t;
            const bool r_ok = r < n_rows;
            const uint32_t q_idx = r_ok ? r / g : 0u, hj = r_ok ? r % g : 0u;
            uint32_t r_lo, r_hi;
            query_range(p, q_idx, &r_lo, &r_hi);
            if (!r_ok) { r_lo = 0u; r_hi = 0u; }
            const uint32_t t_lane = ((warp & 3u) * 32u) << 16;
            const uint32_t tm_s = tmem + wg * 128u, tm_o = tmem + 256u + wg * 128u;
            float mref = kMaskedScore, lrow = 0.f;
            bool ok = true;
            for (uint32_t it = 0; it < n_tiles && ok; ++it) {
                if (tid == 0) TC5H_TRACE(16);
                const uint32_t gi = gt + it;
                if (!mbar_wait(bar(wg), gi & 1u)) { ok = false; break; }
                if (tid == 0 && it == 0u) TC5H_STAMP(15);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
                for (uint32_t h = 0; h < 2u; ++h) {
                    const uint32_t t0 = c_lo + it * BN + h * 64u;
                    if (tid == 0) TC5H_TRACE(17 + 4 * h);
                    float s[64];
                    tmem_ld64(tm_s + t_lane + 64u * h, s);
                    const bool full = t0 >= r_lo && t0 + 64u <= r_hi;
                    const bool warp_full = __all_sync(0xffffffffu, full);
                    float mx = kMaskedScore;
                    if (warp_full && !CAP) {
#pragma unroll
                        for (int j = 0; j < 64; j += 2) mx = fmaxf(mx, fmaxf(s[j], s[j + 1]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 64; ++j) {
                            float x = s[j];
                            if constexpr (CAP) x = p.softcap * tanhf(x / p.softcap) * kLog2e;
                            if (!full) {
                                const uint32_t pos = t0 + j;
                                if (pos < r_lo || pos >= r_hi) x = kMaskedScore;
                            }
                            s[j] = x;
                            mx = fmaxf(mx, x);
                        }
                    }
                    const bool grow = mx > mref + 8.0f;
                    if (__any_sync(0xffffffffu, grow)) {
                        const float mnew = grow ? mx : mref;
                        const float alpha = fast_exp2(mref - mnew);
                        lrow *= alpha;
                        mref = mnew;
                        if (it > 0u || h > 0u) {
                            // O is touched only between P V products: the latest one of this Q tile has to be
                            // complete -- half b of the tile before, or half a of this tile
                            if (!mbar_wait(bar(8u + wg * 2u + (h ^ 1u)), (h == 0u ? gi - 1u : gi) & 1u)) { ok = false; break; }
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
                            for (int c = 0; c < 4; ++c) {
                                float o[32];
                                tmem_ld32(tm_o + t_lane + 32 * c, o);
#pragma unroll
                                for (int j = 0; j < 32; ++j) o[j] *= alpha;
                                tmem_st32(tm_o + t_lane + 32 * c, o);
                                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");   // the registers are reused by the next load
                            }
                        }
                    }
                    if (tid == 0) TC5H_TRACE(18 + 4 * h);
                    // (the offsets and the row sum as packed add.f32x2, two columns an instruction:
                    // 653 -> 696 us on 2048 queries at 14 336, not kept)
                    float sum = 0.f;
                    float pk[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float x0 = s[2 * j], x1 = s[2 * j + 1];
                        float p0 = fast_exp2(x0 - mref), p1 = fast_exp2(x1 - mref);
                        if (!warp_full) {
                            p0 = x0 > 0.5f * kMaskedScore ? p0 : 0.f;
                            p1 = x1 > 0.5f * kMaskedScore ? p1 : 0.f;
                        }
                        sum += p0 + p1;
                        pk[j] = __uint_as_float(pack_half2(p0, p1));   // position 2j in the low half
                    }
                    lrow += sum;
                    // (P of half a stored and S of half b loaded in one statement, both in flight together:
                    // 632 -> 702 us on 2048 queries at 14 336, not kept)
                    tmem_st32(tm_s + t_lane + 64u * h, pk);
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    mbar_arrive(bar(4u + wg * 2u + h));
                    if (tid == 0) TC5H_TRACE(19 + 4 * h);
                }
            }
            if (!ok) *abort_flag = 1u;
            if (tid == 0) TC5H_STAMP(27);
            // the last P V of this Q tile
            bool ran = n_tiles > 0 && ok;
            if (ran && !mbar_wait(bar(8u + wg * 2u + 1u), (gt + n_tiles - 1u) & 1u)) { *abort_flag = 1u; ran = false; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool failed = *abort_flag != 0u;
            if (tid == 0) TC5H_STAMP(28);
            // The rows leave through shared memory so that a warp's store covers one row's 512 bytes (a
            // thread storing its own row writes 32 separate sectors an instruction: 5 us a CTA).  Each
            // softmax warp stages its 32 rows in its own 16 KB of the Q and K tiles, which no product
            // reads any more: every S product was issued before, and so completed before, the P V this
            // thread has just waited for.  16-byte pieces are placed at (piece ^ row) so that neither
            // the row-wise writes nor the piece-wise reads meet in a bank.
            float row_scale;
            float *row_dst;
            float piece_scale[3] = {0.f, 0.f, 0.f};
            constexpr uint64_t PIECE = uint64_t(CTA_ROWS) * (HD + 2);
            if (mode == 4u) {
                // the head of a cut item: the other pieces were the first work of the next CTAs
                const uint32_t rl = wg * BM + t;
                bool got = true;
                for (uint32_t i = 1u; i <= n_more; ++i) got = flag_wait(p.flags + blockIdx.x + i, p.epoch, p.wait_ns) && got;
                if (!got) *abort_flag = 1u;
                const bool mine_ok = ran && !failed;
                float mx = mine_ok ? mref : kMaskedScore, pm[3], pl[3];
#pragma unroll
                for (uint32_t i = 0; i < 3u; ++i) {
                    const bool on = i < n_more && got;
                    const float *pc = p.scratch + uint64_t(blockIdx.x + 1u + (on ? i : 0u)) * 2u * PIECE;
                    pm[i] = on ? __ldcg(pc + CTA_ROWS * HD + rl) : kMaskedScore;
                    pl[i] = on ? __ldcg(pc + CTA_ROWS * HD + CTA_ROWS + rl) : 0.f;
                    mx = fmaxf(mx, pm[i]);
                }
                const float w_own = mine_ok ? fast_exp2(mref - mx) : 0.f;
                float lsum = w_own * lrow;
#pragma unroll
                for (uint32_t i = 0; i < 3u; ++i) {
                    piece_scale[i] = fast_exp2(pm[i] - mx);
                    lsum += piece_scale[i] * pl[i];
                }
                const float inv = (lsum > 0.f && got && !failed) ? 1.0f / lsum : 0.f;
                row_scale = w_own * inv;
#pragma unroll
                for (uint32_t i = 0; i < 3u; ++i) piece_scale[i] *= inv;
                row_dst = r_ok ? p.out + (uint64_t(q_idx) * p.n_q_heads + kvh * g + hj) * HD : nullptr;
            } else if (mode != 0u) {
                // a piece of an item: O as it stands, with the reference maximum (log2 units) and the sum
                float *sc = p.scratch + (uint64_t(blockIdx.x) * 2u + (mode == 2u ? 1u : 0u)) * PIECE;
                const uint32_t rl = wg * BM + t;
                sc[CTA_ROWS * HD + rl] = (ran && !failed) ? mref : kMaskedScore;
                sc[CTA_ROWS * HD + CTA_ROWS + rl] = (ran && !failed) ? lrow : 0.f;
                row_scale = 1.0f;
                row_dst = sc + rl * HD;
            } else {
                row_scale = (lrow > 0.f && !failed) ? 1.0f / lrow : 0.f;
                row_dst = r_ok ? p.out + (uint64_t(q_idx) * p.n_q_heads + kvh * g + hj) * HD : nullptr;
            }
            {
                uint8_t *stage = sm + (q_sm - base) + warp * 16384u;
                const uint32_t lane = tid & 31u;
#pragma unroll 1
                for (uint32_t c = 0; c < 4u; ++c) {
                    float v[32];
                    if (ran && !failed) {
                        tmem_ld32(tm_o + t_lane + 32 * c, v);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = 0.f;
                    }
#pragma unroll
                    for (uint32_t j = 0; j < 8u; ++j)
                        *reinterpret_cast<float4 *>(stage + lane * 512u + ((((8u * c + j) ^ lane) & 31u) << 4)) =
                            make_float4(v[4 * j] * row_scale, v[4 * j + 1] * row_scale, v[4 * j + 2] * row_scale, v[4 * j + 3] * row_scale);
                }
                __syncwarp();
                const unsigned long long mine = reinterpret_cast<unsigned long long>(row_dst);
#pragma unroll 4
                for (uint32_t r = 0; r < 32u; ++r) {
                    const unsigned long long dst = __shfl_sync(0xffffffffu, mine, int(r));
                    float4 x = *reinterpret_cast<const float4 *>(stage + r * 512u + (((lane ^ r) & 31u) << 4));
                    if (mode == 4u) {
#pragma unroll
                        for (uint32_t i = 0; i < 3u; ++i) {
                            const float ps = __shfl_sync(0xffffffffu, piece_scale[i], int(r));
                            if (i < n_more && dst != 0ull) {
                                const float4 y = __ldcg(reinterpret_cast<const float4 *>(
                                    p.scratch + uint64_t(blockIdx.x + 1u + i) * 2u * PIECE + (wg * BM + (warp & 3u) * 32u + r) * HD + 4u * lane));
                                x.x += ps * y.x; x.y += ps * y.y; x.z += ps * y.z; x.w += ps * y.w;
                            }
                        }
                    }
                    if (dst != 0ull) *reinterpret_cast<float4 *>(reinterpret_cast<float *>(dst) + 4u * lane) = x;
                }
                __syncwarp();
            }
        } else if (warp == 8) {
            // ================= the MMA thread ================================================================
            if ((tid & 31u) == 0u && n_tiles > 0u) {
                bool ok = true;
                // S of one Q tile in one piece (N = 128): two N = 64 products take twice the time
                auto issue_s = [&](uint32_t wg, uint32_t b) {
#pragma unroll
                    for (uint32_t ks = 0; ks < HD / 16; ++ks) {
                        const uint32_t o = (ks >> 2) * SLAB + (ks & 3u) * 32;
                        umma_f16(tmem + wg * 128u, smem_desc(q_sm + wg * TILE + o, 16, 1024),
                                 smem_desc(k_sm + b * TILE + o, 16, 1024), idesc_f16(false), ks);
                    }
                    umma_commit(bar(wg));
                };
                if (!mbar_wait(bar(12u + (gt & 1u)), (gt >> 1) & 1u)) ok = false;
                if (ok) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    issue_s(0, gt & 1u); issue_s(1, gt & 1u);
                    umma_commit(bar(16u + (gt & 1u)));
                }
                // Per K/V tile six groups of products: P V of (Q tile, half) x 4 and S of the next tile x 2.
                // They are issued as their inputs arrive -- a look at the four P barriers in turn -- and
                // not in a fixed order: in a fixed order (P V a0, a1, b0, then S0 alternating with P V
                // b1, then S1) Q tile 0 waited for Q tile 1's softmax before its next S was issued
                // (653 -> 643 us on 2048 queries at 14 336, 1258 -> 1234 at 30 000).  The S of the next
                // tile for a Q tile goes right behind that Q tile's P V of half b (its S columns hold
                // P until then; MMAs of one thread execute in order), alternating with a P V of the
                // other Q tile when one is ready at that moment: consecutive MMAs into the same
                // accumulator follow one another about every 60 ns, MMAs into different accumulators
                // about every 40 ns (measured).  (Taking the ready groups of both Q tiles together whenever
                // both are ready, their MMAs alternating, measured 627 -> 710 us: the two softmaxes then
                // run in step and the tensor pipe idles while both compute; the stagger is what keeps it fed.)
                for (uint32_t it = 0; it < n_tiles && ok; ++it) {
                    const uint32_t gi = gt + it, b = gi & 1u;
                    const bool more = it + 1u < n_tiles;
                    auto pv_step = [&](uint32_t wg, uint32_t h, uint32_t kk) {
                        umma_f16_ts(tmem + 256u + wg * 128u, tmem + wg * 128u + 64u * h + kk * 8u,
                                    smem_desc(v_sm + b * TILE + (4u * h + kk) * 2048u, SLAB, 1024), idesc_f16(true),
                                    (it | h | kk) != 0u ? 1u : 0u);
                    };
                    auto s_step = [&](uint32_t wg, uint32_t bb, uint32_t ks) {
                        const uint32_t o = (ks >> 2) * SLAB + (ks & 3u) * 32;
                        umma_f16(tmem + wg * 128u, smem_desc(q_sm + wg * TILE + o, 16, 1024),
                                 smem_desc(k_sm + bb * TILE + o, 16, 1024), idesc_f16(false), ks);
                    };
                    TC5H_TRACE(0);
                    if (!mbar_wait(bar(14u + b), (gi >> 1) & 1u)) { ok = false; break; }
                    bool k_next = !more;
                    uint32_t todo = 0xFu;                  // bit h * 2 + wg: P V of (Q tile wg, half h) not issued yet
                    uint64_t t_idle = 0;
                    uint32_t idle = 0;
                    while (todo != 0u && ok) {
                        bool did = false;
#pragma unroll 1
                        for (uint32_t wg = 0; wg < 2u && ok; ++wg) {
                            const uint32_t h = ((todo >> wg) & 1u) ? 0u : 1u;            // half a before half b
                            if (((todo >> (h * 2u + wg)) & 1u) == 0u) continue;
                            if (!mbar_test(bar(4u + wg * 2u + h), gi & 1u)) continue;
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                            did = true;
#pragma unroll
                            for (uint32_t kk = 0; kk < 4u; ++kk) pv_step(wg, h, kk);
                            umma_commit(bar(8u + wg * 2u + h));
                            todo &= ~(1u << (h * 2u + wg));
                            if (h == 0u || !more) continue;
                            // S of the next K/V tile for this Q tile: its S columns are free behind the P V
                            // just issued.  Alternating with a P V of the other Q tile if one is ready now.
                            if (!k_next) {
                                if (!mbar_wait(bar(12u + (b ^ 1u)), ((gi + 1u) >> 1) & 1u)) { ok = false; break; }
                                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                                k_next = true;
                            }
                            const uint32_t other = wg ^ 1u, ho = ((todo >> other) & 1u) ? 0u : 1u;
                            const bool pair = ((todo >> (ho * 2u + other)) & 1u) != 0u && mbar_test(bar(4u + other * 2u + ho), gi & 1u);
                            if (pair) asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                            for (uint32_t ks = 0; ks < HD / 16; ++ks) {
                                s_step(wg, b ^ 1u, ks);
                                if (pair && ks < 4u) pv_step(other, ho, ks);
                            }
                            if (pair) {
                                umma_commit(bar(8u + other * 2u + ho));
                                todo &= ~(1u << (ho * 2u + other));
                            }
                            umma_commit(bar(wg));
                            if (pair && ho == 1u) {
#pragma unroll
                                for (uint32_t ks = 0; ks < HD / 16; ++ks) s_step(other, b ^ 1u, ks);
                                umma_commit(bar(other));
                            }
                        }
                        if (!did) {
                            if ((++idle & 1023u) == 0u) {
                                if (t_idle == 0) t_idle = timer_ns();
                                else if (timer_ns() - t_idle > 1000000000ull) ok = false;
                            }
                        } else {
                            idle = 0; t_idle = 0;
                        }
                    }
                    if (!ok) break;
                    umma_commit(bar(18u + b));
                    if (more) umma_commit(bar(16u + (b ^ 1u)));
                    TC5H_TRACE(12);
                }
                if (!ok) *abort_flag = 1u;
            }
        } else {
            // ================= K/V tiles: fetch, widen, place (96 threads) =====================================
            const uint32_t pt = tid - 288u;
            constexpr uint32_t ES = DT == VFKV_F8 ? 1u : 2u;
            constexpr uint32_t PIECES = DT == VFKV_F8 ? 1024u : 2048u;          // 16-byte pieces of one K (or V) tile
            constexpr int NP = DT == VFKV_F8 ? 11 : 11;                          // pieces per thread and pass
            constexpr int PASSES = DT == VFKV_F8 ? 1 : 2;
            const uint8_t *kg = p.k + uint64_t(kvh) * HD * ES, *vg = p.v + uint64_t(kvh) * HD * ES;
            bool ok = true;
            auto move = [&](const uint8_t *src, uint32_t t0, uint32_t tile_sm, uint32_t free_bar, uint32_t gi) {
                uint8_t *dst = sm + (tile_sm - base);
#pragma unroll 1
                for (int pass = 0; pass < PASSES; ++pass) {
                    uint4 raw[NP];
#pragma unroll
                    for (int i = 0; i < NP; ++i) {
                        const uint32_t idx = pt + 96u * uint32_t(i) + uint32_t(pass) * (96u * NP);
                        const uint32_t pos = DT == VFKV_F8 ? idx >> 3 : idx >> 4, c = DT == VFKV_F8 ? idx & 7u : idx & 15u;
                        const bool in = idx < PIECES && t0 + pos < p.n_kv;
                        const uint64_t off = uint64_t(in ? t0 + pos : 0u) * p.row_bytes + c * 16;
                        raw[i] = in ? __ldg(reinterpret_cast<const uint4 *>(src + off)) : make_uint4(0u, 0u, 0u, 0u);
                    }
                    // the buffer is free once the products of the tile that used it two tiles ago are complete
                    if (pass == 0 && gi >= 2u && !mbar_wait(free_bar, ((gi >> 1) & 1u) ^ 1u)) ok = false;
#pragma unroll
                    for (int i = 0; i < NP; ++i) {
                        const uint32_t idx = pt + 96u * uint32_t(i) + uint32_t(pass) * (96u * NP);
                        if (idx >= PIECES) continue;
                        if constexpr (DT == VFKV_F8) {
                            const uint32_t pos = idx >> 3, c16 = idx & 7u;
                            const uint4 x = raw[i];
                            __half2 h0 = e4m3x2_to_half2(x.x & 0xffffu), h1 = e4m3x2_to_half2(x.x >> 16);
                            __half2 h2 = e4m3x2_to_half2(x.y & 0xffffu), h3 = e4m3x2_to_half2(x.y >> 16);
                            __half2 h4 = e4m3x2_to_half2(x.z & 0xffffu), h5 = e4m3x2_to_half2(x.z >> 16);
                            __half2 h6 = e4m3x2_to_half2(x.w & 0xffffu), h7 = e4m3x2_to_half2(x.w >> 16);
                            // (two ways of taking the two-way bank conflict out of these stores -- even pieces
                            // from four threads of a row and odd pieces from the other four; two adjacent rows
                            // x four pieces per group of eight threads -- both measured 4-5 % slower at contexts
                            // of 30 000 and more, and the same below)
                            *reinterpret_cast<uint4 *>(dst + tile_off(pos, 2 * c16)) =
                                make_uint4(*reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1),
                                           *reinterpret_cast<uint32_t *>(&h2), *reinterpret_cast<uint32_t *>(&h3));
                            *reinterpret_cast<uint4 *>(dst + tile_off(pos, 2 * c16 + 1)) =
                                make_uint4(*reinterpret_cast<uint32_t *>(&h4), *reinterpret_cast<uint32_t *>(&h5),
                                           *reinterpret_cast<uint32_t *>(&h6), *reinterpret_cast<uint32_t *>(&h7));
                        } else {
                            *reinterpret_cast<uint4 *>(dst + tile_off(idx >> 4, idx & 15u)) = raw[i];
                        }
                    }
                }
            };
            if (DT == VFKV_F16 && p.use_tma != 0u) {
                // F16 rows need no widening: one thread has the TMA unit copy each tile's two slabs of
                // K and of V (box = 128 bytes x 128 positions, the swizzle the descriptors expect;
                // positions from n_kv on, outside the map, arrive as zeros)
                if (pt == 0u) {
                    for (uint32_t it = 0; it < n_tiles && ok; ++it) {
                        const uint32_t gi = gt + it, b = gi & 1u;
                        const int32_t t0 = int32_t(c_lo + it * BN), x = int32_t(kvh * HD * 2u);
                        TC5H_TRACE(24);
                        if (gi >= 2u && !mbar_wait(bar(16u + b), ((gi >> 1) & 1u) ^ 1u)) { ok = false; break; }
                        mbar_expect_tx(bar(12u + b), TILE);
                        tma_load_2d(k_sm + b * TILE, &tm_k, x, t0, bar(12u + b));
                        tma_load_2d(k_sm + b * TILE + SLAB, &tm_k, x + 128, t0, bar(12u + b));
                        TC5H_TRACE(25);
                        if (gi >= 2u && !mbar_wait(bar(18u + b), ((gi >> 1) & 1u) ^ 1u)) { ok = false; break; }
                        mbar_expect_tx(bar(14u + b), TILE);
                        tma_load_2d(v_sm + b * TILE, &tm_v, x, t0, bar(14u + b));
                        tma_load_2d(v_sm + b * TILE + SLAB, &tm_v, x + 128, t0, bar(14u + b));
                        TC5H_TRACE(26);
                    }
                }
            } else
            for (uint32_t it = 0; it < n_tiles && ok; ++it) {
                const uint32_t gi = gt + it, b = gi & 1u, t0 = c_lo + it * BN;
                if (pt == 0) TC5H_TRACE(24);
                move(kg, t0, k_sm + b * TILE, bar(16u + b), gi);
                if (pt == 0) TC5H_TRACE(25);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(bar(12u + b));
                move(vg, t0, v_sm + b * TILE, bar(18u + b), gi);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(bar(14u + b));
                if (pt == 0) TC5H_TRACE(26);
            }
            if (!ok) *abort_flag = 1u;
        }
        // end of the segment: every product of it is complete (the softmax threads waited for the last
        // P V before they read O), so Q, the tensor memory and the barriers' phases can be taken over
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (tid == 0) TC5H_STAMP(29);
        if (mode == 3u && tid == 0 && blockIdx.x != p.fail_cta) {
            // the piece is in scratch (every thread's stores are ordered before the barrier above)
            __threadfence();
            asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(p.flags + blockIdx.x), "r"(s_abort != 0u ? 0u : p.epoch) : "memory");
        }
        if (s_abort != 0u || p.n_cta == 0u) break;
        gt += n_tiles;
        cur += n_tiles;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (s_abort != 0u && tid == 0) atomicOr(p.status, 1u);
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "n"(TMEM_COLS) : "memory");
    }
}



// Items that the even spread cut into pieces: combine the pieces' O, reference maxima and sums
// (the split-merge of flash_attn_reduce.comp, per row).  grid = (n_cta - 1 share boundaries, 16
// sixteenths of the 256 rows): the block of the first boundary inside an item merges it; a warp
// per row, a lane per four output dims.
__global__ void __launch_bounds__(256) prefill_tc5_merge_kernel(const Tc5Params p)
{
    __shared__ uint32_t s_tj[kMaxRowBlocks];
    for (uint32_t rb = threadIdx.x; rb < p.n_rb; rb += 256u) {
        uint32_t r0, cl, tj;
        item_extent(p, rb, &r0, &cl, &tj);
        s_tj[rb] = tj;
    }
    __syncthreads();
    asm volatile("griddepcontrol.wait;" ::: "memory");     // launched ahead of the end of the attention kernel
    const uint64_t T = p.total_tiles, n = p.n_cta;
    const uint32_t cut = uint32_t(uint64_t(blockIdx.x + 1u) * T / n);      // first tile of CTA blockIdx.x + 1
    uint32_t acc = 0u, rb = 0u, tj = 0u;
    for (; rb < p.n_rb; ++rb) {
        tj = s_tj[rb];
        if (cut < acc + tj * p.n_kv_heads) break;
        acc += tj * p.n_kv_heads;
    }
    if (rb == p.n_rb) return;
    const uint32_t kvh = (cut - acc) / tj;
    const uint32_t s = acc + kvh * tj, e = s + tj;
    if (cut == s) return;                                                   // the share ends where the item does
    const uint32_t c_first = uint32_t((uint64_t(s + 1u) * n - 1u) / T), c_last = uint32_t((uint64_t(e) * n - 1u) / T);
    if (c_first != blockIdx.x) return;                                      // an earlier boundary lies inside this item too
    const uint32_t g = p.group, n_rows = p.m * g, row0 = (p.n_rb - 1u - rb) * uint32_t(CTA_ROWS);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    constexpr uint64_t PIECE = uint64_t(CTA_ROWS) * (HD + 2);
    for (uint32_t rl = blockIdx.y * 16u + warp; rl < blockIdx.y * 16u + 16u; rl += 8u) {
        const uint32_t r = row0 + rl;
        if (r >= n_rows) break;
        // the pieces' reference maxima and sums a lane each (an item cut into many pieces would
        // otherwise pay one round trip a piece, twice), 32 pieces a pass
        const uint32_t np = c_last - c_first + 1u;
        auto piece_of = [&](uint32_t i) {
            const uint32_t c = c_first + i;
            const uint32_t slot = uint32_t(uint64_t(c) * T / n) >= s ? 0u : 1u;
            return p.scratch + (uint64_t(c) * 2u + slot) * PIECE;
        };
        float mx = kMaskedScore;
        for (uint32_t i = lane; i < np; i += 32u) mx = fmaxf(mx, piece_of(i)[CTA_ROWS * HD + rl]);
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
        float l = 0.f;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t i0 = 0u; i0 < np; i0 += 32u) {
            float w_mine = 0.f;
            if (i0 + lane < np) {
                const float *pc = piece_of(i0 + lane);
                w_mine = fast_exp2(pc[CTA_ROWS * HD + rl] - mx);
                l += w_mine * pc[CTA_ROWS * HD + CTA_ROWS + rl];
            }
            const uint32_t cnt = min(32u, np - i0);
#pragma unroll 4
            for (uint32_t i = 0u; i < cnt; ++i) {
                const float w = __shfl_sync(0xffffffffu, w_mine, int(i));
                const float4 x = *reinterpret_cast<const float4 *>(piece_of(i0 + i) + rl * HD + 4u * lane);
                o.x += w * x.x; o.y += w * x.y; o.z += w * x.z; o.w += w * x.w;
            }
        }
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) l += __shfl_xor_sync(0xffffffffu, l, d);
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        float *out = p.out + (uint64_t(r / g) * p.n_q_heads + kvh * g + r % g) * HD + 4u * lane;
        *reinterpret_cast<float4 *>(out) = make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv);
    }
}

// Whether the even shares are allowed for this call and expected to pay; the sum of all items'
// tiles and the longest item on the way.  p.n_rb is set.
bool spread_pays(const vfkv_ctx *ctx, const Tc5Params &p, uint64_t *total_out, uint32_t *tj_max_out)
{
    if (!(ctx->tune_stages == 0 || ctx->tune_stages == 3) || ctx->tune_warps == 4 || p.n_rb > kMaxRowBlocks ||
        p.kv_start >= std::min(p.q_start + 1u, p.n_kv))
        return false;
    const uint32_t n_sm = uint32_t(ctx->sm_count);
    const uint64_t items = uint64_t(p.n_rb) * p.n_kv_heads;
    uint64_t total = 0;
    uint32_t tj_max = 0;
    for (uint32_t rb = 0; rb < p.n_rb; ++rb) {
        uint32_t r0, cl, tj;
        item_extent(p, rb, &r0, &cl, &tj);
        total += uint64_t(tj) * p.n_kv_heads;
        tj_max = std::max(tj_max, tj);
    }
    *total_out = total;
    *tj_max_out = tj_max;
    const uint64_t waves = (items + n_sm - 1) / n_sm;
    // Items for at most half the SMs: shares of two tiles or more, if they shorten the longest CTA
    // by ten tiles (29 us) -- the shares' segments, the pieces and the merge kernel cost about half of
    // that (512 queries at 1024, 64 items of 12 tiles: 46 us one CTA an item, 56 us in shares of 5;
    // 256 queries at 2048, 32 items of 18: 63 against 54; 256 at 8192, 32 of 66: 193 against 85).
    const bool few = items * 2 <= n_sm && uint64_t(tj_max) >= total / n_sm + 10;
    const bool worth = ctx->tune_warps == 8 || few || (items * 20 < waves * n_sm * 19 && total >= items * 96);
    return worth && n_sm >= 2 && total >= uint64_t(n_sm) * (few ? 2 : 8) && total < (1ull << 31);
}

}  // namespace

bool prefill_tc5_supported(uint32_t dtype, uint32_t head_dim, uint32_t group, bool has_scales)
{
    return (dtype == VFKV_F8 || dtype == VFKV_F16) && head_dim == 128 && !has_scales && group != 0 && BM % group == 0;
}

bool prefill_tc5_pays(const vfkv_ctx *ctx, uint32_t n_q_heads, uint32_t n_kv_heads, uint32_t m, uint32_t q_start,
                      uint32_t n_kv, uint32_t kv_start, uint32_t window)
{
    Tc5Params p{};
    p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.group = n_q_heads / n_kv_heads;
    p.m = m; p.q_start = q_start; p.n_kv = n_kv; p.kv_start = kv_start; p.window = window;
    p.n_rb = (m * p.group + CTA_ROWS - 1) / CTA_ROWS;
    // 256-row blocks that fill most of the GPU
    if (uint64_t(p.n_rb) * n_kv_heads * 4 >= uint64_t(ctx->sm_count) * 3) return true;
    uint64_t total = 0;
    uint32_t tj_max = 0;
    if (p.n_rb > kMaxRowBlocks) return false;
    if (spread_pays(ctx, p, &total, &tj_max)) return true;
    // Fewer blocks, one CTA each: a CTA pays about 12 us once and 2.9 us per 128 positions, the
    // 64-row mma.sync kernel (four times the CTAs) 2.15 us per 64 positions -- measured on 64
    // queries at 4096: 103 against 140 us, on 128 at 2048: 60 against 76 -- so from ten K/V tiles on
    // the tcgen05 kernel is ahead even on a few SMs.
    tj_max = 0;
    for (uint32_t rb = 0; rb < p.n_rb; ++rb) {
        uint32_t r0, cl, tj;
        item_extent(p, rb, &r0, &cl, &tj);
        tj_max = std::max(tj_max, tj);
    }
    return tj_max >= 10;
}

int32_t launch_prefill_tc5(vfkv_ctx *ctx, uint32_t dtype, const uint8_t *k, const uint8_t *v, const float *q, float *out,
                           uint64_t row_bytes, uint32_t n_q_heads, uint32_t n_kv_heads, uint32_t m, uint32_t q_start,
                           uint32_t n_kv, uint32_t kv_start, uint32_t window, float scale, float softcap,
                           cudaStream_t st)
{
    Tc5Params p{};
    p.k = k; p.v = v; p.q = q; p.out = out; p.row_bytes = row_bytes;
    p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.group = n_q_heads / n_kv_heads;
    p.m = m; p.q_start = q_start; p.n_kv = n_kv; p.kv_start = kv_start; p.window = window;
    p.scale = scale; p.softcap = softcap; p.status = ctx->d_status;
    p.trace = ctx->d_trace;
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        const void *kernels[4] = {reinterpret_cast<const void *>(prefill_tc5_kernel<VFKV_F8, false>),
                                  reinterpret_cast<const void *>(prefill_tc5_kernel<VFKV_F8, true>),
                                  reinterpret_cast<const void *>(prefill_tc5_kernel<VFKV_F16, false>),
                                  reinterpret_cast<const void *>(prefill_tc5_kernel<VFKV_F16, true>)};
        for (const void *kn : kernels) {
            cudaError_t e = cudaFuncSetAttribute(kn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
            if (e != cudaSuccess) return check_cuda(ctx, e, "cudaFuncSetAttribute(tcgen05 prefill attention)");
        }
        configured[ctx->device & 63] = true;
    }
    const dim3 grid((m * p.group + CTA_ROWS - 1) / CTA_ROWS, n_kv_heads);
    const bool cap = softcap > 0.f;
    // One CTA per (kv-head, row block) item leaves the last wave part empty (256 items on 148 SMs:
    // the time of two items for 1.73 items' worth of SM time) and, with few items, most SMs (a chunk
    // of 64 queries x 8 kv-heads is 8 items, however long the context).  When that loses more than
    // a twentieth and the items are long, the specialised form runs one CTA per SM, each taking an
    // even share of all K/V tiles; the pieces of items cut by the shares are put together by the
    // CTA that holds the item's head (up to four pieces an item) or by prefill_tc5_merge_kernel.
    // Needs every query to see at least one position, 39 MB of scratch that the context allocates
    // at the first such call (not inside a stream capture), and tuning 0x0 or 8x3; 4x3 keeps one
    // CTA per item.  Measured: 2048 queries at 14 336 (256 items of ~120 tiles) 706 -> 658 us;
    // 256 queries at 60 000 (32 items) 1356 -> 332 us; 4096 queries at 4096 (512 items of ~48
    // tiles) 579 -> 584 us, hence the floor of 96 tiles an item.
    p.n_rb = grid.x;
    const uint32_t n_sm = uint32_t(ctx->sm_count);
    const uint64_t items = uint64_t(p.n_rb) * n_kv_heads;
    bool spread = false;
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    {
        uint64_t total = 0;
        uint32_t tj_max = 0;
        if (spread_pays(ctx, p, &total, &tj_max)) {
            cudaStreamIsCapturing(st, &capturing);
            if (ctx->d_prefill_scratch == nullptr && capturing == cudaStreamCaptureStatusNone) {
                const size_t bytes = size_t(n_sm) * 2 * CTA_ROWS * (HD + 2) * sizeof(float);
                void *d = nullptr;
                // the pieces, then one flag per CTA
                if (cudaMalloc(&d, bytes + n_sm * sizeof(uint32_t)) == cudaSuccess &&
                    cudaMemset(static_cast<uint8_t *>(d) + bytes, 0, n_sm * sizeof(uint32_t)) == cudaSuccess) {
                    ctx->d_prefill_scratch = static_cast<float *>(d);
                    ctx->prefill_scratch_ctas = n_sm;
                } else {
                    (void)cudaGetLastError();      // no room: one CTA per item
                }
            }
            if (ctx->d_prefill_scratch != nullptr && ctx->prefill_scratch_ctas >= n_sm) {
                spread = true;
                p.total_tiles = uint32_t(total);
                p.n_cta = n_sm;
                p.scratch = ctx->d_prefill_scratch;
                p.flags = reinterpret_cast<uint32_t *>(p.scratch + size_t(n_sm) * 2 * CTA_ROWS * (HD + 2));
                // An item is cut into at most ceil(longest item / smallest share) + 1 pieces.  A
                // captured launch would replay with the flag value of the capture, which the flags
                // still hold from the replay before: those go through the merge kernel.
                const uint64_t share = total / n_sm;
                p.inline_merge = ((tj_max + share - 1) / share <= 3 && capturing == cudaStreamCaptureStatusNone) ? 1u : 0u;
            }
        }
    }
    // The specialised form (roles on separate warps) is the default; vfkv_ctx_set_attn_tuning(ctx, 4, 2)
    // keeps the pipelined form, (4, 1) the simple one.  F16 rows are twice the bytes of FP8 codes and
    // three warps of plain loads do not bring them in fast enough (441-516 against 532-558 TFLOP/s
    // for the pipelined form), so for F16 caches the tiles come by TMA (776-836); without the
    // driver entry point for tensor maps they stay on the pipelined form -- unless the items are so
    // few that one CTA an item would leave half the SMs idle.
    const bool f16_h = dtype == VFKV_F16 && (ctx->encode_tiled != nullptr || (spread && items * 2 <= n_sm));
    if ((ctx->tune_stages == 0 && (dtype == VFKV_F8 || f16_h)) || ctx->tune_stages == 3) {
        static bool configured_h[64] = {};
        if (!configured_h[ctx->device & 63]) {
            const void *kernels[4] = {reinterpret_cast<const void *>(prefill_tc5h_kernel<VFKV_F8, false>),
                                      reinterpret_cast<const void *>(prefill_tc5h_kernel<VFKV_F8, true>),
                                      reinterpret_cast<const void *>(prefill_tc5h_kernel<VFKV_F16, false>),
                                      reinterpret_cast<const void *>(prefill_tc5h_kernel<VFKV_F16, true>)};
            for (const void *kn : kernels) {
                cudaError_t e = cudaFuncSetAttribute(kn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
                if (e != cudaSuccess) return check_cuda(ctx, e, "cudaFuncSetAttribute(tcgen05 prefill attention)");
            }
            configured_h[ctx->device & 63] = true;
        }
        const dim3 grid_h = spread ? dim3(n_sm, 1, 1) : dim3(grid.y, grid.x);
        // F16 rows by TMA: byte-typed maps of the slot's rows [0, n_kv), one row = one position
        CUtensorMap tm_k, tm_v;
        memset(&tm_k, 0, sizeof tm_k);
        memset(&tm_v, 0, sizeof tm_v);
        if (dtype == VFKV_F16 && ctx->encode_tiled != nullptr && n_kv != 0u) {
            typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                              const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
            cuuint64_t dims[2] = {row_bytes, n_kv};
            cuuint64_t strides[1] = {row_bytes};
            cuuint32_t box[2] = {128, 128};
            cuuint32_t estr[2] = {1, 1};
            auto enc = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled);
            const bool made =
                enc(&tm_k, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(k), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS &&
                enc(&tm_v, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(v), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
            p.use_tma = made ? 1u : 0u;
        }
        void (*kern)(const Tc5Params, const CUtensorMap, const CUtensorMap) = dtype == VFKV_F8 ? (cap ? prefill_tc5h_kernel<VFKV_F8, true> : prefill_tc5h_kernel<VFKV_F8, false>)
                                                         : (cap ? prefill_tc5h_kernel<VFKV_F16, true> : prefill_tc5h_kernel<VFKV_F16, false>);
        if (spread && p.inline_merge != 0u) {
            // CTAs of this launch wait for one another's pieces: a cooperative launch, which the
            // driver accepts only if the whole grid is resident at once
            if (++ctx->prefill_epoch == 0u) ++ctx->prefill_epoch;
            p.epoch = ctx->prefill_epoch;
            p.wait_ns = ctx->merge_wait_ns;
            p.fail_cta = ctx->debug_fail_split;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = grid_h;
            cfg.blockDim = dim3(384);
            cfg.dynamicSmemBytes = kSmemBytes;
            cfg.stream = st;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeCooperative;
            attr[0].val.cooperative = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            if (cudaLaunchKernelEx(&cfg, kern, p, tm_k, tm_v) == cudaSuccess) {
                ctx->launches++;
                return check_cuda(ctx, cudaGetLastError(), "tcgen05 prefill attention launch");
            }
            (void)cudaGetLastError();          // not all resident: the pieces go to the merge kernel instead
            p.inline_merge = 0u;
        }
        kern<<<grid_h, 384, kSmemBytes, st>>>(p, tm_k, tm_v);
        ctx->launches++;
        if (spread) {
            // launched as a programmatic dependent: it is resident, its table built, when the last CTA
            // of the attention kernel ends
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(p.n_cta - 1, 16);
            cfg.blockDim = dim3(256);
            cfg.stream = st;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            cudaError_t e = cudaLaunchKernelEx(&cfg, prefill_tc5_merge_kernel, p);
            if (e != cudaSuccess) return check_cuda(ctx, e, "tcgen05 prefill merge launch");
            ctx->launches++;
        }
        return check_cuda(ctx, cudaGetLastError(), "tcgen05 prefill attention launch");
    }
    if (ctx->tune_stages != 1) {          // the pipelined form; vfkv_ctx_set_attn_tuning(ctx, 4, 1) keeps the simple one
        static bool configured_p[64] = {};
        if (!configured_p[ctx->device & 63]) {
            const void *kernels[4] = {reinterpret_cast<const void *>(prefill_tc5p_kernel<VFKV_F8, false>),
                                      reinterpret_cast<const void *>(prefill_tc5p_kernel<VFKV_F8, true>),
                                      reinterpret_cast<const void *>(prefill_tc5p_kernel<VFKV_F16, false>),
                                      reinterpret_cast<const void *>(prefill_tc5p_kernel<VFKV_F16, true>)};
            for (const void *kn : kernels) {
                cudaError_t e = cudaFuncSetAttribute(kn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
                if (e != cudaSuccess) return check_cuda(ctx, e, "cudaFuncSetAttribute(tcgen05 prefill attention)");
            }
            configured_p[ctx->device & 63] = true;
        }
        if (dtype == VFKV_F8) {
            if (cap) prefill_tc5p_kernel<VFKV_F8, true><<<grid, 256, kSmemBytes, st>>>(p);
            else prefill_tc5p_kernel<VFKV_F8, false><<<grid, 256, kSmemBytes, st>>>(p);
        } else {
            if (cap) prefill_tc5p_kernel<VFKV_F16, true><<<grid, 256, kSmemBytes, st>>>(p);
            else prefill_tc5p_kernel<VFKV_F16, false><<<grid, 256, kSmemBytes, st>>>(p);
        }
        ctx->launches++;
        return check_cuda(ctx, cudaGetLastError(), "tcgen05 prefill attention launch");
    }
    if (dtype == VFKV_F8) {
        if (cap) prefill_tc5_kernel<VFKV_F8, true><<<grid, 256, kSmemBytes, st>>>(p);
        else prefill_tc5_kernel<VFKV_F8, false><<<grid, 256, kSmemBytes, st>>>(p);
    } else {
        if (cap) prefill_tc5_kernel<VFKV_F16, true><<<grid, 256, kSmemBytes, st>>>(p);
        else prefill_tc5_kernel<VFKV_F16, false><<<grid, 256, kSmemBytes, st>>>(p);
    }
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "tcgen05 prefill attention launch");
}

}  // namespace vfkv
