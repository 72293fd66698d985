// Split-K GQA decode attention for FP8 (E4M3) and F16 caches: TMA-fed, tensor-core
// products, fused log-sum-exp merge.
//
// Replaces vk_shaders/flash_attn_split.comp + flash_attn_reduce.comp (and
// flash_attn.comp for short sequences) for the shapes it covers; the CUDA-core
// kernel in attn_generic.cu covers the rest.  Same math as the shaders
// (score = scale * q.k, masked lanes excluded, p = exp(score - max), running
// (max, sum, acc) merge of partials), different organisation:
//
//   CTA  = (split, kv-head, sequence); the q-heads that share the kv-head are
//          the M rows of the tensor-core tile, so K and V stream through once
//          per kv-head (the shader streams them once per q-head).
//   warp = owns a private ring of TMA stages.  Lane 0 issues
//          cp.async.bulk.tensor.2d boxes of [TP positions x 128 bytes]
//          (128-byte swizzle) for K and V and the warp waits on its own
//          mbarrier; there is no CTA-wide synchronisation while streaming.
//   FP8  : the E4M3 codes go from shared memory to registers (ldmatrix for K, ld.shared + prmt
//          pairing for V) and are widened there to half precision (cvt.rn.f16x2.e4m3x2, exact):
//          the FP8 -> F16 cache read fused into the load.  The products run on
//          mma.sync.m16n8k16.f16.  (mma.sync with e4m3 operands measured slower here: each one
//          costs a dozen conversion instructions on the ALU pipe on top of two f16 MMAs.)
//   F16  : mma.sync.m16n8k16.f16 with ldmatrix / ldmatrix.trans.
//   both : with up to 8 q-heads per kv-head the M tile has rows to spare, so Q and P are each
//          split into a high and a low half-precision term (rows 0-7 / 8-15) and the result
//          carries f32-grade operand precision.
//   few  : with at most 4 q-heads per kv-head the products are transposed (S^T = K Q^T,
//          O^T = V^T P^T): positions and output dims on the M side, the heads' high and low
//          terms on the 8 columns, P^T moved from accumulator to operand layout by movmatrix.
//          Half the MMAs per tile (the legacy tensor path bounds the stream of a small grid)
//          and two thirds of the registers.
//   tail : warp partials merge in shared memory; the last CTAs of a
//          (sequence, kv-head) to finish merge the split partials with the
//          reduce shader's update (flash_attn_reduce.comp:51-80), so there is no
//          second launch.
//
// Every mbarrier wait is bounded: on expiry the kernel raises bit 0 of the
// context's status word and returns without touching the output.
#include <cuda.h>

#include <atomic>

#include "attn_params.cuh"
#include "fp8_codec.cuh"

namespace vfkv {

namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
// P goes into the tensor cores as half-precision terms.  With tens of thousands of positions most
// p = 2^(x - m) lie below the smallest normal half (6.1e-5), where the terms keep few or no bits
// (measured: 6.5e-5 absolute error at 40 000 positions).  So P is fed as p * 2^14 (still at most
// 16 384) and the accumulators are scaled back when the warp's partial is written; both scalings
// are exact, and l is summed from the unscaled p.
constexpr float kPScale = 16384.0f, kInvPScale = 1.0f / 16384.0f;

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Waits at most about one second; false means the data never arrived.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity)
{
    if (mbar_try_wait(bar, parity)) return true;
    // the timer is slow to read: it is looked at only after a few hundred misses
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 255u) {
            if (t0 == 0) t0 = global_timer_ns();
            else if (global_timer_ns() - t0 > 1000000000ull) return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int32_t x, int32_t y,
                                            uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ ulonglong2 lds_u64x2(uint32_t addr)
{
    ulonglong2 w;
    asm("ld.shared.v2.u64 {%0, %1}, [%2];" : "=l"(w.x), "=l"(w.y) : "r"(addr) : "memory");
    return w;
}
// The shared-memory loads take a register base plus a compile-time byte offset, so that the
// per-lane swizzled part of an address is computed once per tile and the rest is an immediate.
template <int IMM>
__device__ __forceinline__ void ldmatrix_x4(uint32_t base, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4+%5];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(base), "n"(IMM));
}
template <int IMM>
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t base, uint32_t &r0, uint32_t &r1, uint32_t &r2,
                                                  uint32_t &r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4+%5];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(base), "n"(IMM));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
template <int IMM> __device__ __forceinline__ uint32_t lds32(uint32_t base)
{
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1+%2];" : "=r"(v) : "r"(base), "n"(IMM));
    return v;
}
__device__ __forceinline__ float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two values -> (hi, lo) half2 pairs with hi + lo == value to about 2^-22.
__device__ __forceinline__ void split_f16x2(float x0, float x1, uint32_t &hi, uint32_t &lo)
{
    __half2 h = __floats2half2_rn(x0, x1);
    float2 hf = __half22float2(h);
    hi = *reinterpret_cast<uint32_t *>(&h);
    lo = f32x2_to_f16x2(x0 - hf.x, x1 - hf.y);
}

struct MmaParams {
    AttnParams a;
    // Split merge (n_splits > 1): 256 64-bit ticket words per (sequence, kv-head), one per split count,
    // and the partials as tagged 8-byte words (see vfkv_workspace).
    unsigned long long *tickets;
    uint64_t *tag_part;
    uint64_t merge_wait_ns;       // limit of the merging CTA's wait for the other splits' partials
    uint32_t launch_seq;          // host-side count of split launches on this workspace (part of the tag)
    uint32_t n_mergers;           // CTAs per (sequence, kv-head) that share the merge of its splits
    const float *k_new, *v_new;   // [seq][kv_head][dim] f32 token to append at position len-1, or null
    unsigned long long *trace;    // null, or 16 timestamps (ns) per CTA written by thread 0 (this launch's block of the buffer)
    uint32_t pdl;                 // 0 plain launch, 1 dependent launch, 2 dependent launch with early K/V prefetch
    uint32_t cluster;             // 1: the splits of a (sequence, kv-head) are one thread-block cluster
    uint32_t fan_merge;           // with a.fan: also wait for the other ranks' blocks and write the final rows
    uint32_t fail_split;          // test hook: this split of (sequence 0, kv-head 0) acts as if a TMA wait ran out
    uint32_t per_recip;           // ceil(2^32 / output pairs per merging CTA): idx / per == umulhi(idx, per_recip) for idx < 65536
    uint64_t tag_words;           // host side only: size of tag_part in words
};

// Phase timestamps for latency analysis; costs one predicated branch when tracing is off.
#define VFKV_TRACE(i)                                                                               \
    do {                                                                                            \
        if (mp.trace != nullptr && threadIdx.x == 0)                                                \
            mp.trace[((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 16 + (i)] = global_timer_ns(); \
    } while (0)

// Shape-dependent constants.
template <int DT, int D, int W, int NS> struct Shape {
    static constexpr int ES = DT == VFKV_F8 ? 1 : 2;
    static constexpr int TP = DT == VFKV_F8 ? 32 : 16;        // positions per tile
    static constexpr int NB = TP / 8;                         // 8-position blocks per tile
    static constexpr int NC = D * ES / 128;                   // 128-byte column chunks per head slice
    static constexpr int KSTEPS = D * ES / 32;                // 32 bytes of the head slice per QK step
    static constexpr int NDB = D / 8;                         // 8-dim blocks of the output
    static constexpr int TILE_BYTES = TP * 128 * NC;          // K (or V) tile
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    static constexpr int RING_BYTES = W * NS * STAGE_BYTES;
    static constexpr int SMEM_BYTES = RING_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// Byte address of 16-byte unit `unit` of row `row` in chunk `chunk` of a tile (128-byte swizzle:
// the unit index is XORed with the row's low three bits; tiles are 1024-byte aligned).
template <int TP>
__device__ __forceinline__ uint32_t tile_addr(uint32_t tile, uint32_t chunk, uint32_t row, uint32_t unit)
{
    return tile + chunk * (TP * 128) + row * 128 + ((unit ^ (row & 7u)) << 4);
}

// ---- unrolled tile steps; the recursion only exists to make the shared-memory offsets immediates ----

// Four E4M3 codes -> two half2: bytes 0,1 and bytes 2,3 (exact).
__device__ __forceinline__ void e4m3x4_to_half2x2(uint32_t w, uint32_t &lo, uint32_t &hi)
{
    asm("{\n\t.reg .b16 a, b;\n\t"
        "mov.b32 {a, b}, %2;\n\t"
        "cvt.rn.f16x2.e4m3x2 %0, a;\n\t"
        "cvt.rn.f16x2.e4m3x2 %1, b;\n\t}"
        : "=r"(lo), "=r"(hi)
        : "r"(w));
}

// S += Q K^T for one 32-byte step of the head slice: N blocks JP*2 and JP*2+1 (16 positions).
// F16 cache: 32 bytes = 16 dims = one MMA, a = its A fragment, a2 unused.
// FP8 cache: 32 bytes = 32 dims = two MMAs (a, a2).  ldmatrix hands each thread four consecutive
// codes of its position; they are widened to half precision in registers (the cache read's
// FP8 -> F16 step, kv_fp8_to_f16.comp, fused into the load) and fed as k slots {2tig, 2tig+1} and
// {8+2tig, 9+2tig}, the order the Q fragments were built in.
template <bool FP8, int NB, int IMM, int JP = 0>
__device__ __forceinline__ void qk_blocks(uint32_t base, const uint32_t (&a)[4], const uint32_t (&a2)[4],
                                          float (&sc)[NB][4])
{
    if constexpr (JP < NB / 2) {
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4<IMM + JP * 16 * 128>(base, r0, r1, r2, r3);
        if constexpr (FP8) {
            uint32_t b0, b1;
            e4m3x4_to_half2x2(r0, b0, b1); mma_f16(sc[2 * JP], a, b0, b1);
            e4m3x4_to_half2x2(r1, b0, b1); mma_f16(sc[2 * JP], a2, b0, b1);
            e4m3x4_to_half2x2(r2, b0, b1); mma_f16(sc[2 * JP + 1], a, b0, b1);
            e4m3x4_to_half2x2(r3, b0, b1); mma_f16(sc[2 * JP + 1], a2, b0, b1);
        } else {
            mma_f16(sc[2 * JP], a, r0, r1);
            mma_f16(sc[2 * JP + 1], a, r2, r3);
        }
        qk_blocks<FP8, NB, IMM, JP + 1>(base, a, a2, sc);
    }
}
// kb[u] = K tile base + this lane's swizzled offset for units 2u, 2u+1
template <bool FP8, int TP, int NB, int KSTEPS, int QSTEPS, int KS = 0>
__device__ __forceinline__ void qk_steps(const uint32_t (&kb)[4], const uint32_t (&qa)[QSTEPS][4], float (&sc)[NB][4])
{
    if constexpr (KS < KSTEPS) {
        if constexpr (FP8) qk_blocks<FP8, NB, (KS / 4) * TP * 128>(kb[KS % 4], qa[2 * KS], qa[2 * KS + 1], sc);
        else qk_blocks<FP8, NB, (KS / 4) * TP * 128>(kb[KS % 4], qa[KS], qa[KS], sc);
        qk_steps<FP8, TP, NB, KSTEPS, QSTEPS, KS + 1>(kb, qa, sc);
    }
}
// FP8 O += P V for dims 32Q .. 32Q+31.  vb[2u + e] = V tile base + this lane's offset for rows of
// parity e and unit pair u.  A word holds dims 32Q + 4*gid + {0..3} of one position; prmt pairs the
// codes of two positions dim by dim, the widening cvt turns each pair into the half2 B fragment of
// one 8-dim output block.  pa[h] is the A fragment of positions 16h .. 16h+15.
template <int TP, int D, int Q = 0>
__device__ __forceinline__ void pv_fp8(const uint32_t (&vb)[8], const uint32_t (&pa)[2][4], float (&acc)[D / 8][4])
{
    if constexpr (Q < D / 32) {
        constexpr int C = (Q / 4) * TP * 128, u = Q % 4;
        const uint32_t be = vb[2 * u], bo = vb[2 * u + 1];
        uint32_t w[8];
        w[0] = lds32<C>(be);             w[1] = lds32<C>(bo);              // positions 2tig, 2tig+1
        w[2] = lds32<C + 8 * 128>(be);   w[3] = lds32<C + 8 * 128>(bo);    // + 8
        w[4] = lds32<C + 16 * 128>(be);  w[5] = lds32<C + 16 * 128>(bo);   // + 16
        w[6] = lds32<C + 24 * 128>(be);  w[7] = lds32<C + 24 * 128>(bo);   // + 24
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t b0[4], b1[4];       // per dim i: (pos, pos+1) and (pos+8, pos+9) as half2
            e4m3x4_to_half2x2(prmt(w[4 * h], w[4 * h + 1], 0x5140), b0[0], b0[1]);
            e4m3x4_to_half2x2(prmt(w[4 * h], w[4 * h + 1], 0x7362), b0[2], b0[3]);
            e4m3x4_to_half2x2(prmt(w[4 * h + 2], w[4 * h + 3], 0x5140), b1[0], b1[1]);
            e4m3x4_to_half2x2(prmt(w[4 * h + 2], w[4 * h + 3], 0x7362), b1[2], b1[3]);
#pragma unroll
            for (int i = 0; i < 4; ++i) mma_f16(acc[4 * Q + i], pa[h], b0[i], b1[i]);
        }
        pv_fp8<TP, D, Q + 1>(vb, pa, acc);
    }
}
// F16 O += P V for the 8-dim blocks NBK and NBK+1 (ldmatrix.trans gives the B fragments directly).
template <int TP, int D, int NBK = 0>
__device__ __forceinline__ void pv_f16(const uint32_t (&vb)[4], const uint32_t (&pa)[4], float (&acc)[D / 8][4])
{
    if constexpr (NBK < D / 8) {
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4_trans<(NBK / 8) * TP * 128>(vb[(NBK % 8) / 2], r0, r1, r2, r3);
        mma_f16(acc[NBK], pa, r0, r1);
        mma_f16(acc[NBK + 1], pa, r2, r3);
        pv_f16<TP, D, NBK + 2>(vb, pa, acc);
    }
}

// ---- transposed products (at most 4 q-heads per kv-head) ------------------------------------------
// With few q-heads the M = 16 rows of an MMA are mostly padding when the heads sit on M.  The
// transposed products put the positions (S^T = K Q^T) and the output dims (O^T = V^T P^T) on M and
// the heads on the N = 8 columns: column 2h carries the high half-precision term of head h, column
// 2h + 1 the low term.  Half the MMAs per tile, and half the accumulator registers.

// 8x8 transpose of 16-bit elements across the warp: row r of the result is column r of the source.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x)
{
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
// p -> half2 {high term, low term}: the two columns of this thread's head
__device__ __forceinline__ uint32_t hi_lo_f16x2(float x)
{
    const __half h = __float2half_rn(x);
    const __half2 v = __halves2half2(h, __float2half_rn(x - __half2float(h)));
    return *reinterpret_cast<const uint32_t *>(&v);
}
// S^T += K Q^T.  ksw[u] = K tile base + this lane's ldmatrix offset for unit pair u of a 128-byte
// chunk (matrices in the order rows 0-7 / 8-15 of unit 2u, then of unit 2u + 1).
// FP8: one ldmatrix covers 16 positions x 32 dims = two MMAs (qb[2J], qb[2J + 1]); the codes are
// widened in registers, k slots {2tig, 2tig+1, 8+2tig, 9+2tig} <-> dims 4tig .. 4tig+3 of the unit.
// F16: one ldmatrix is the A fragment of 16 positions x 16 dims.
template <bool FP8, int TP, int D, int J = 0>
__device__ __forceinline__ void qk_t(const uint32_t (&ksw)[4], const uint32_t (&qb)[D / 16][2], float (&sc)[TP / 16][4])
{
    constexpr int NJ = FP8 ? D / 32 : D / 16;
    if constexpr (J < NJ) {
        constexpr int C = (J / 4) * TP * 128;
        uint32_t r0, r1, r2, r3;
        if constexpr (FP8) {
#pragma unroll
            for (int mb = 0; mb < TP / 16; ++mb) {
                if (mb == 0) ldmatrix_x4<C>(ksw[J % 4], r0, r1, r2, r3);
                else ldmatrix_x4<C + 16 * 128>(ksw[J % 4], r0, r1, r2, r3);
                uint32_t a[4];
                e4m3x4_to_half2x2(r0, a[0], a[2]); e4m3x4_to_half2x2(r1, a[1], a[3]);
                mma_f16(sc[mb], a, qb[2 * J][0], qb[2 * J][1]);
                e4m3x4_to_half2x2(r2, a[0], a[2]); e4m3x4_to_half2x2(r3, a[1], a[3]);
                mma_f16(sc[mb], a, qb[2 * J + 1][0], qb[2 * J + 1][1]);
            }
        } else {
            ldmatrix_x4<C>(ksw[J % 4], r0, r1, r2, r3);
            const uint32_t a[4] = {r0, r1, r2, r3};
            mma_f16(sc[0], a, qb[J][0], qb[J][1]);
        }
        qk_t<FP8, TP, D, J + 1>(ksw, qb, sc);
    }
}
// FP8 O^T += V^T P^T for dims 32Q .. 32Q+31: the same words, byte pairing and widening as pv_fp8; a
// pair of positions of one dim is now an A register.  Row gid of block 2Q + pr is dim
// 32Q + 4gid + 2pr, row gid + 8 is that dim + 1.  pb[h] = P^T fragment of positions 16h .. 16h+15.
template <int TP, int D, int Q = 0>
__device__ __forceinline__ void pv_t_fp8(const uint32_t (&vb)[8], const uint32_t (&pb)[2][2], float (&acc)[D / 16][4])
{
    if constexpr (Q < D / 32) {
        constexpr int C = (Q / 4) * TP * 128, u = Q % 4;
        const uint32_t be = vb[2 * u], bo = vb[2 * u + 1];
        uint32_t w[8];
        w[0] = lds32<C>(be);             w[1] = lds32<C>(bo);
        w[2] = lds32<C + 8 * 128>(be);   w[3] = lds32<C + 8 * 128>(bo);
        w[4] = lds32<C + 16 * 128>(be);  w[5] = lds32<C + 16 * 128>(bo);
        w[6] = lds32<C + 24 * 128>(be);  w[7] = lds32<C + 24 * 128>(bo);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t b0[4], b1[4];       // per dim i: positions (2tig, 2tig+1) and (8+2tig, 9+2tig) of half h
            e4m3x4_to_half2x2(prmt(w[4 * h], w[4 * h + 1], 0x5140), b0[0], b0[1]);
            e4m3x4_to_half2x2(prmt(w[4 * h], w[4 * h + 1], 0x7362), b0[2], b0[3]);
            e4m3x4_to_half2x2(prmt(w[4 * h + 2], w[4 * h + 3], 0x5140), b1[0], b1[1]);
            e4m3x4_to_half2x2(prmt(w[4 * h + 2], w[4 * h + 3], 0x7362), b1[2], b1[3]);
            const uint32_t a0[4] = {b0[0], b0[1], b1[0], b1[1]};
            const uint32_t a1[4] = {b0[2], b0[3], b1[2], b1[3]};
            mma_f16(acc[2 * Q], a0, pb[h][0], pb[h][1]);
            mma_f16(acc[2 * Q + 1], a1, pb[h][0], pb[h][1]);
        }
        pv_t_fp8<TP, D, Q + 1>(vb, pb, acc);
    }
}
// F16 O^T += V^T P^T for dims 16DB .. 16DB+15: ldmatrix.trans hands out the A fragment (matrices in
// the order positions 0-7 of units 2u, 2u+1, then positions 8-15).
template <int TP, int D, int DB = 0>
__device__ __forceinline__ void pv_t_f16(const uint32_t (&vb)[4], const uint32_t (&pb)[2], float (&acc)[D / 16][4])
{
    if constexpr (DB < D / 16) {
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4_trans<(DB / 4) * TP * 128>(vb[DB % 4], r0, r1, r2, r3);
        const uint32_t a[4] = {r0, r1, r2, r3};
        mma_f16(acc[DB], a, pb[0], pb[1]);
        pv_t_f16<TP, D, DB + 1>(vb, pb, acc);
    }
}

// W = warps per CTA, NS = TMA stages per warp.  Grids of several waves run 4 warps x 2 stages, which
// lets three CTAs share an SM (12 warps hide the MMA / shuffle latencies of one another); grids that
// leave SMs idle run 8 warps x 3 stages, spreading a CTA's short stream over more warps.
// CAP compiles the score soft-cap in or out.
// TR selects the transposed products (heads on the N side; the host picks it for groups of at most 4).
template <int DT, int D, bool ROWS2, int W, int NS, bool CAP, bool TR>
__global__ void __launch_bounds__(W * 32, (W == 4 && NS == 2 && Shape<DT, D, W, NS>::STAGE_BYTES <= 8192) ? 3 : 1)
attn_split_mma_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const MmaParams mp)
{
    using S = Shape<DT, D, W, NS>;
    constexpr int kWarps = W;
    constexpr int kStages = NS;
    constexpr int TP = S::TP, NB = S::NB, NC = S::NC, KSTEPS = S::KSTEPS, NDB = S::NDB;
    constexpr bool FP8 = DT == VFKV_F8;
    static_assert(!(TR && ROWS2), "the transposed products hold at most 4 heads");
    constexpr int RS = (!FP8 && ROWS2) ? 2 : 1;          // logical score rows per thread
    constexpr int MB = TP / 16;                          // transposed form: 16-position M blocks per tile
    constexpr int NQB = D / 16;                          // transposed form: 16-dim k steps of Q K^T / M blocks of O^T
    // With at most 8 q-heads per kv-head the M tile has room for a second term: rows 0-7 carry the
    // high part of Q (and of P), rows 8-15 the low part, and their products are summed in f32.
    constexpr bool SPLIT = FP8 || !ROWS2;
    const AttnParams &p = mp.a;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *ring_ptr = smem_raw + (ring - smem_u32(smem_raw));
    const uint32_t bars = ring + S::RING_BYTES;           // kWarps*kStages mbarriers, 8 bytes each
    __shared__ uint32_t s_flag, s_epoch, s_tag, s_merger, s_late;
    __shared__ PeerFanout s_fan;          // the group's fan-out table (position-sharded calls only)

    const uint32_t split = blockIdx.x, kvh = blockIdx.y, s = blockIdx.z;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t gid = lane >> 2, tig = lane & 3;
    const uint32_t g = p.group;

    // Q is fetched first: its address depends on the block index only, so these loads overlap the
    // (dependent) read of the sequence's position and the first TMA round trip.
    // element layout this thread needs: FP8  d = 32ks + 4tig + i  and  32ks + 16 + 4tig + i   (i < 4)
    //                                   F16  d = 16ks + 2tig + i  and  16ks + 8 + 2tig + i    (i < 2)
    // transposed form: this lane's column is head gid / 2 (high term in even, low term in odd
    // columns) and it holds the dims its k slots carry:
    //                                   FP8  d = 16u + 4tig + i                                (i < 4)
    //                                   F16  d = 16u + 2tig + {0, 1}, 16u + 8 + 2tig + {0, 1}
    float qv[TR ? 1 : RS][TR ? 1 : KSTEPS][4], qv2[TR ? 1 : RS][TR ? 1 : KSTEPS][4];
    float qt[TR ? NQB : 1][4];
    // Programmatic dependent launch: this grid lets its successor in the stream begin once every CTA
    // has drawn its ticket (and, in mode 2, has seen its predecessor complete), and itself waits for
    // its predecessor before it touches anything the predecessor may have produced.  mp.pdl == 2 is
    // the caller's promise that the kernel directly before this one writes neither the position /
    // slot arrays nor this layer's cache rows, so the K/V prefetch may start before the wait; Q, the
    // new token and every store come after it.  Because the successor is released only after this
    // grid's own wait, the early prefetch can only ever overlap the direct predecessor.
    // Both instructions do nothing in a launch without the attribute.
    if (mp.pdl != 2u) asm volatile("griddepcontrol.wait;" ::: "memory");
    auto load_q = [&]() {
    if constexpr (TR) {
        const uint32_t hcol = gid >> 1;
        const bool hv = hcol < g;
        const float *qp = p.q + (uint64_t(s) * p.n_q_heads + kvh * g + (hv ? hcol : 0)) * D;
#pragma unroll
        for (int u = 0; u < NQB; ++u) {
            if constexpr (FP8) {
                const float4 a = hv ? *reinterpret_cast<const float4 *>(qp + 16 * u + 4 * tig) : make_float4(0, 0, 0, 0);
                qt[u][0] = a.x; qt[u][1] = a.y; qt[u][2] = a.z; qt[u][3] = a.w;
            } else {
                const float2 a = hv ? *reinterpret_cast<const float2 *>(qp + 16 * u + 2 * tig) : make_float2(0, 0);
                const float2 b = hv ? *reinterpret_cast<const float2 *>(qp + 16 * u + 8 + 2 * tig) : make_float2(0, 0);
                qt[u][0] = a.x; qt[u][1] = a.y; qt[u][2] = b.x; qt[u][3] = b.y;
            }
        }
    } else {
#pragma unroll
    for (int r = 0; r < RS; ++r) {
        const uint32_t hrow = gid + 8 * r;
        const bool hv = hrow < g;
        const float *qp = p.q + (uint64_t(s) * p.n_q_heads + kvh * g + (hv ? hrow : 0)) * D;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            if constexpr (FP8) {
                float4 a = hv ? *reinterpret_cast<const float4 *>(qp + 32 * ks + 4 * tig) : make_float4(0, 0, 0, 0);
                float4 b = hv ? *reinterpret_cast<const float4 *>(qp + 32 * ks + 16 + 4 * tig) : make_float4(0, 0, 0, 0);
                qv[r][ks][0] = a.x; qv[r][ks][1] = a.y; qv[r][ks][2] = a.z; qv[r][ks][3] = a.w;
                qv2[r][ks][0] = b.x; qv2[r][ks][1] = b.y; qv2[r][ks][2] = b.z; qv2[r][ks][3] = b.w;
            } else {
                float2 a = hv ? *reinterpret_cast<const float2 *>(qp + 16 * ks + 2 * tig) : make_float2(0, 0);
                float2 b = hv ? *reinterpret_cast<const float2 *>(qp + 16 * ks + 8 + 2 * tig) : make_float2(0, 0);
                qv[r][ks][0] = a.x; qv[r][ks][1] = a.y; qv[r][ks][2] = 0.f; qv[r][ks][3] = 0.f;
                qv2[r][ks][0] = b.x; qv2[r][ks][1] = b.y; qv2[r][ks][2] = 0.f; qv2[r][ks][3] = 0.f;
            }
        }
    }
    }
    };
    // Exchange number of a position-sharded call: read after the wait (the kernel that closed the
    // previous exchange wrote it), kept in shared memory for the epilogue.  When this kernel also
    // closes the exchange (fan_merge), the CTA that draws the last exchange ticket advances the
    // number at once: every CTA reads the number before it draws (the ticket's operand depends on
    // the value read), so the last drawer knows that all of them hold the old number.
    auto load_epoch = [&]() {
        if (threadIdx.x == 32 && p.fan != nullptr) {
            s_fan = *p.fan;
            const uint32_t e = *reinterpret_cast<const volatile uint32_t *>(s_fan.epoch);
            s_epoch = e;
            if (mp.fan_merge != 0u) {
                uint32_t one;
                asm volatile("sub.u32 %0, %1, %2;" : "=r"(one) : "r"(e + 1u), "r"(e));
                const uint32_t total = gridDim.x * gridDim.y * gridDim.z;
                if (atomicAdd(&s_fan.ctl[1], one) == total - 1u) {
                    s_fan.ctl[1] = 0u;
                    *reinterpret_cast<volatile uint32_t *>(&s_fan.ctl[0]) = e + 1u;
                }
            }
        }
    };
    if (mp.pdl != 2u) { load_q(); load_epoch(); }

    VFKV_TRACE(0);
    uint32_t slot, start, len, begin, end;
    seq_range(p, s, &slot, &start, &len);
    split_range(start, len, p.n_splits, split, 32, &begin, &end);
    const uint32_t n_tiles = (end - begin + TP - 1) / TP;
    VFKV_TRACE(1);

    if (threadIdx.x == 0) {
        for (int i = 0; i < kWarps * kStages; ++i) mbar_init(bars + 8 * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_flag = 0;
        s_late = 0;
    }

    __syncthreads();
    VFKV_TRACE(2);
    if (mp.pdl != 2u) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // ---- this warp's pipeline -------------------------------------------------------------
    const uint32_t my_tiles = n_tiles > warp ? (n_tiles - warp + kWarps - 1) / kWarps : 0;
    const uint32_t stage0 = ring + warp * kStages * S::STAGE_BYTES;
    const uint32_t bar0 = bars + 8 * warp * kStages;
    const int32_t x0 = int32_t(kvh * D * S::ES);
    const int64_t row0 = int64_t(slot) * p.max_seq;
    auto issue = [&](uint32_t n) {     // lane 0 only: fetch this warp's n-th tile into stage n % kStages
        const uint32_t st = n % kStages;
        const uint32_t t0 = begin + (warp + n * kWarps) * TP;
        const uint32_t bar = bar0 + 8 * st;
        const uint32_t kt = stage0 + st * S::STAGE_BYTES, vt = kt + S::TILE_BYTES;
        mbar_expect_tx(bar, S::STAGE_BYTES);
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            tma_load_2d(kt + c * TP * 128, &tm_k, x0 + c * 128, int32_t(row0 + t0), bar);
            tma_load_2d(vt + c * TP * 128, &tm_v, x0 + c * 128, int32_t(row0 + t0), bar);
        }
    };
    if (lane == 0) {
        const uint32_t pre = my_tiles < uint32_t(kStages) ? my_tiles : uint32_t(kStages);
        for (uint32_t n = 0; n < pre; ++n) issue(n);
    }

    if (mp.pdl == 2u) {       // the prefetch is in flight; now wait for the predecessor, then read Q
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        load_q();
        load_epoch();
    }

    // ---- fused append (KvWrite of the decode step): the CTA whose range ends at the sequence's
    // last position quantises this kv-head's slice of the new token, stores it in the cache and
    // patches it into the tile it has just fetched, so the row is used whether or not the TMA
    // read saw the store.  Encoding as in append.cu (kv_store_fp8.comp / kv_copy_fp16.comp).
    constexpr uint32_t UPT = D * S::ES / 16;             // 16-byte units per head slice
    constexpr uint32_t NEWU = (2 * UPT + 31) / 32;       // units per lane, K then V
    const bool has_new = mp.k_new != nullptr && end == len && begin < end;
    const uint32_t new_tile = has_new ? (len - 1 - begin) / TP : 0;
    const bool new_owner = has_new && (new_tile % kWarps) == warp;
    uint4 newu[NEWU];
    if (new_owner) {
#pragma unroll
        for (uint32_t i = 0; i < NEWU; ++i) {
            const uint32_t u = lane + 32 * i;
            newu[i] = make_uint4(0, 0, 0, 0);
            if (u < 2 * UPT) {
                const float *src = (u < UPT ? mp.k_new : mp.v_new) + (uint64_t(s) * p.n_kv_heads + kvh) * D +
                                   (u % UPT) * (16 / S::ES);
                const float4 *s4 = reinterpret_cast<const float4 *>(src);
                if constexpr (FP8) {
                    const float4 a = s4[0], b = s4[1], c = s4[2], d = s4[3];
                    newu[i] = make_uint4(f32x4_to_e4m3x4(a.x, a.y, a.z, a.w), f32x4_to_e4m3x4(b.x, b.y, b.z, b.w),
                                         f32x4_to_e4m3x4(c.x, c.y, c.z, c.w), f32x4_to_e4m3x4(d.x, d.y, d.z, d.w));
                } else {
                    const float4 a = s4[0], b = s4[1];
                    newu[i] = make_uint4(f32x2_to_f16x2(a.x, a.y), f32x2_to_f16x2(a.z, a.w),
                                         f32x2_to_f16x2(b.x, b.y), f32x2_to_f16x2(b.z, b.w));
                }
                uint8_t *dst = const_cast<uint8_t *>(u < UPT ? p.k : p.v) + uint64_t(slot) * p.slot_stride_bytes +
                               uint64_t(len - 1) * p.n_kv_heads * D * S::ES + uint64_t(kvh) * D * S::ES + (u % UPT) * 16;
                *reinterpret_cast<uint4 *>(dst) = newu[i];
            }
        }
    }

    // ---- Q fragments (A operand), scaled per head by a power of two into [128, 256) --------
    // FP8: rows 0-7 of the M tile hold the high E4M3 term of heads 0-7, rows 8-15 the low term.
    // F16: rows are heads 0-15.
    constexpr int QSTEPS = D / 16;       // one A fragment per 16 dims
    uint32_t qa[TR ? 1 : QSTEPS][4];
    uint32_t qb[TR ? NQB : 1][2];        // transposed form: B fragments of this lane's column
    float mult[RS];                      // score multiplier per logical row: scale / q_scale
    if constexpr (TR) {
        float amax = 0.f;
#pragma unroll
        for (int u = 0; u < NQB; ++u)
#pragma unroll
            for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fabsf(qt[u][i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        int e = int((__float_as_uint(amax) >> 23) & 0xFF) - 127;
        e = amax > 0.f ? max(-100, min(100, e)) : 7;
        const float qs = __uint_as_float(uint32_t(7 - e + 127) << 23);
        const float inv_qs = __uint_as_float(uint32_t(e - 7 + 127) << 23);
        const bool low = (gid & 1u) != 0u;
#pragma unroll
        for (int u = 0; u < NQB; ++u) {
            uint32_t h0, l0, h1, l1;
            split_f16x2(qt[u][0] * qs, qt[u][1] * qs, h0, l0);
            split_f16x2(qt[u][2] * qs, qt[u][3] * qs, h1, l1);
            qb[u][0] = low ? l0 : h0;
            qb[u][1] = low ? l1 : h1;
        }
        // the scores this lane will hold belong to head tig: fetch that head's multiplier from a
        // lane whose column is one of its two
        mult[0] = __shfl_sync(0xffffffffu, p.scale * inv_qs * (CAP ? 1.0f : kLog2e), (2u * tig) << 2);
    } else {
#pragma unroll
        for (int r = 0; r < RS; ++r) {
            float amax = 0.f;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks)
#pragma unroll
                for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fmaxf(fabsf(qv[r][ks][i]), fabsf(qv2[r][ks][i])));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            // q_scale = 2^(7 - floor(log2 amax)); exact in both directions
            int e = int((__float_as_uint(amax) >> 23) & 0xFF) - 127;
            e = amax > 0.f ? max(-100, min(100, e)) : 7;
            const float qs = __uint_as_float(uint32_t(7 - e + 127) << 23);
            const float inv_qs = __uint_as_float(uint32_t(e - 7 + 127) << 23);
            mult[r] = p.scale * inv_qs * (CAP ? 1.0f : kLog2e);
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                if constexpr (FP8) {
                    // 16-dim block 2ks holds dims 32ks + 4tig + {0..3} of this thread, block 2ks+1 the
                    // same + 16.  Within a block the MMA's k slots {2tig, 2tig+1} are dims 4tig + {0, 1}
                    // and slots {8+2tig, 9+2tig} are dims 4tig + {2, 3}: the order in which the bytes of
                    // a K row arrive from ldmatrix.
                    split_f16x2(qv[r][ks][0] * qs, qv[r][ks][1] * qs, qa[2 * ks][0], qa[2 * ks][1]);
                    split_f16x2(qv[r][ks][2] * qs, qv[r][ks][3] * qs, qa[2 * ks][2], qa[2 * ks][3]);
                    split_f16x2(qv2[r][ks][0] * qs, qv2[r][ks][1] * qs, qa[2 * ks + 1][0], qa[2 * ks + 1][1]);
                    split_f16x2(qv2[r][ks][2] * qs, qv2[r][ks][3] * qs, qa[2 * ks + 1][2], qa[2 * ks + 1][3]);
                } else if constexpr (SPLIT) {
                    split_f16x2(qv[r][ks][0] * qs, qv[r][ks][1] * qs, qa[ks][0], qa[ks][1]);
                    split_f16x2(qv2[r][ks][0] * qs, qv2[r][ks][1] * qs, qa[ks][2], qa[ks][3]);
                } else {
                    qa[ks][0 + r] = f32x2_to_f16x2(qv[r][ks][0] * qs, qv[r][ks][1] * qs);
                    qa[ks][2 + r] = f32x2_to_f16x2(qv2[r][ks][0] * qs, qv2[r][ks][1] * qs);
                }
            }
        }
    }

    // ---- stream the tiles -------------------------------------------------------------------
    float m[RS], l[RS];
#pragma unroll
    for (int r = 0; r < RS; ++r) { m[r] = kMaskedScore; l[r] = 0.f; }
    constexpr int NACC = TR ? NQB : NDB;
    float acc[NACC][4];
#pragma unroll
    for (int nb = 0; nb < NACC; ++nb) { acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0.f; }
    bool timed_out = false;
    // ---- split ticket -----------------------------------------------------------------------------
    // Every CTA of a (sequence, kv-head) draws one ticket from a 64-bit word that only ever counts
    // up; there is one word per split count, so ticket / n_splits is the number of the launch among
    // those that used the word and ticket % n_splits the CTA's place in the draw.  The CTA that
    // draws last merges the splits; the launch number, together with the host's count of launches
    // on this workspace, is the tag of this launch's partials.  The ticket is drawn by one thread
    // as its warp starts on its last tile: late enough that the last drawer is one of the last
    // CTAs to finish, early enough that the answer is there when the stream ends.  Nothing waits
    // for a ticket, nothing resets one, and every CTA draws exactly one whatever happens to its
    // tiles, so the words stay consistent.
    unsigned long long ticket = 0ull;
    bool drawn = false;
    const bool draws = threadIdx.x == 32 && p.n_splits > 1u && mp.cluster == 0u;
    auto draw_ticket = [&]() {
        ticket = atomicAdd(mp.tickets + (uint64_t(s) * p.n_kv_heads + kvh) * 256u + p.n_splits, 1ull);
        drawn = true;
    };
    if (draws && my_tiles <= 1u) draw_ticket();
    VFKV_TRACE(3);

    // Lane-constant parts of the swizzled shared-memory addresses (tile_addr with the tile base
    // left out).  In every case the unit index is an even compile-time number plus a lane bit, so
    // unit ^ (row & 7) = even_part ^ (lane_bit ^ row & 7) and four variants cover all units.
    const uint32_t lm = lane >> 3, lr = lane & 7;
    uint32_t qk_sw[4];        // K ldmatrix: row 8*(2jp + lm/2) + lr, unit 2u + (lm & 1)
#pragma unroll
    for (uint32_t u = 0; u < 4; ++u)
        qk_sw[u] = TR ? ((lm & 1) * 8 + lr) * 128 + (((2 * u) ^ ((lm >> 1) ^ lr)) << 4)     // row half lm & 1, unit 2u + lm / 2
                      : ((lm >> 1) * 8 + lr) * 128 + (((2 * u) ^ ((lm & 1) ^ lr)) << 4);
    // FP8 V words: row 2*tig + e (+8, +16, +24), unit 2u + gid/4, word gid%4
    // F16 V ldmatrix.trans: row 8*(lm & 1) + lr, unit 2u + lm/2
    uint32_t v_sw[FP8 ? 8 : 4];
    if constexpr (FP8) {
#pragma unroll
        for (uint32_t u = 0; u < 4; ++u)
#pragma unroll
            for (uint32_t e = 0; e < 2; ++e)
                v_sw[2 * u + e] = (2 * tig + e) * 128 + ((u ^ tig) << 5) + (((gid >> 2) ^ e) << 4) + (gid & 3) * 4;
    } else {
#pragma unroll
        for (uint32_t u = 0; u < 4; ++u)
            v_sw[u] = TR ? (8 * (lm >> 1) + lr) * 128 + (((2 * u) ^ ((lm & 1) ^ lr)) << 4)  // row half lm / 2, unit 2u + (lm & 1)
                         : (8 * (lm & 1) + lr) * 128 + (((2 * u) ^ ((lm >> 1) ^ lr)) << 4);
    }

    for (uint32_t n = 0; n < my_tiles; ++n) {
        const uint32_t st = n % kStages;
        const uint32_t t0 = begin + (warp + n * kWarps) * TP;
        const uint32_t kt = stage0 + st * S::STAGE_BYTES, vt = kt + S::TILE_BYTES;
        if (draws && n != 0u && n + 1u == my_tiles) draw_ticket();
        if (!mbar_wait_bounded(bar0 + 8 * st, (n / kStages) & 1u)) { timed_out = true; break; }
        const uint32_t n_valid = min(uint32_t(TP), end - t0);
        if (n == 0) VFKV_TRACE(4);

        // rows at and beyond `end` may hold anything (stale tokens, another slot): zero them in V so
        // that 0 * garbage cannot become NaN; their scores are masked below.
        if (n_valid < uint32_t(TP)) {
            const uint32_t units = (TP - n_valid) * NC * 8;
            for (uint32_t i = lane; i < units; i += 32) {
                const uint32_t r = n_valid + i / (NC * 8), c = (i / 8) % NC, u = i % 8;
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(vt + c * TP * 128 + r * 128 + u * 16), "r"(0u) : "memory");
            }
            __syncwarp();
        }

        if (new_owner && n == new_tile / kWarps) {       // the appended token's row of this tile
            const uint32_t r = len - 1 - t0;
#pragma unroll
            for (uint32_t i = 0; i < NEWU; ++i) {
                const uint32_t u = lane + 32 * i;
                if (u < 2 * UPT) {
                    const uint32_t uu = u % UPT;
                    const uint32_t addr = tile_addr<TP>(u < UPT ? kt : vt, uu / 8, r, uu % 8);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(newu[i].x), "r"(newu[i].y),
                                 "r"(newu[i].z), "r"(newu[i].w) : "memory");
                }
            }
            __syncwarp();
        }

        const bool full = n_valid == uint32_t(TP);
        if constexpr (TR) {
        // ---- S^T = K Q^T : M = 16 positions per block, N = the heads' high / low columns ----------
        float sc[MB][4];
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) { sc[mb][0] = sc[mb][1] = sc[mb][2] = sc[mb][3] = 0.f; }
        {
            const uint32_t kb[4] = {kt + qk_sw[0], kt + qk_sw[1], kt + qk_sw[2], kt + qk_sw[3]};
            qk_t<FP8, TP, D>(kb, qb, sc);
        }
        // this thread's scores: head tig, positions t0 + 16mb + gid and + 8 (high + low column summed)
        float x[MB][2];
        float tmax = kMaskedScore;
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                float v = (sc[mb][2 * i] + sc[mb][2 * i + 1]) * mult[0];
                if constexpr (CAP) v = p.softcap * tanhf(v / p.softcap) * kLog2e;
                if (!full) v = uint32_t(16 * mb + 8 * i) + gid < n_valid ? v : kMaskedScore;
                x[mb][i] = v;
                tmax = fmaxf(tmax, v);
            }
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 8));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 16));
        const float mn = fmaxf(m[0], tmax);
        const float corr = fast_exp2(m[0] - mn);
        const bool changed = mn != m[0];
        m[0] = mn;
        l[0] *= corr;
        if (__any_sync(0xffffffffu, changed)) {
#pragma unroll
            for (int nb = 0; nb < NACC; ++nb) { acc[nb][0] *= corr; acc[nb][1] *= corr; acc[nb][2] *= corr; acc[nb][3] *= corr; }
        }
        // p = 2^(x - m) as {high, low} half pairs = this thread's two columns of a position row;
        // the 8x8 transpose turns them into the B fragment (k = positions, n = columns) of O^T += V^T P^T
        uint32_t pb[MB][2];
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float pv = fast_exp2(x[mb][i] - mn);
                l[0] += pv;
                pb[mb][i] = movmatrix_trans(hi_lo_f16x2(pv * kPScale));
            }
        if constexpr (FP8) {
            uint32_t vb[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) vb[i] = vt + v_sw[i];
            pv_t_fp8<TP, D>(vb, pb, acc);
        } else {
            const uint32_t vb[4] = {vt + v_sw[0], vt + v_sw[1], vt + v_sw[2], vt + v_sw[3]};
            pv_t_f16<TP, D>(vb, pb[0], acc);
        }
        } else {
        // ---- S = Q K^T : M = q rows, N = 8 positions per block, K = 32 bytes of the head slice ----
        float sc[NB][4];
#pragma unroll
        for (int j = 0; j < NB; ++j) { sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f; }
        {
            const uint32_t kb[4] = {kt + qk_sw[0], kt + qk_sw[1], kt + qk_sw[2], kt + qk_sw[3]};
            qk_steps<FP8, TP, NB, KSTEPS, QSTEPS>(kb, qa, sc);
        }

        // ---- softmax bookkeeping in the log2 domain -------------------------------------------
        // this thread's scores: logical row r, block j, element i  <->  position t0 + 8j + 2tig + i
        float x[RS][NB][2];
        float tmax[RS];
#pragma unroll
        for (int r = 0; r < RS; ++r) {
            tmax[r] = kMaskedScore;
#pragma unroll
            for (int j = 0; j < NB; ++j)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    float v = SPLIT ? (sc[j][i] + sc[j][i + 2]) : sc[j][2 * r + i];
                    if constexpr (CAP) {
                        v *= mult[r];
                        v = p.softcap * tanhf(v / p.softcap) * kLog2e;
                    } else {
                        v *= mult[r];                      // scale * log2(e) / q_scale
                    }
                    x[r][j][i] = v;
                }
            if (!full) {                                   // a split's last tile: mask the tail
#pragma unroll
                for (int j = 0; j < NB; ++j)
#pragma unroll
                    for (int i = 0; i < 2; ++i)
                        x[r][j][i] = uint32_t(8 * j + 2 * tig + i) < n_valid ? x[r][j][i] : kMaskedScore;
            }
#pragma unroll
            for (int j = 0; j < NB; ++j) tmax[r] = fmaxf(tmax[r], fmaxf(x[r][j][0], x[r][j][1]));
            tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
            tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
        }
        float corr[RS];
        bool changed = false;
#pragma unroll
        for (int r = 0; r < RS; ++r) {
            const float mn = fmaxf(m[r], tmax[r]);
            corr[r] = fast_exp2(m[r] - mn);
            changed |= mn != m[r];
            m[r] = mn;
            l[r] *= corr[r];
        }
        if (__any_sync(0xffffffffu, changed)) {
#pragma unroll
            for (int nb = 0; nb < NDB; ++nb) {
                acc[nb][0] *= corr[0]; acc[nb][1] *= corr[0];
                acc[nb][2] *= corr[SPLIT ? 0 : 1]; acc[nb][3] *= corr[SPLIT ? 0 : 1];
            }
        }
        // p = 2^(x - m); a masked score is -1e30 against a finite m (every tile has a valid position),
        // which gives exactly 0.
#pragma unroll
        for (int r = 0; r < RS; ++r) {
            const float mo = m[r];
#pragma unroll
            for (int j = 0; j < NB; ++j)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const float pv = fast_exp2(x[r][j][i] - mo);
                    x[r][j][i] = pv * kPScale;
                    l[r] += pv;
                }
        }

        // ---- O += P V ----------------------------------------------------------------------------
        if constexpr (FP8) {
            // A rows 0-7: high half-precision term of p, rows 8-15: low term.  First k step: positions
            // {2tig, 2tig+1} and {8+2tig, 9+2tig}; second k step: the same + 16.
            uint32_t pa[2][4];
            split_f16x2(x[0][0][0], x[0][0][1], pa[0][0], pa[0][1]);
            split_f16x2(x[0][1][0], x[0][1][1], pa[0][2], pa[0][3]);
            split_f16x2(x[0][2][0], x[0][2][1], pa[1][0], pa[1][1]);
            split_f16x2(x[0][3][0], x[0][3][1], pa[1][2], pa[1][3]);
            uint32_t vb[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) vb[i] = vt + v_sw[i];
            pv_fp8<TP, D>(vb, pa, acc);
        } else {
            uint32_t pa[4];
            if constexpr (SPLIT) {
                split_f16x2(x[0][0][0], x[0][0][1], pa[0], pa[1]);
                split_f16x2(x[0][1][0], x[0][1][1], pa[2], pa[3]);
            } else {
                pa[0] = f32x2_to_f16x2(x[0][0][0], x[0][0][1]);
                pa[2] = f32x2_to_f16x2(x[0][1][0], x[0][1][1]);
                pa[1] = f32x2_to_f16x2(x[RS - 1][0][0], x[RS - 1][0][1]);
                pa[3] = f32x2_to_f16x2(x[RS - 1][1][0], x[RS - 1][1][1]);
            }
            const uint32_t vb[4] = {vt + v_sw[0], vt + v_sw[1], vt + v_sw[2], vt + v_sw[3]};
            pv_f16<TP, D>(vb, pa, acc);
        }
        }

        // ---- refill this stage -----------------------------------------------------------------
        // The stage was only read (ldmatrix / ld.shared) since its barrier completed, except in a
        // split's last tile, which is never refilled; __syncwarp orders those reads before the issue.
        __syncwarp();
        if (lane == 0 && n + kStages < my_tiles) issue(n + kStages);
    }

    VFKV_TRACE(5);
    // host-side failure injection (tests): after its tiles have all landed, so that no copy is still
    // in flight, this CTA reports a wait that ran out and publishes nothing
    if (split == mp.fail_split && kvh == 0u && s == 0u) timed_out = true;
    if (timed_out) {
        if (lane == 0) { atomicOr(p.status, 1u); s_flag = 1; }
    }
    if (threadIdx.x == 32) {
        uint32_t tag = 0u, merger = 0u;
        if (draws) {
            if (!drawn) draw_ticket();            // a wait that ran out before the last tile
            uint32_t place, launch_no;
            if ((ticket >> 32) == 0ull) {         // the usual case, without a 64-bit division
                place = uint32_t(ticket) % p.n_splits; launch_no = uint32_t(ticket) / p.n_splits;
            } else {
                place = uint32_t(ticket % p.n_splits); launch_no = uint32_t(ticket / p.n_splits);
            }
            // the last n_mergers drawers merge: merger = 1 + its rank among them, 0 for the others
            const uint32_t n_mrg = min(mp.n_mergers, p.n_splits);
            merger = place + n_mrg >= p.n_splits ? place + n_mrg - p.n_splits + 1u : 0u;
            // never 0, the value of a cleared workspace; launches that share a host count are replays
            // of one graph node (same addresses), which the device-side number tells apart
            tag = 0x80000000u | ((mp.launch_seq & 0x7FFFu) << 16) | (launch_no & 0xFFFFu);
        }
        s_tag = tag; s_merger = merger;
    }
    __syncthreads();          // all tiles consumed (or abandoned): the ring is free for the merge
    VFKV_TRACE(6);
    const bool gave_up = s_flag != 0u;
    if (gave_up && mp.cluster == 0u) return;      // in a cluster every CTA has to reach the cluster barriers

    // ---- merge the warps' partials in shared memory ---------------------------------------------
    constexpr int NH = (FP8 || !ROWS2) ? 8 : 16;              // head rows this CTA can hold
    constexpr int DP = D + 1;                                 // odd row pitch: the 32 lanes hit 32 banks
    float *sm_o = reinterpret_cast<float *>(ring_ptr);        // [kWarps][NH][DP]
    float *sm_m = sm_o + kWarps * NH * DP;                    // [kWarps][NH]
    float *sm_l = sm_m + kWarps * NH;                         // [kWarps][NH]
    if constexpr (TR) {
        // this thread's head is tig; its l covers the positions of its own gid
        l[0] += __shfl_xor_sync(0xffffffffu, l[0], 4);
        l[0] += __shfl_xor_sync(0xffffffffu, l[0], 8);
        l[0] += __shfl_xor_sync(0xffffffffu, l[0], 16);
        if (tig < g) {
            if (gid == 0) { sm_m[warp * NH + tig] = m[0]; sm_l[warp * NH + tig] = l[0]; }
            float *o = sm_o + (warp * NH + tig) * DP;
#pragma unroll
            for (int db = 0; db < NACC; ++db) {
                if constexpr (FP8) {
                    const uint32_t d0 = 32 * (db / 2) + 4 * gid + 2 * (db % 2);
                    o[d0] = (acc[db][0] + acc[db][1]) * kInvPScale;
                    o[d0 + 1] = (acc[db][2] + acc[db][3]) * kInvPScale;
                } else {
                    o[16 * db + gid] = (acc[db][0] + acc[db][1]) * kInvPScale;
                    o[16 * db + 8 + gid] = (acc[db][2] + acc[db][3]) * kInvPScale;
                }
            }
        }
    } else {
#pragma unroll
    for (int r = 0; r < RS; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        if (tig == 0) {
            sm_m[warp * NH + gid + 8 * r] = m[r];
            sm_l[warp * NH + gid + 8 * r] = l[r];
        }
    }
#pragma unroll
    for (int nb = 0; nb < NDB; ++nb) {
        if constexpr (FP8) {
            // column n of block nb is dim 32*(nb/4) + 4n + nb%4 (see the V transpose above)
            const uint32_t d0 = 32 * (nb / 4) + 4 * (2 * tig) + (nb % 4);
            float *o = sm_o + (warp * NH + gid) * DP;
            o[d0] = (acc[nb][0] + acc[nb][2]) * kInvPScale;
            o[d0 + 4] = (acc[nb][1] + acc[nb][3]) * kInvPScale;
        } else {
            const uint32_t d0 = 8 * nb + 2 * tig;
            float *o = sm_o + (warp * NH + gid) * DP;
            if constexpr (SPLIT) {
                o[d0] = (acc[nb][0] + acc[nb][2]) * kInvPScale; o[d0 + 1] = (acc[nb][1] + acc[nb][3]) * kInvPScale;
            } else {
                o[d0] = acc[nb][0] * kInvPScale; o[d0 + 1] = acc[nb][1] * kInvPScale;
                o[8 * DP + d0] = acc[nb][2] * kInvPScale; o[8 * DP + d0 + 1] = acc[nb][3] * kInvPScale;
            }
        }
    }
    }
    __syncthreads();

    const bool direct = p.n_splits == 1;
    const bool fan = p.fan != nullptr;
    FanoutSlot fs{};
    if (fan) fs = fanout_slot(s_fan, D, s_fan.rank, s_epoch + 1u);

    // ---- cluster form of the split merge -----------------------------------------------------------
    // The CTAs of one (sequence, kv-head) are a thread-block cluster: each leaves its partial in its
    // own shared memory, and after one cluster barrier CTA r merges the r-th slice of the g x D
    // outputs across all CTAs through distributed shared memory (flash_attn_reduce.comp:51-80).
    // No partial goes to global memory, no ticket is drawn.  The closing barrier keeps every CTA's
    // shared memory alive until its peers have read it.
    if (mp.cluster != 0u) {
        float *cx_o = sm_l + kWarps * NH;                      // [g][D]
        float *cx_m = cx_o + NH * D;                           // [g]
        float *cx_l = cx_m + NH;                               // [g]
        for (uint32_t idx = threadIdx.x; idx < g * D; idx += blockDim.x) {
            const uint32_t j = idx / D, d = idx % D;
            float M = kMaskedScore;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) M = fmaxf(M, sm_m[w * NH + j]);
            float L = 0.f, O = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float f = fast_exp2(sm_m[w * NH + j] - M);
                L = fmaf(sm_l[w * NH + j], f, L);
                O = fmaf(sm_o[(w * NH + j) * DP + d], f, O);
            }
            if (gave_up) { M = kMaskedScore; L = 0.f; O = 0.f; }
            cx_o[idx] = O;
            if (d == 0) { cx_m[j] = M * kLn2; cx_l[j] = L; }
        }
        VFKV_TRACE(7);
        __syncthreads();
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        VFKV_TRACE(8);
        const uint32_t n = p.n_splits;
        const uint32_t per = (g * D + n - 1) / n;
        const uint32_t e_end = min((split + 1) * per, g * D);
        for (uint32_t e = split * per + threadIdx.x; e < e_end; e += blockDim.x) {
            const uint32_t j = e / D, d = e % D;
            const uint32_t a_o = smem_u32(cx_o + e), a_m = smem_u32(cx_m + j), a_l = smem_u32(cx_l + j);
            constexpr uint32_t CH = 16;
            float oo[CH], mm[CH], ll[CH];
#pragma unroll
            for (uint32_t i = 0; i < CH; ++i) {
                oo[i] = 0.f; mm[i] = kMaskedScore; ll[i] = 0.f;
                if (i < n) {
                    uint32_t ro, rm, rl;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ro) : "r"(a_o), "r"(i));
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rm) : "r"(a_m), "r"(i));
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rl) : "r"(a_l), "r"(i));
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(oo[i]) : "r"(ro) : "memory");
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(mm[i]) : "r"(rm) : "memory");
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(ll[i]) : "r"(rl) : "memory");
                }
            }
            float gmax = kMaskedScore, gsum = 0.f, a = 0.f;
#pragma unroll
            for (uint32_t i = 0; i < CH; ++i) gmax = fmaxf(gmax, mm[i]);
#pragma unroll
            for (uint32_t i = 0; i < CH; ++i) {
                const float kn = __expf(mm[i] - gmax);
                gsum = fmaf(ll[i], kn, gsum);
                a = fmaf(oo[i], kn, a);
            }
            const uint64_t row = uint64_t(s) * p.n_q_heads + kvh * g + j;
            if (p.out) p.out[row * D + d] = gsum > 0.f ? a * (1.0f / gsum) : 0.f;
            if (p.out_o) {
                p.out_o[row * D + d] = a;
                if (d == 0) { p.out_m[row] = gmax; p.out_l[row] = gsum; }
            }
            if (fan) {
#pragma unroll
                for (uint32_t r = 0; r < 8; ++r) {
                    if (r < s_fan.world) {
                        uint64_t *dst = s_fan.base[r];
                        fanout_store(dst + fs.o + row * D + d, a, fs.epoch);
                        if (d == 0) {
                            fanout_store(dst + fs.m + row, gmax, fs.epoch);
                            fanout_store(dst + fs.m + s_fan.n_rows + row, gsum, fs.epoch);
                        }
                    }
                }
            }
        }
        VFKV_TRACE(9);
        __syncthreads();                                       // reconverge before the aligned barrier
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        return;
    }
    // ---- this CTA's partial: the warps' partials merged, two dims per thread ----------------------
    const uint32_t HD2 = D / 2;
    const uint32_t n_pairs = g * HD2;                          // pairs of output values of this (sequence, kv-head)
    auto cta_partial = [&](uint32_t j, uint32_t d, float &O0, float &O1, float &Mn, float &L) {
        float M = kMaskedScore;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) M = fmaxf(M, sm_m[w * NH + j]);
        L = 0.f; O0 = 0.f; O1 = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float f = fast_exp2(sm_m[w * NH + j] - M);
            L = fmaf(sm_l[w * NH + j], f, L);
            O0 = fmaf(sm_o[(w * NH + j) * DP + d], f, O0);
            O1 = fmaf(sm_o[(w * NH + j) * DP + d + 1], f, O1);
        }
        Mn = M * kLn2;                                         // partials carry natural-log maxima
    };
    // Final values of one output pair: the caller's buffers and, in a position-sharded call, every
    // GPU's exchange buffer.
    auto emit = [&](uint32_t idx, float a0, float a1, float gmax, float gsum) {
        const uint32_t j = idx / HD2, d = 2 * (idx % HD2);
        const uint64_t row = uint64_t(s) * p.n_q_heads + kvh * g + j;
        if (p.out && mp.fan_merge == 0u) {
            const float inv = gsum > 0.f ? 1.0f / gsum : 0.f;
            *reinterpret_cast<float2 *>(p.out + row * D + d) = make_float2(a0 * inv, a1 * inv);
        }
        if (p.out_o) {
            *reinterpret_cast<float2 *>(p.out_o + row * D + d) = make_float2(a0, a1);
            if (d == 0) { p.out_m[row] = gmax; p.out_l[row] = gsum; }
        }
        if (fan) {
            for (uint32_t r = 0; r < s_fan.world; ++r) {
                uint64_t *dst = s_fan.base[r];
                fanout_store2(dst + fs.o + row * D + d, a0, a1, fs.epoch);
                if (d == 0) {
                    fanout_store(dst + fs.m + row, gmax, fs.epoch);
                    fanout_store(dst + fs.m + s_fan.n_rows + row, gsum, fs.epoch);
                }
            }
        }
    };

    // ---- several splits: publish the partial; the CTA that drew the last ticket merges -------------
    // The partial goes to the workspace as tagged words (one 16-byte store = two {value, tag}
    // words).  No fence and no flag follow: whoever merges polls the words themselves until each
    // carries this launch's tag.  Every other CTA is done once its stores are issued and leaves
    // its SM to the next launch.  The last drawer has drawn after every CTA of its group had begun
    // its last tile, so it only ever waits for CTAs that are about to store.
    // Layout of the group's partials: [slice of the output pairs = one per merging CTA][split][span],
    // span = the o words of the slice's `per` pairs, then the {m, l} words of all g heads (every slice
    // has its own copy of those), padded to an odd number of 16-byte units so that lanes reading the
    // same unit of consecutive splits fall into different shared-memory banks.  All that one merging
    // CTA needs is then one contiguous block.
    const uint32_t tag = s_tag;
    const uint64_t grp = uint64_t(s) * p.n_kv_heads + kvh;
    const uint32_t n_mrg = direct ? 1u : min(mp.n_mergers, p.n_splits);
    const uint32_t per = (n_pairs + n_mrg - 1) / n_mrg;
    const uint32_t span = 2u * (per + g) + (((per + g) & 1u) ? 0u : 2u);
    uint64_t *const gp = mp.tag_part + grp * (uint64_t(p.n_splits) * n_mrg * span);
    if (!direct) {
        for (uint32_t idx = threadIdx.x; idx < n_pairs; idx += blockDim.x) {
            const uint32_t j = idx / HD2, d = 2 * (idx % HD2);
            float O0, O1, Mn, L;
            cta_partial(j, d, O0, O1, Mn, L);
            const uint32_t sl = per > 1u ? __umulhi(idx, mp.per_recip) : idx;       // = idx / per
            tagged_store2(gp + (uint64_t(sl) * p.n_splits + split) * span + 2u * (idx - sl * per), O0, O1, tag);   // = o[j][d], o[j][d + 1]
            const uint32_t c = idx % HD2;          // the first n_mrg threads of a head each write one copy of its {m, l}
            if (c < n_mrg) tagged_store2(gp + (uint64_t(c) * p.n_splits + split) * span + 2u * per + 2u * j, Mn, L, tag);
        }
        VFKV_TRACE(7);
        if (s_merger == 0u) return;
    } else {                  // a single split: this CTA's partial is the local result
        for (uint32_t idx = threadIdx.x; idx < n_pairs; idx += blockDim.x) {
            float a0, a1, gmax, gsum;
            cta_partial(idx / HD2, 2 * (idx % HD2), a0, a1, gmax, gsum);
            emit(idx, a0, a1, gmax, gsum);
        }
        VFKV_TRACE(8);
    }
    const bool xrank = fan && mp.fan_merge != 0u;
    if (direct && !xrank) { VFKV_TRACE(9); return; }

    // ---- the last drawers merge the splits ---------------------------------------------------------------
    // Everything from here on runs once per launch on a few CTAs per (sequence, kv-head), straight
    // after the hot loop: measured, such code costs what it takes to fetch its instructions, ten
    // cycles and more apiece, and one SM reads its L2 at some 64 bytes per clock, so the code is kept
    // short and rolled and the work is shared: the last n_mergers drawers each take one slice of the
    // output pairs.  (Only CTAs that have drawn wait, and at most n_mergers per group, far fewer
    // than there are SMs, so a CTA that has yet to start always finds one.)  A merger brings its
    // slice of every split's partial into the now idle ring with asynchronous copies; then teams of lanes
    // merge its output pairs out of shared memory (flash_attn_reduce.comp:51-80, maximum first)
    // and check the tags as they go.  A word that does not carry this launch's tag yet sends the
    // step round again, up to the time limit.
    __syncthreads();          // the warps' partials in the ring are dead (uniform: the whole CTA merges or none of it)
    uint64_t *const stgw = reinterpret_cast<uint64_t *>(ring_ptr);
    const uint32_t stg_base = ring;                               // shared-window address of stgw
    // this CTA's slice of the pairs
    const uint32_t lo = direct ? 0u : min((s_merger - 1u) * per, n_pairs), hi = min(lo + per, n_pairs);
    const uint32_t n_mine = hi - lo;
    if (!direct) {
        uint32_t team = 1u;                                       // power of two, at most a warp
        while (team < 32u && 2u * team * n_mine <= blockDim.x && 2u * team <= p.n_splits) team *= 2u;
        // Asynchronous 16-byte copies bring the slice's block ([split][span], contiguous) into the ring,
        // all requests in flight at once; the tag checks of the merge below tell whether every word
        // of this launch was there, and if not the step goes round again.  With a few splits the first
        // copy is issued at once -- the merging CTAs are the last to finish, so the partials are
        // usually there, and a look first would cost one more round trip.  With many splits, and in
        // every later round, thread i first polls the word of split i that is stored last in this
        // slice, so that a copy is not spent on a block that is still incomplete.
        const uint64_t *const block = gp + uint64_t(s_merger - 1u) * p.n_splits * span;
        uint64_t t0 = 0;
        for (uint32_t round = 0;; ++round) {
            if (round != 0u || p.n_splits > 32u) {
                bool late = false;
                const uint64_t t_in = global_timer_ns();
                for (uint32_t i = threadIdx.x; i < p.n_splits; i += blockDim.x) {
                    const uint64_t *w = block + uint64_t(i) * span + (n_mine != 0u ? 2u * (n_mine - 1u) : 2u * per);
                    while (!tags_are(tagged_load2(w), tag)) {
                        if (global_timer_ns() - t_in > mp.merge_wait_ns) { late = true; break; }
                        __nanosleep(20);
                    }
                }
                if (__syncthreads_or(late)) {                     // a partial of this launch never arrived
                    if (threadIdx.x == 0) atomicOr(p.status, 1u);
                    return;
                }
            }
            if (round == 0u) VFKV_TRACE(10);
            for (uint32_t k = threadIdx.x; k < p.n_splits * span / 2u; k += blockDim.x)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(stg_base + 16u * k), "l"(block + 2ull * k) : "memory");
            asm volatile("cp.async.wait_all;" ::: "memory");
            __syncthreads();
            if (round == 0u) VFKV_TRACE(11);
            // `team` neighbouring lanes share one output pair, each taking every team-th split (a
            // slice has fewer pairs than the CTA has threads); they combine through shuffles
            bool missing = false;
            const uint32_t sub = threadIdx.x % team, per_pass = blockDim.x / team;
            for (uint32_t b = 0; b < n_mine; b += per_pass) {
                const uint32_t q2 = b + threadIdx.x / team;
                const bool live = q2 < n_mine;
                const uint32_t idx = lo + (live ? q2 : 0u), j = idx / HD2;
                const uint32_t po = stg_base + 8u * (sub * span + 2u * (idx - lo)), pm = stg_base + 8u * (sub * span + 2u * per + 2u * j);
                const uint32_t step = 8u * team * span;
                float gmax = kMaskedScore, gsum = 0.f, a0 = 0.f, a1 = 0.f;
#pragma unroll 4
                for (uint32_t i = sub, a = pm; i < p.n_splits; i += team, a += step) {
                    const ulonglong2 mw = lds_u64x2(a);
                    missing = missing || !tags_are(mw, tag);
                    gmax = fmaxf(gmax, tagged_value(mw.x));
                }
                for (uint32_t o = 1; o < team; o <<= 1) gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, o));
#pragma unroll 4
                for (uint32_t i = sub, a = po, am = pm; i < p.n_splits; i += team, a += step, am += step) {
                    const ulonglong2 ow = lds_u64x2(a);
                    const ulonglong2 mw = lds_u64x2(am);
                    missing = missing || !tags_are(ow, tag);
                    const float kn = __expf(tagged_value(mw.x) - gmax);
                    gsum = fmaf(tagged_value(mw.y), kn, gsum);
                    a0 = fmaf(tagged_value(ow.x), kn, a0);
                    a1 = fmaf(tagged_value(ow.y), kn, a1);
                }
                for (uint32_t o = 1; o < team; o <<= 1) {
                    gsum += __shfl_xor_sync(0xffffffffu, gsum, o);
                    a0 += __shfl_xor_sync(0xffffffffu, a0, o);
                    a1 += __shfl_xor_sync(0xffffffffu, a1, o);
                }
                const bool bad = __any_sync(0xffffffffu, missing);
                if (live && sub == 0u && !bad) emit(idx, a0, a1, gmax, gsum);
            }
            if (!__syncthreads_or(missing)) break;               // also: every thread is done with the staged words
            const uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            if (__syncthreads_or(now - t0 > mp.merge_wait_ns)) { // a partial of this launch never arrived (decided together)
                if (threadIdx.x == 0) atomicOr(p.status, 1u);
                return;
            }
        }
        VFKV_TRACE(8);
    }
    if (!xrank) { VFKV_TRACE(9); return; }

    // ---- position-sharded call: merge the blocks of all ranks ------------------------------------------
    // Every rank's kernel stores its block of these rows into this GPU's buffer, this rank's own
    // block included (emit above).  The same scheme as above for this CTA's pairs, with the
    // exchange's time limit: the o words of a slice are contiguous in each rank's block and come in
    // by asynchronous copies, the few m and l words by one polling load per thread.  Loads touch
    // this GPU's memory only.
    {
        const uint64_t *local = s_fan.base[s_fan.rank];
        const uint32_t e = fs.epoch, world = s_fan.world;
        const uint64_t row0 = uint64_t(s) * p.n_q_heads + kvh * g;
        const uint32_t span = 2u * per;                           // words per rank
        float *const s_ml = reinterpret_cast<float *>(stgw + uint64_t(world) * span);   // [world][2][g]
        uint64_t t0 = 0;
        bool late = false;
        for (;;) {
            for (uint32_t k = threadIdx.x; k < world * n_mine; k += blockDim.x) {
                const uint32_t r = k / n_mine, q2 = k % n_mine;
                const FanoutSlot rs = fanout_slot(s_fan, D, r, e);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                             ::"r"(stg_base + 8u * (r * span + 2u * q2)), "l"(local + rs.o + row0 * D + 2ull * (lo + q2)) : "memory");
            }
            bool missing = false;
            for (uint32_t k = threadIdx.x; k < world * 2u * g; k += blockDim.x) {
                const uint32_t r = k / (2u * g), which = (k / g) & 1u, j = k % g;
                const FanoutSlot rs = fanout_slot(s_fan, D, r, e);
                const uint64_t w = tagged_load1_sys(local + rs.m + uint64_t(which) * s_fan.n_rows + row0 + j);
                missing = missing || uint32_t(w >> 32) != e;
                s_ml[k] = tagged_value(w);
            }
            asm volatile("cp.async.wait_all;" ::: "memory");
            __syncthreads();
            for (uint32_t idx = lo + threadIdx.x; idx < hi; idx += blockDim.x) {
                const uint32_t j = idx / HD2;
                float gmax = kMaskedScore, gsum = 0.f, a0 = 0.f, a1 = 0.f;
                for (uint32_t r = 0; r < world; ++r) gmax = fmaxf(gmax, s_ml[(r * 2u) * g + j]);
                for (uint32_t r = 0; r < world; ++r) {
                    const ulonglong2 ow = *reinterpret_cast<const ulonglong2 *>(stgw + uint64_t(r) * span + 2 * (idx - lo));
                    missing = missing || !tags_are(ow, e);
                    const float kn = __expf(s_ml[(r * 2u) * g + j] - gmax);
                    gsum = fmaf(s_ml[(r * 2u + 1u) * g + j], kn, gsum);
                    a0 = fmaf(tagged_value(ow.x), kn, a0);
                    a1 = fmaf(tagged_value(ow.y), kn, a1);
                }
                // a rank that never answered: the row is written as zeros, not as a partial sum
                const float inv = (gsum > 0.f && !late) ? 1.0f / gsum : 0.f;
                if ((!missing || late) && p.out)
                    *reinterpret_cast<float2 *>(p.out + row0 * D + 2 * idx) = make_float2(a0 * inv, a1 * inv);
            }
            if (!__syncthreads_or(missing) || late) break;
            const uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            late = __syncthreads_or(now - t0 > s_fan.wait_ns);    // decided together; one more round writes the zeros
            __nanosleep(100);
        }
        if (late && threadIdx.x == 0) atomicOr(p.status, 8u);
    }
    VFKV_TRACE(9);
}

// ---- host side -------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// A byte-typed 2-D view of one layer's slab(s): inner = one token row, outer = slots * max_seq rows.
bool encode_map(vfkv_ctx *ctx, CUtensorMap *out, const void *base, uint64_t row_bytes, uint64_t rows, uint32_t box_rows)
{
    if (!ctx->encode_tiled) return false;
    cuuint64_t dims[2] = {row_bytes, rows};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled)(
        out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

template <int DT, int D, bool ROWS2, int W, int NS, bool CAP, bool TR>
int32_t launch_k(vfkv_ctx *ctx, const CUtensorMap &tk, const CUtensorMap &tv, const MmaParams &mp, cudaStream_t st)
{
    using S = Shape<DT, D, W, NS>;
    constexpr int kNH = (DT == VFKV_F8 || !ROWS2) ? 8 : 16;
    // the ring doubles as the scratch of the cross-warp merge: [W][NH][D + 1] + 2 [W][NH] floats
    constexpr bool kMergeFits = (W * kNH * (D + 1) + 2 * W * kNH) * 4 <= S::RING_BYTES;
    if constexpr (S::SMEM_BYTES > 227 * 1024 || !kMergeFits) {
        return set_error(ctx, VFKV_ERR_UNSUPPORTED, "tuning does not fit in shared memory for this shape");
    } else {
        auto kern = attn_split_mma_kernel<DT, D, ROWS2, W, NS, CAP, TR>;
        // per device, shared by every context and thread: setting the attribute twice is harmless,
        // the flag only saves the call
        static std::atomic<bool> configured[64];
        if (!configured[ctx->device & 63].load(std::memory_order_acquire)) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM_BYTES);
            if (e != cudaSuccess) return check_cuda(ctx, e, "cudaFuncSetAttribute(tensor-core attention)");
            configured[ctx->device & 63].store(true, std::memory_order_release);
        }
        MmaParams lp = mp;
        // A merging CTA stages its slice of every split's partial in the ring, and the group's partials
        // ([slice][split][span] words, see the kernel) have to fit the workspace: fewer splits where the
        // ring is too small, fewer merging CTAs where the workspace is.
        const uint64_t n_pairs = uint64_t(mp.a.group) * (D / 2), groups = uint64_t(mp.a.n_kv_heads) * mp.a.n_seqs;
        auto span_of = [&](uint32_t n_mrg) {
            const uint64_t per = (n_pairs + n_mrg - 1) / n_mrg;
            return 2 * (per + mp.a.group) + (((per + mp.a.group) & 1) ? 0 : 2);
        };
        if (lp.n_mergers == 0u) lp.n_mergers = 1u;
        for (int pass = 0; pass < 3 && lp.a.n_splits > 1u; ++pass) {      // fewer splits can mean fewer mergers, hence larger slices
            const uint32_t n_mrg = lp.n_mergers < lp.a.n_splits ? lp.n_mergers : lp.a.n_splits;
            const uint64_t sbytes = span_of(n_mrg) * 8;
            if (uint64_t(lp.a.n_splits) * sbytes <= uint64_t(S::RING_BYTES)) break;
            lp.a.n_splits = uint32_t(S::RING_BYTES / sbytes) > 0u ? uint32_t(S::RING_BYTES / sbytes) : 1u;
        }
        while (lp.a.n_splits > 1u) {
            const uint32_t n_mrg = lp.n_mergers < lp.a.n_splits ? lp.n_mergers : lp.a.n_splits;
            if (groups * lp.a.n_splits * n_mrg * span_of(n_mrg) <= mp.tag_words) break;
            if (lp.n_mergers == 1u) return set_error(ctx, VFKV_ERR_INVALID, "workspace too small for this call");
            lp.n_mergers = n_mrg - 1u;
        }
        if (lp.a.n_splits > 1u) {          // the last check of the ring, with the number of merging CTAs that was settled on
            const uint32_t n_mrg = lp.n_mergers < lp.a.n_splits ? lp.n_mergers : lp.a.n_splits;
            if (uint64_t(lp.a.n_splits) * span_of(n_mrg) * 8 > uint64_t(S::RING_BYTES))
                lp.a.n_splits = uint32_t(S::RING_BYTES / (span_of(n_mrg) * 8)) > 0u ? uint32_t(S::RING_BYTES / (span_of(n_mrg) * 8)) : 1u;
        }
        {
            const uint32_t n_mrg = lp.a.n_splits > 1u ? (lp.n_mergers < lp.a.n_splits ? lp.n_mergers : lp.a.n_splits) : 1u;
            const uint64_t per = (n_pairs + n_mrg - 1) / n_mrg;
            lp.per_recip = per > 1 ? uint32_t(((1ull << 32) + per - 1) / per) : 0xFFFFFFFFu;
        }
        if (lp.fan_merge && 8ull * (uint64_t(mp.a.group) * D * 8 + 2ull * mp.a.group * 4) > uint64_t(S::RING_BYTES))
            return set_error(ctx, VFKV_ERR_UNSUPPORTED, "one-launch exchange does not fit this kernel shape");
        dim3 grid(lp.a.n_splits, mp.a.n_kv_heads, mp.a.n_seqs);
        {
            ProfScope ps(ctx, VFKV_PROF_FA_SPLIT, st);
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = grid;
            cfg.blockDim = dim3(W * 32);
            cfg.dynamicSmemBytes = S::SMEM_BYTES;
            cfg.stream = st;
            cudaLaunchAttribute attr[2];
            unsigned n_attr = 0;
            if (mp.pdl) {
                attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
                attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
                ++n_attr;
            }
            cfg.attrs = attr;
            cfg.numAttrs = n_attr;
            // Cluster form of the split merge: the splits of one (sequence, kv-head) as one cluster.
            // Used when the context asks for it, the merge scratch fits beside the ring, and the
            // device can keep every cluster of the grid resident at once (so none waits for another).
            constexpr int NH = (DT == VFKV_F8 || !ROWS2) ? 8 : 16;
            constexpr bool kFits = (W * NH * (D + 1) + 2 * W * NH + NH * D + 2 * NH) * 4 <= S::RING_BYTES;
            if (kFits && ctx->cluster_merge && mp.fan_merge == 0u && lp.a.n_splits >= 2 && lp.a.n_splits <= 16) {
                static std::atomic<int> max_clusters[64][17];   // per device and cluster size; 0 = not asked yet, -1 = no
                std::atomic<int> &slot_known = max_clusters[ctx->device & 63][lp.a.n_splits];
                int known = slot_known.load(std::memory_order_acquire);
                cudaLaunchAttribute &ca = attr[n_attr];
                ca.id = cudaLaunchAttributeClusterDimension;
                ca.val.clusterDim.x = lp.a.n_splits; ca.val.clusterDim.y = 1; ca.val.clusterDim.z = 1;
                cfg.numAttrs = n_attr + 1;
                if (known == 0) {
                    known = -1;
                    bool ok = true;
                    if (lp.a.n_splits > 8)
                        ok = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
                    int n = 0;
                    if (ok && cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n > 0) known = n;
                    cudaGetLastError();
                    slot_known.store(known, std::memory_order_release);
                }
                const uint64_t clusters = uint64_t(mp.a.n_kv_heads) * mp.a.n_seqs;
                if (known > 0 && clusters <= uint64_t(known)) lp.cluster = 1;
                else cfg.numAttrs = n_attr;
            }
            cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tk, tv, lp);
            if (e != cudaSuccess) return check_cuda(ctx, e, "tensor-core attention launch");
        }
        ctx->launches++;
        return check_cuda(ctx, cudaGetLastError(), "tensor-core attention launch");
    }
}

template <int DT, int D, bool ROWS2, bool CAP, bool TR>
int32_t launch_c(vfkv_ctx *ctx, const CUtensorMap &tk, const CUtensorMap &tv, const MmaParams &mp, cudaStream_t st)
{
    // Small grids (at most one CTA per SM): 8 warps x 3 stages where that fits in shared memory.
    // Everything else: 4 warps x 3 stages, two CTAs per SM at 8 KB stages (measured faster than
    // three CTAs of 4 x 2, whose 168-register cap costs more than the extra warps give).
    constexpr bool kWide = Shape<DT, D, 8, 3>::SMEM_BYTES <= 200 * 1024;
    const uint64_t ctas = uint64_t(mp.a.n_splits) * mp.a.n_kv_heads * mp.a.n_seqs;
    uint32_t w = ctx->tune_warps, ns = ctx->tune_stages;
    if (w == 0) w = (kWide && ctas <= uint64_t(ctx->sm_count)) ? 8 : 4;
    // 4 warps: as many stages (up to 3) as still let two CTAs share an SM.  At head_dim 256 a stage
    // is 16 KB, so that is one stage (64 KB per CTA): measured 5.5 TB/s against 3.9 TB/s with three
    // stages and a single CTA of 4 warps per SM (F16, 8 sequences x 32768, windows 1024 / none).
    constexpr int kTwoPerSm = 113 * 1024;
    constexpr int kNH = (DT == VFKV_F8 || !ROWS2) ? 8 : 16;
    constexpr int kMergeBytes = (4 * kNH * (D + 1) + 2 * 4 * kNH) * 4;       // cross-warp merge scratch, 4 warps
    constexpr bool kOk2 = Shape<DT, D, 4, 2>::SMEM_BYTES <= kTwoPerSm && kMergeBytes <= Shape<DT, D, 4, 2>::RING_BYTES;
    constexpr bool kOk1 = Shape<DT, D, 4, 1>::SMEM_BYTES <= kTwoPerSm && kMergeBytes <= Shape<DT, D, 4, 1>::RING_BYTES;
    if (ns == 0) ns = (w == 8 || Shape<DT, D, 4, 3>::SMEM_BYTES <= kTwoPerSm) ? 3 : kOk2 ? 2 : kOk1 ? 1 : 3;
    if (w == 8 && ns == 3) return launch_k<DT, D, ROWS2, 8, 3, CAP, TR>(ctx, tk, tv, mp, st);
    if (w == 4 && ns == 3) return launch_k<DT, D, ROWS2, 4, 3, CAP, TR>(ctx, tk, tv, mp, st);
    if (w == 4 && ns == 2) return launch_k<DT, D, ROWS2, 4, 2, CAP, TR>(ctx, tk, tv, mp, st);
    if (w == 4 && ns == 1) return launch_k<DT, D, ROWS2, 4, 1, CAP, TR>(ctx, tk, tv, mp, st);
    if (w == 8 && ns == 1) return launch_k<DT, D, ROWS2, 8, 1, CAP, TR>(ctx, tk, tv, mp, st);
    return set_error(ctx, VFKV_ERR_INVALID, "attention tuning must be 4x1, 4x2, 4x3, 8x1 or 8x3 (warps x stages)");
}

template <int DT, int D, bool ROWS2>
int32_t launch_t(vfkv_ctx *ctx, const CUtensorMap &tk, const CUtensorMap &tv, const MmaParams &mp, cudaStream_t st)
{
    // groups of at most 4 q-heads: the transposed products (heads on the N side of the MMAs)
    if constexpr (!ROWS2) {
        if (mp.a.group <= 4u)
            return mp.a.softcap > 0.f ? launch_c<DT, D, ROWS2, true, true>(ctx, tk, tv, mp, st)
                                      : launch_c<DT, D, ROWS2, false, true>(ctx, tk, tv, mp, st);
    }
    return mp.a.softcap > 0.f ? launch_c<DT, D, ROWS2, true, false>(ctx, tk, tv, mp, st)
                              : launch_c<DT, D, ROWS2, false, false>(ctx, tk, tv, mp, st);
}

}  // namespace

bool attn_mma_supported(const AttnArgs &a)
{
    if (a.kv.k_scales || a.kv.v_scales) return false;
    if (a.kv.n_kv_heads == 0 || a.n_q_heads % a.kv.n_kv_heads != 0) return false;
    const uint32_t g = a.n_q_heads / a.kv.n_kv_heads, D = a.kv.head_dim;
    if (uint64_t(a.kv.n_slots) * a.kv.max_seq >= (1ull << 31)) return false;
    if ((reinterpret_cast<uintptr_t>(a.kv.k) | reinterpret_cast<uintptr_t>(a.kv.v)) % 16 != 0) return false;
    if (reinterpret_cast<uintptr_t>(a.q) % 16 != 0) return false;
    if ((reinterpret_cast<uintptr_t>(a.out) | reinterpret_cast<uintptr_t>(a.out_o)) % 16 != 0) return false;
    if (a.kv.dtype == VFKV_F8) return g <= 8 && (D == 128 || D == 256);
    if (a.kv.dtype == VFKV_F16) return g <= 16 && (D == 64 || D == 128 || D == 256);
    return false;
}

int32_t launch_attn_mma(vfkv_ctx *ctx, vfkv_workspace *ws, const AttnArgs &a, uint32_t n_splits, cudaStream_t st)
{
    if (!ctx->encode_tiled) return set_error(ctx, VFKV_ERR_CUDA, "cuTensorMapEncodeTiled is unavailable in this driver");
    const uint32_t D = a.kv.head_dim, es = a.kv.dtype == VFKV_F8 ? 1 : 2;
    const uint64_t row_bytes = uint64_t(a.kv.n_kv_heads) * D * es;
    const uint64_t rows = uint64_t(a.kv.n_slots) * a.kv.max_seq;
    if (a.kv.n_slots > 1 && a.kv.slot_stride_bytes != uint64_t(a.kv.max_seq) * row_bytes)
        return set_error(ctx, VFKV_ERR_INVALID, "slots must be contiguous slabs");
    const uint32_t box_rows = a.kv.dtype == VFKV_F8 ? 32 : 16;
    CUtensorMap tk, tv;
    if (a.kv.tm_k && a.kv.tm_v) {
        tk = *static_cast<const CUtensorMap *>(a.kv.tm_k);
        tv = *static_cast<const CUtensorMap *>(a.kv.tm_v);
    } else if (!encode_map(ctx, &tk, a.kv.k, row_bytes, rows, box_rows) ||
               !encode_map(ctx, &tv, a.kv.v, row_bytes, rows, box_rows)) {
        return set_error(ctx, VFKV_ERR_CUDA, "cuTensorMapEncodeTiled failed");
    }
    MmaParams mp;
    mp.a = make_params(ctx, ws, a, n_splits);
    mp.tickets = ws ? ws->tickets : nullptr;
    mp.tag_part = ws ? ws->tag_part : nullptr;
    mp.tag_words = ws ? ws->tag_words : 0;
    mp.merge_wait_ns = ctx->merge_wait_ns;
    mp.launch_seq = (ws && n_splits > 1) ? ws->launch_seq++ : 0u;
    // Several CTAs per (sequence, kv-head) share the merge -- four, or up to sixteen when a few
    // groups have the GPU to themselves and are cut into many splits -- as long as all the CTAs that
    // may be waiting at one time stay a small part of the SMs (a waiting CTA holds its SM).
    {
        const uint64_t groups = uint64_t(a.seq.n_seqs) * a.kv.n_kv_heads;
        const uint64_t room = uint64_t(ctx->sm_count) / 4 / (groups ? groups : 1);
        const uint64_t most = n_splits > 16 ? (n_splits + 7) / 8 : 4;      // a merger for every eight splits
        mp.n_mergers = uint32_t(room < 1 ? 1 : room > most ? most : room);
        if (mp.n_mergers > 16u) mp.n_mergers = 16u;
    }
    mp.trace = ctx->d_trace;
    if (ctx->d_trace && ctx->trace_ring > 1) {      // successive launches write successive blocks of the buffer
        const uint64_t ctas = uint64_t(n_splits) * a.kv.n_kv_heads * a.seq.n_seqs;
        mp.trace = ctx->d_trace + (ctx->trace_seq++ % ctx->trace_ring) * ctas * 16;
    }
    // Mode 2 prefetches K/V before it waits for the kernel in front of it.  When that kernel was
    // launched through this context and wrote rows of the very slab this call reads (the same layer
    // twice in a row, or a layer that reads its publisher's slab right after the publisher's
    // append), the prefetch has to wait as well.
    mp.pdl = (ctx->pdl == 2u && (ctx->last_written_slab == a.kv.k || ctx->last_written_slab == kAnySlab)) ? 1u : ctx->pdl;
    mp.cluster = 0;
    mp.fan_merge = (a.fan && a.fan_merge) ? 1u : 0u;
    mp.fail_split = ctx->debug_fail_split;
    mp.k_new = a.k_new;
    mp.v_new = a.v_new;
    if ((reinterpret_cast<uintptr_t>(a.k_new) | reinterpret_cast<uintptr_t>(a.v_new)) % 16 != 0)
        return set_error(ctx, VFKV_ERR_INVALID, "new K/V rows must be 16-byte aligned");
    if (n_splits > 1 && (!mp.tickets || !mp.tag_part)) return set_error(ctx, VFKV_ERR_INVALID, "workspace has no split-merge storage");
    if (n_splits > 255) return set_error(ctx, VFKV_ERR_UNSUPPORTED, "the tensor-core attention kernel merges at most 255 splits");
    if (n_splits > 1 && uint64_t(a.seq.n_seqs) * a.kv.n_kv_heads > ws->n_counters)
        return set_error(ctx, VFKV_ERR_INVALID, "workspace too small for this call");
    const uint32_t g = a.n_q_heads / a.kv.n_kv_heads;
    auto run = [&]() -> int32_t {
        if (a.kv.dtype == VFKV_F8) {
            if (D == 128) return launch_t<VFKV_F8, 128, false>(ctx, tk, tv, mp, st);
            if (D == 256) return launch_t<VFKV_F8, 256, false>(ctx, tk, tv, mp, st);
        } else {
            const bool r2 = g > 8;
            if (D == 64) return r2 ? launch_t<VFKV_F16, 64, true>(ctx, tk, tv, mp, st) : launch_t<VFKV_F16, 64, false>(ctx, tk, tv, mp, st);
            if (D == 128) return r2 ? launch_t<VFKV_F16, 128, true>(ctx, tk, tv, mp, st) : launch_t<VFKV_F16, 128, false>(ctx, tk, tv, mp, st);
            if (D == 256) return r2 ? launch_t<VFKV_F16, 256, true>(ctx, tk, tv, mp, st) : launch_t<VFKV_F16, 256, false>(ctx, tk, tv, mp, st);
        }
        return set_error(ctx, VFKV_ERR_UNSUPPORTED, "shape outside the tensor-core attention kernel");
    };
    const int32_t rc = run();
    if (rc == VFKV_OK) ctx->last_written_slab = a.k_new ? a.kv.k : nullptr;
    return rc;
}

// Pre-encodes the two tensor maps of one layer of a cache (host memory; reused by every call).
bool encode_layer_maps(vfkv_ctx *ctx, const KvView &v, void *tm_k_out, void *tm_v_out)
{
    if (v.dtype == VFKV_F32) return false;
    const uint32_t es = v.dtype == VFKV_F8 ? 1 : 2;
    const uint64_t row_bytes = uint64_t(v.n_kv_heads) * v.head_dim * es;
    if (row_bytes < 128 || (uint64_t(v.head_dim) * es) % 128 != 0) return false;
    const uint64_t rows = uint64_t(v.n_slots) * v.max_seq;
    const uint32_t box_rows = v.dtype == VFKV_F8 ? 32 : 16;
    return encode_map(ctx, static_cast<CUtensorMap *>(tm_k_out), v.k, row_bytes, rows, box_rows) &&
           encode_map(ctx, static_cast<CUtensorMap *>(tm_v_out), v.v, row_bytes, rows, box_rows);
}

}  // namespace vfkv

extern "C" int32_t vfkv_ctx_set_cluster_merge(vfkv_ctx *ctx, uint32_t on)
{
    if (!ctx || on > 1) return VFKV_ERR_INVALID;
    ctx->cluster_merge = on;
    return VFKV_OK;
}
