// Log-sum-exp merge of split-K partials and the attention dispatcher.
//
// Replaces vk_shaders/flash_attn_reduce.comp and the host half of
// Forward::run_flash_attn_split_reduce (src/backend/vulkan/forward/runs.rs:1463-1571).
#include "attn_params.cuh"

namespace vfkv {

// flash_attn_reduce.comp:51-80: out = sum_i o_i e^(m_i - M) / sum_i l_i e^(m_i - M) with M the
// maximum of the partial maxima; the final multiply by 1/sum is skipped when
// the caller wants the unnormalised triple (sequence-dimension sharding).
// Partial i of row r: m and l at i*ml_part + r*ml_row, o at i*o_part + r*o_row (+ dim), all in floats.
__global__ void __launch_bounds__(128)
merge_kernel(const float *__restrict__ pm, const float *__restrict__ pl, const float *__restrict__ po,
             uint32_t n_parts, uint64_t ml_part, uint64_t ml_row, uint64_t o_part, uint64_t o_row, uint32_t head_dim,
             float *__restrict__ out, float *__restrict__ out_m, float *__restrict__ out_l,
             float *__restrict__ out_o)
{
    const uint64_t row = blockIdx.x;
    constexpr int kMaxDims = 4;                      // 128 threads x 4 = head_dim 512
    __shared__ float s_red[4], s_sum[4];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // The shader walks the partials with a running (max, sum, acc); the same result, up to
    // rounding, comes from taking the maximum first and then one weighted sum, which leaves
    // every load independent of the others.  The launch is a chain of L2 round trips and nothing
    // else, so it is kept to two: the maxima and sums (one or two parts per thread), then the o rows.
    float gmax = kMaskedScore;
    float m_own[2] = {kMaskedScore, kMaskedScore}, l_own[2] = {0.f, 0.f};      // parts tid and tid + 128
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const uint32_t i = threadIdx.x + 128 * k;
        if (i < n_parts) {
            const uint64_t pi = uint64_t(i) * ml_part + row * ml_row;
            m_own[k] = pm[pi];
            l_own[k] = pl[pi];
        }
    }
    gmax = fmaxf(m_own[0], m_own[1]);
    for (uint32_t i = threadIdx.x + 256; i < n_parts; i += 128) gmax = fmaxf(gmax, pm[uint64_t(i) * ml_part + row * ml_row]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, o));
    if (lane == 0) s_red[warp] = gmax;
    __syncthreads();
    gmax = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
    float gsum = fmaf(l_own[0], __expf(m_own[0] - gmax), l_own[1] * __expf(m_own[1] - gmax));
    for (uint32_t i = threadIdx.x + 256; i < n_parts; i += 128) {
        const uint64_t pi = uint64_t(i) * ml_part + row * ml_row;
        gsum = fmaf(pl[pi], __expf(pm[pi] - gmax), gsum);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) gsum += __shfl_xor_sync(0xffffffffu, gsum, o);
    if (lane == 0) s_sum[warp] = gsum;
    float acc[kMaxDims] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 16
    for (uint32_t i = 0; i < n_parts; ++i) {
        const uint64_t oi = uint64_t(i) * o_part + row * o_row;
        const float kn = __expf(pm[uint64_t(i) * ml_part + row * ml_row] - gmax);
#pragma unroll
        for (int j = 0; j < kMaxDims; ++j) {
            uint32_t d = threadIdx.x + j * 128;
            float t = d < head_dim ? po[oi + d] : 0.f;
            acc[j] = fmaf(t, kn, acc[j]);
        }
    }
    __syncthreads();
    gsum = (s_sum[0] + s_sum[1]) + (s_sum[2] + s_sum[3]);
    const float inv = gsum > 0.f ? 1.0f / gsum : 0.f;   // an empty range yields zeros, not NaN
#pragma unroll
    for (int j = 0; j < kMaxDims; ++j) {
        uint32_t d = threadIdx.x + j * 128;
        if (d < head_dim) {
            if (out) out[row * head_dim + d] = acc[j] * inv;
            if (out_o) out_o[row * head_dim + d] = acc[j];
        }
    }
    if (out_o && threadIdx.x == 0) { out_m[row] = gmax; out_l[row] = gsum; }
}

int32_t launch_merge_ws(vfkv_ctx *ctx, vfkv_workspace *ws, const AttnArgs &a, uint32_t n_splits,
                        cudaStream_t st)
{
    const uint32_t rows = a.seq.n_seqs * a.n_q_heads;
    ProfScope ps(ctx, VFKV_PROF_FA_REDUCE, st);
    const uint64_t D = a.kv.head_dim;
    merge_kernel<<<rows, 128, 0, st>>>(ws->part_m, ws->part_l, ws->part_o, n_splits, 1, n_splits, D, n_splits * D,
                                      a.kv.head_dim, a.out, a.out_m, a.out_l, a.out_o);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "merge launch");
}

int32_t launch_merge_partials(vfkv_ctx *ctx, const float *m, const float *l, const float *o,
                              uint32_t n_parts, uint32_t n_rows, uint32_t head_dim, float *out,
                              cudaStream_t st)
{
    if (n_rows == 0) return VFKV_OK;
    ProfScope ps(ctx, VFKV_PROF_FA_REDUCE, st);
    merge_kernel<<<n_rows, 128, 0, st>>>(m, l, o, n_parts, n_rows, 1, uint64_t(n_rows) * head_dim, head_dim,
                                        head_dim, out, nullptr, nullptr, nullptr);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "merge_partials launch");
}

// One block of n_rows*(head_dim+2) floats per part: m[n_rows], l[n_rows], o[n_rows][head_dim] --
// the layout an all-gather of per-GPU partials produces.
int32_t launch_merge_partials_packed(vfkv_ctx *ctx, const float *packed, uint32_t n_parts, uint32_t n_rows,
                                     uint32_t head_dim, float *out, cudaStream_t st)
{
    if (n_rows == 0) return VFKV_OK;
    const uint64_t block = uint64_t(n_rows) * (head_dim + 2);
    ProfScope ps(ctx, VFKV_PROF_FA_REDUCE, st);
    merge_kernel<<<n_rows, 128, 0, st>>>(packed, packed + n_rows, packed + 2 * uint64_t(n_rows), n_parts, block, 1,
                                        block, head_dim, head_dim, out, nullptr, nullptr, nullptr);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "merge_partials_packed launch");
}

// Split count when the caller passes 0.  The reference always cuts at 64
// positions (runs.rs:766-769); here the count only has to fill the GPU: aim
// for about two CTAs per SM, never cut below 256 positions per split (128 on the tensor cores
// with an F16 cache).
uint32_t choose_splits(const vfkv_ctx *ctx, const AttnArgs &a, uint32_t tile)
{
    uint32_t max_len = a.seq.max_len_hint ? a.seq.max_len_hint : a.kv.max_seq;
    if (!a.seq.seq_lens && !a.seq.positions) max_len = a.seq.seq_len_scalar - a.seq.kv_start_scalar;
    if (a.seq.window && max_len > a.seq.window) max_len = a.seq.window;
    // One split per (sequence, kv-head) once that alone gives every SM two CTAs: the stream is
    // HBM-bound, so a ragged last wave costs little, while every extra split costs a partial
    // write, a ticket and a merge.  Smaller grids are cut until about two CTAs per SM exist, but
    // never below 256 positions per split.
    const uint64_t base = uint64_t(a.seq.n_seqs) * a.kv.n_kv_heads;
    const uint64_t slots = uint64_t(ctx->sm_count) * 2;
    // (an 8-warp CTA of the tensor-core kernel takes 8 tiles at a time: 256 positions of an FP8
    // cache, 128 of an F16 cache, where 16 splits of 128 measured 6.2 us against 6.6 us with 8 of 256
    // on 32 q / 8 kv / 128 at 2048 positions)
    const uint32_t min_chunk = (tile >= 128 && a.kv.dtype == VFKV_F16) ? 128 : tile < 256 ? 256 : tile;
    uint64_t cap = (uint64_t(max_len) + min_chunk - 1) / min_chunk;
    if (cap < 1) cap = 1;
    if (cap > 64) cap = 64;
    uint64_t want = base ? (slots + base - 1) / base : 1;
    // The CTA that merges reads every split's partial: beyond 16 splits that tail costs more than
    // the extra CTAs save (one sequence of 16384 positions, 64 q-heads: 15.9 us with 16 splits,
    // 19.5 us with 37), unless the length rule below asks for more.
    if (want > 16) want = 16;
    // Fewer than eight groups (one long sequence whose kv-heads are spread over several GPUs): the
    // merge is then shared by up to sixteen CTAs of the group, each combining its outputs with a
    // team of lanes, and one CTA per SM pays: 148 / groups splits.
    const bool few_groups = base > 0 && base * 32 <= uint64_t(ctx->sm_count) && tile >= 128;
    if (few_groups) {
        want = uint64_t(ctx->sm_count) / base;
        if (want > 255) want = 255;
        cap = (uint64_t(max_len) + min_chunk - 1) / min_chunk;
        if (cap < 1) cap = 1;
        if (want > cap) want = cap;
        // a CTA of 8 warps takes 256 positions per round of tiles: the fewest splits that need no
        // more rounds than that count does (131 072 positions on one kv-head: 128 splits of 4
        // rounds, 14.1 us, where 148 ragged ones took 15.6 us)
        const uint64_t rounds = ((uint64_t(max_len) + want - 1) / want + 255) / 256;
        const uint64_t fewest = (uint64_t(max_len) + rounds * 256 - 1) / (rounds * 256);
        if (fewest >= 1 && fewest < want) want = fewest;
    }
    // A CTA keeps at most its own ring of stages in flight, which bounds one CTA's stream to a few
    // tens of GB/s: in a ragged batch a sequence much longer than the rest would finish last on
    // its own.  No CTA gets more than 8192 positions, 4096 once contexts beyond 8192 are possible
    // (measured: 64 sequences of 512..16384 tokens 5.0 / 5.5 / 6.1 TB/s with 1 / 2 / 4 splits;
    // 64 x 8192 uniform 6.3 / 6.0 / 5.9 TB/s).
    // The rule is for batches that fill the GPU by themselves; a single long sequence is better off
    // with its 16 splits on 8-warp CTAs, one per SM (131 072 positions, 8 kv-heads: 46.3 us with
    // 16 splits of 8 warps, 51.1 us with 32 splits of 4 warps).
    const uint64_t per_cta = max_len > 8192 ? 4096 : 8192;
    const uint64_t by_len = (uint64_t(max_len) + per_cta - 1) / per_cta;
    if (want < by_len && base >= slots) want = by_len;
    if (want > cap) want = cap;
    if (want < 1) want = 1;
    // A stream-bound grid that spills a few CTAs into another wave pays for a whole wave: 64
    // (sequence, kv-head) pairs x 5 splits = 320 CTAs on 296 slots took 571 us where 9 splits (576
    // CTAs, two full waves) took 354 us and 4 splits (one wave, 86 % full) 379 us (F16, head_dim
    // 256, 8 x 32768 positions).  So when the count above overshoots the slots, take the nearby
    // count that fills its waves best, with a small price per split for the merge.
    if (base * want > slots && base < slots) {
        double best = -1.0;
        uint64_t pick = want;
        const uint64_t hi = cap < 4 * want ? cap : 4 * want;
        for (uint64_t n = want > 1 ? want - 1 : 1; n <= hi; ++n) {
            const uint64_t ctas = base * n, waves = (ctas + slots - 1) / slots;
            const double score = double(ctas) / double(waves * slots) - 0.008 * double(n);
            if (score > best) { best = score; pick = n; }
        }
        want = pick;
    }
    return uint32_t(want);
}

int32_t launch_attention(vfkv_ctx *ctx, vfkv_workspace *ws, const AttnArgs &a, cudaStream_t st)
{
    if (a.seq.n_seqs == 0) return VFKV_OK;
    if (a.kv.n_kv_heads == 0 || a.n_q_heads == 0 || a.n_q_heads % a.kv.n_kv_heads != 0)
        return set_error(ctx, VFKV_ERR_INVALID, "n_q_heads must be a non-zero multiple of n_kv_heads");
    const bool mma_ok = attn_mma_supported(a);
    if (ctx->attn_impl == 2 && !mma_ok)
        return set_error(ctx, VFKV_ERR_UNSUPPORTED, "shape outside the tensor-core attention kernel");
    const bool use_mma = mma_ok && ctx->attn_impl != 1;

    uint32_t n_splits = a.n_splits ? a.n_splits : choose_splits(ctx, a, use_mma ? 128 : 32);
    if (n_splits > 1) {
        if (!ws) return set_error(ctx, VFKV_ERR_INVALID, "a workspace is required when n_splits > 1");
        if (n_splits > ws->max_splits) n_splits = ws->max_splits;
        if (a.seq.n_seqs > ws->max_seqs || a.n_q_heads > ws->n_q_heads || a.kv.head_dim > ws->head_dim)
            return set_error(ctx, VFKV_ERR_INVALID, "workspace too small for this call");
    }
    int32_t rc = use_mma ? launch_attn_mma(ctx, ws, a, n_splits, st)
                         : launch_attn_generic(ctx, ws, a, n_splits, st);
    if (rc != VFKV_OK) return rc;
    // the tensor-core kernel merges its own partials (last CTA of each kv-head)
    if (n_splits > 1 && !use_mma) rc = launch_merge_ws(ctx, ws, a, n_splits, st);
    return rc;
}

}  // namespace vfkv
