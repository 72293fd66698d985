// Split-K GQA decode attention on CUDA cores: every cache dtype (F32 / F16 /
// E4M3), head_dim 64..512, any group size.  This is the shape-complete path and
// the one the reference's own kernel-level tests (F32 cache,
// tests/correctness.rs:2791-2894) run through; the tensor-core kernel in
// attn_mma.cu takes over for the FP8 / F16 shapes it covers.
//
// Replaces vk_shaders/flash_attn_split.comp (and flash_attn.comp for short
// sequences).  Differences in how the work is laid out, none in the math:
//   - one CTA serves one KV head and all the q-heads that share it, so K and V
//     are read once per KV head instead of once per q-head
//     (flash_attn_split.comp:83-95 re-reads them group-size times);
//   - a warp reads a K (or V) head-slice as one contiguous 128..2048-byte row
//     (the shader has lane t walk row t, a stride of one whole token);
//   - positions below kv_start are never visited (the shader dispatches those
//     tiles and multiplies V by zero, :133-144);
//   - the partial count is a parameter instead of ceil(seq_len / 64).
#include "attn_params.cuh"
#include "fp8_codec.cuh"

namespace vfkv {

template <int NB> struct RawVec { uint32_t w[NB / 4]; };
template <> struct RawVec<2> { uint32_t w[1]; };

template <int NB> __device__ __forceinline__ RawVec<NB> load_raw(const uint8_t *p)
{
    RawVec<NB> r;
    if constexpr (NB == 2) {
        r.w[0] = *reinterpret_cast<const uint16_t *>(p);
    } else if constexpr (NB == 4) {
        r.w[0] = *reinterpret_cast<const uint32_t *>(p);
    } else if constexpr (NB == 8) {
        uint2 t = *reinterpret_cast<const uint2 *>(p);
        r.w[0] = t.x; r.w[1] = t.y;
    } else {
#pragma unroll
        for (int i = 0; i < NB / 16; ++i) {
            uint4 t = reinterpret_cast<const uint4 *>(p)[i];
            r.w[4 * i] = t.x; r.w[4 * i + 1] = t.y; r.w[4 * i + 2] = t.z; r.w[4 * i + 3] = t.w;
        }
    }
    return r;
}

template <int DT, int VEC>
__device__ __forceinline__ void decode_vec(const RawVec<VEC * (DT == VFKV_F32 ? 4 : DT == VFKV_F16 ? 2 : 1)> &r,
                                           float *x)
{
    if constexpr (DT == VFKV_F32) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) x[i] = __uint_as_float(r.w[i]);
    } else if constexpr (DT == VFKV_F16) {
#pragma unroll
        for (int i = 0; i < VEC / 2; ++i) {
            uint32_t w = r.w[i];
            float2 f = __half22float2(*reinterpret_cast<__half2 *>(&w));
            x[2 * i] = f.x; x[2 * i + 1] = f.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < VEC / 2; ++i) {
            uint32_t w = r.w[i / 2] >> ((i & 1) * 16);
            float2 f = e4m3x2_to_float2(w & 0xFFFFu);
            x[2 * i] = f.x; x[2 * i + 1] = f.y;
        }
    }
}

constexpr int kGenericWarps = 8;
constexpr int kUnroll = 4;   // positions a warp handles per iteration

template <int DT, int VEC, int GB>
__global__ void __launch_bounds__(kGenericWarps * 32)
attn_split_generic_kernel(const AttnParams p)
{
    constexpr int ES = DT == VFKV_F32 ? 4 : DT == VFKV_F16 ? 2 : 1;
    constexpr int NB = VEC * ES;
    extern __shared__ float smem[];

    const uint32_t split = blockIdx.x;
    const uint32_t head_blocks = (p.group + GB - 1) / GB;
    const uint32_t kvh = blockIdx.y / head_blocks, hb = blockIdx.y % head_blocks;
    const uint32_t s = blockIdx.z;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t D = p.head_dim;
    const uint32_t h0 = kvh * p.group + hb * GB;
    const uint32_t nh = min(uint32_t(GB), p.group - hb * GB);

    uint32_t slot, start, len, begin, end;
    seq_range(p, s, &slot, &start, &len);
    split_range(start, len, p.n_splits, split, 32, &begin, &end);

    // this lane's slice of each of the CTA's q rows
    float q[GB][VEC];
#pragma unroll
    for (int j = 0; j < GB; ++j) {
        const float *qr = p.q + (uint64_t(s) * p.n_q_heads + h0 + (j < nh ? j : 0)) * D + lane * VEC;
#pragma unroll
        for (int i = 0; i < VEC; ++i) q[j][i] = (j < nh) ? qr[i] : 0.f;
    }

    const uint64_t row_bytes = uint64_t(p.n_kv_heads) * D * ES;
    const uint8_t *kbase = p.k + uint64_t(slot) * p.slot_stride_bytes + uint64_t(kvh) * D * ES + lane * NB;
    const uint8_t *vbase = p.v + uint64_t(slot) * p.slot_stride_bytes + uint64_t(kvh) * D * ES + lane * NB;
    const float *ksc = p.k_scales ? p.k_scales + uint64_t(slot) * p.slot_stride_scales + kvh : nullptr;
    const float *vsc = p.v_scales ? p.v_scales + uint64_t(slot) * p.slot_stride_scales + kvh : nullptr;

    float m[GB], l[GB], acc[GB][VEC];
#pragma unroll
    for (int j = 0; j < GB; ++j) {
        m[j] = kMaskedScore; l[j] = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[j][i] = 0.f;
    }

    for (uint32_t t0 = begin + warp * kUnroll; t0 < end; t0 += kGenericWarps * kUnroll) {
        RawVec<NB> kr[kUnroll], vr[kUnroll];
        float kscale[kUnroll], vscale[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            uint32_t t = min(t0 + u, end - 1);          // clamped loads stay in range; masked below
            kr[u] = load_raw<NB>(kbase + uint64_t(t) * row_bytes);
            vr[u] = load_raw<NB>(vbase + uint64_t(t) * row_bytes);
            kscale[u] = ksc ? ksc[uint64_t(t) * p.n_kv_heads] : 1.f;
            vscale[u] = vsc ? vsc[uint64_t(t) * p.n_kv_heads] : 1.f;
        }
        float sc[kUnroll][GB];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            float kx[VEC];
            decode_vec<DT, VEC>(kr[u], kx);
#pragma unroll
            for (int j = 0; j < GB; ++j) {
                float d = 0.f;
#pragma unroll
                for (int i = 0; i < VEC; ++i) d = fmaf(q[j][i], kx[i], d);
                sc[u][j] = d;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < kUnroll; ++u)
#pragma unroll
                for (int j = 0; j < GB; ++j) sc[u][j] += __shfl_xor_sync(0xffffffffu, sc[u][j], o);

        float mnew[GB];
#pragma unroll
        for (int j = 0; j < GB; ++j) mnew[j] = m[j];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const bool valid = (t0 + u) < end;
#pragma unroll
            for (int j = 0; j < GB; ++j) {
                float x = apply_softcap(sc[u][j] * kscale[u] * p.scale, p.softcap);
                x = valid ? x : kMaskedScore;
                sc[u][j] = x;
                mnew[j] = fmaxf(mnew[j], x);
            }
        }
#pragma unroll
        for (int j = 0; j < GB; ++j) {
            float corr = __expf(m[j] - mnew[j]);
            m[j] = mnew[j];
            l[j] *= corr;
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[j][i] *= corr;
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const bool valid = (t0 + u) < end;
            float vx[VEC];
            decode_vec<DT, VEC>(vr[u], vx);
#pragma unroll
            for (int j = 0; j < GB; ++j) {
                float pj = valid ? __expf(sc[u][j] - m[j]) : 0.f;
                l[j] += pj;
                pj *= vscale[u];
#pragma unroll
                for (int i = 0; i < VEC; ++i) acc[j][i] = fmaf(pj, valid ? vx[i] : 0.f, acc[j][i]);
            }
        }
    }

    // ---- merge the warps' partials (the reduce shader's update, once per warp) ----
    float *sm_m = smem;                                   // [W][GB]
    float *sm_l = sm_m + kGenericWarps * GB;              // [W][GB]
    float *sm_o = sm_l + kGenericWarps * GB;              // [W][GB][D]
#pragma unroll
    for (int j = 0; j < GB; ++j) {
        if (lane == 0) { sm_m[warp * GB + j] = m[j]; sm_l[warp * GB + j] = l[j]; }
#pragma unroll
        for (int i = 0; i < VEC; ++i) sm_o[(warp * GB + j) * D + lane * VEC + i] = acc[j][i];
    }
    __syncthreads();
    for (uint32_t idx = threadIdx.x; idx < nh * D; idx += blockDim.x) {
        uint32_t j = idx / D, d = idx % D;
        float M = kMaskedScore;
#pragma unroll
        for (int w = 0; w < kGenericWarps; ++w) M = fmaxf(M, sm_m[w * GB + j]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < kGenericWarps; ++w) {
            float f = __expf(sm_m[w * GB + j] - M);
            L = fmaf(sm_l[w * GB + j], f, L);
            O = fmaf(sm_o[(w * GB + j) * D + d], f, O);
        }
        const uint64_t row = uint64_t(s) * p.n_q_heads + h0 + j;
        if (p.n_splits == 1) {
            if (p.out) p.out[row * D + d] = L > 0.f ? O * (1.0f / L) : 0.f;
            if (p.out_o) {
                p.out_o[row * D + d] = O;
                if (d == 0) { p.out_m[row] = M; p.out_l[row] = L; }
            }
        } else {
            const uint64_t pi = row * p.n_splits + split;
            p.part_o[pi * D + d] = O;
            if (d == 0) { p.part_m[pi] = M; p.part_l[pi] = L; }
        }
    }
}

template <int DT, int VEC, int GB>
static int32_t launch_one(vfkv_ctx *ctx, const AttnParams &p, cudaStream_t st)
{
    const uint32_t head_blocks = (p.group + GB - 1) / GB;
    dim3 grid(p.n_splits, p.n_kv_heads * head_blocks, p.n_seqs);
    size_t smem = sizeof(float) * size_t(kGenericWarps) * GB * (p.head_dim + 2);
    auto kern = attn_split_generic_kernel<DT, VEC, GB>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return check_cuda(ctx, e, "cudaFuncSetAttribute(generic attention)");
    }
    {
        ProfScope ps(ctx, VFKV_PROF_FA_SPLIT, st);
        kern<<<grid, kGenericWarps * 32, smem, st>>>(p);
    }
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "generic attention launch");
}

template <int DT, int VEC>
static int32_t launch_gb(vfkv_ctx *ctx, const AttnParams &p, cudaStream_t st)
{
    // heads per CTA: the group itself up to 8; larger groups take several CTAs per KV head
    if (p.group == 1) return launch_one<DT, VEC, 1>(ctx, p, st);
    if (p.group == 2) return launch_one<DT, VEC, 2>(ctx, p, st);
    if (p.group <= 4) return launch_one<DT, VEC, 4>(ctx, p, st);
    if constexpr (VEC <= 8) return launch_one<DT, VEC, 8>(ctx, p, st);
    else return launch_one<DT, VEC, 4>(ctx, p, st);      // head_dim 512: keep registers in bounds
}

template <int DT>
static int32_t launch_vec(vfkv_ctx *ctx, const AttnParams &p, cudaStream_t st)
{
    switch (p.head_dim) {
    case 64: return launch_gb<DT, 2>(ctx, p, st);
    case 128: return launch_gb<DT, 4>(ctx, p, st);
    case 256: return launch_gb<DT, 8>(ctx, p, st);
    case 512: return launch_gb<DT, 16>(ctx, p, st);
    }
    return set_error(ctx, VFKV_ERR_UNSUPPORTED, "head_dim must be 64, 128, 256 or 512");
}

int32_t launch_attn_generic(vfkv_ctx *ctx, vfkv_workspace *ws, const AttnArgs &a, uint32_t n_splits,
                            cudaStream_t st)
{
    AttnParams p = make_params(ctx, ws, a, n_splits);
    switch (a.kv.dtype) {
    case VFKV_F32: return launch_vec<VFKV_F32>(ctx, p, st);
    case VFKV_F16: return launch_vec<VFKV_F16>(ctx, p, st);
    case VFKV_F8: return launch_vec<VFKV_F8>(ctx, p, st);
    }
    return set_error(ctx, VFKV_ERR_INVALID, "unknown dtype");
}

}  // namespace vfkv
