// Kernel parameter block shared by the attention kernels and the per-sequence
// argument decoding (slot, visible length, sliding-window lower bound).
#pragma once

#include "common.cuh"

namespace vfkv {

struct AttnParams {
    const uint8_t *k, *v;
    const float *k_scales, *v_scales;
    uint64_t slot_stride_bytes, slot_stride_scales;
    const float *q;
    float *part_o, *part_m, *part_l;       // workspace partials [seq][q_head][split]
    float *out, *out_m, *out_l, *out_o;    // final outputs when one split covers a sequence
    const uint32_t *slot_ids, *seq_lens, *kv_starts, *positions;
    uint32_t slot0, seq_len_scalar, kv_start_scalar, window;
    uint32_t n_q_heads, n_kv_heads, head_dim, group, max_seq, n_slots, n_splits, n_seqs;
    float scale, softcap;
    uint32_t *status;
    const PeerFanout *fan;             // device memory, or null
};

inline AttnParams make_params(const vfkv_ctx *ctx, const vfkv_workspace *ws, const AttnArgs &a,
                              uint32_t n_splits)
{
    AttnParams p{};
    p.k = static_cast<const uint8_t *>(a.kv.k);
    p.v = static_cast<const uint8_t *>(a.kv.v);
    p.k_scales = a.kv.k_scales;
    p.v_scales = a.kv.v_scales;
    p.slot_stride_bytes = a.kv.slot_stride_bytes;
    p.slot_stride_scales = a.kv.slot_stride_scales;
    p.q = a.q;
    p.part_o = ws ? ws->part_o : nullptr;
    p.part_m = ws ? ws->part_m : nullptr;
    p.part_l = ws ? ws->part_l : nullptr;
    p.out = a.out; p.out_m = a.out_m; p.out_l = a.out_l; p.out_o = a.out_o;
    p.slot_ids = a.seq.slot_ids; p.seq_lens = a.seq.seq_lens; p.kv_starts = a.seq.kv_starts;
    p.positions = a.seq.positions;
    p.slot0 = a.seq.slot0; p.seq_len_scalar = a.seq.seq_len_scalar;
    p.kv_start_scalar = a.seq.kv_start_scalar; p.window = a.seq.window;
    p.n_q_heads = a.n_q_heads; p.n_kv_heads = a.kv.n_kv_heads; p.head_dim = a.kv.head_dim;
    p.group = a.n_q_heads / a.kv.n_kv_heads;
    p.max_seq = a.kv.max_seq; p.n_slots = a.kv.n_slots; p.n_splits = n_splits;
    p.n_seqs = a.seq.n_seqs;
    p.scale = a.scale; p.softcap = a.softcap;
    p.status = ctx->d_status;
    p.fan = a.fan;
    return p;
}

#ifdef __CUDACC__
// Visible range [start, len) of sequence s and its slot.  Out-of-range
// arguments from device arrays are clamped and reported through the status
// word instead of being dereferenced.
__device__ __forceinline__ void seq_range(const AttnParams &p, uint32_t s, uint32_t *slot,
                                          uint32_t *start, uint32_t *len)
{
    uint32_t sl = p.slot_ids ? p.slot_ids[s] : p.slot0 + s;
    uint32_t n, st;
    if (p.positions) {
        n = p.positions[s] + 1u;
        st = p.window ? (n > p.window ? n - p.window : 0u)
                      : (p.kv_starts ? p.kv_starts[s] : p.kv_start_scalar);
    } else {
        n = p.seq_lens ? p.seq_lens[s] : p.seq_len_scalar;
        st = p.kv_starts ? p.kv_starts[s] : p.kv_start_scalar;
    }
    if (sl >= p.n_slots || n > p.max_seq) {
        if (threadIdx.x == 0) atomicOr(p.status, 4u);
        if (sl >= p.n_slots) { sl = 0; n = 0; }
        if (n > p.max_seq) n = p.max_seq;
    }
    if (st > n) st = n;
    *slot = sl; *start = st; *len = n;
}

// Positions [*begin, *end) of split `split`; chunks are multiples of `align`.
__device__ __forceinline__ void split_range(uint32_t start, uint32_t len, uint32_t n_splits,
                                            uint32_t split, uint32_t align, uint32_t *begin,
                                            uint32_t *end)
{
    uint32_t eff = len - start;
    uint32_t chunk = (eff + n_splits - 1) / n_splits;
    chunk = (chunk + align - 1) / align * align;
    uint64_t b = uint64_t(start) + uint64_t(split) * chunk;
    uint64_t e = b + chunk;
    if (b > len) b = len;
    if (e > len) e = len;
    *begin = uint32_t(b); *end = uint32_t(e);
}

// Words in one source rank's block of an exchange buffer: m[n_rows], l[n_rows], o[n_rows][head_dim].
__host__ __device__ __forceinline__ uint64_t fanout_block_words(uint32_t n_rows, uint32_t head_dim)
{
    return uint64_t(n_rows) * (head_dim + 2);
}
// Word offsets of source rank `src`'s block of exchange number `epoch` inside any rank's buffer.
struct FanoutSlot {
    uint32_t epoch;
    uint64_t m;          // m[n_rows]; l follows at + n_rows
    uint64_t o;          // o[n_rows][head_dim]; even, so pairs of words are 16-byte aligned
};
__device__ __forceinline__ FanoutSlot fanout_slot(const PeerFanout &f, uint32_t head_dim, uint32_t src, uint32_t epoch)
{
    FanoutSlot s;
    s.epoch = epoch;
    s.m = (uint64_t(epoch & 1u) * f.world + src) * fanout_block_words(f.n_rows, head_dim);
    s.o = s.m + 2ull * f.n_rows;
    return s;
}
__device__ __forceinline__ uint64_t fanout_word(float v, uint32_t tag)
{
    return uint64_t(__float_as_uint(v)) | (uint64_t(tag) << 32);
}
__device__ __forceinline__ void fanout_store(uint64_t *dst, float v, uint32_t tag)
{
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" :: "l"(dst), "l"(fanout_word(v, tag)) : "memory");
}
// Two consecutive values as one 16-byte store of two tagged words (dst 16-byte aligned).  The vector
// store is performed as two 8-byte accesses, each single-copy atomic, which is all a reader relies
// on: it checks the tag of every word it uses.  System scope: the destination may be a peer GPU.
__device__ __forceinline__ void fanout_store2(uint64_t *dst, float v0, float v1, uint32_t tag)
{
    asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" :: "l"(dst), "l"(fanout_word(v0, tag)), "l"(fanout_word(v1, tag)) : "memory");
}
// four consecutive values (dst 16-byte aligned) as two 16-byte stores
__device__ __forceinline__ void fanout_store4(uint64_t *dst, float4 v, uint32_t tag)
{
    fanout_store2(dst, v.x, v.y, tag);
    fanout_store2(dst + 2, v.z, v.w, tag);
}
// The same pair of tagged words inside this GPU's own memory (split partials of the workspace).
__device__ __forceinline__ void tagged_store2(uint64_t *dst, float v0, float v1, uint32_t tag)
{
    asm volatile("st.relaxed.gpu.global.v2.u64 [%0], {%1, %2};" :: "l"(dst), "l"(fanout_word(v0, tag)), "l"(fanout_word(v1, tag)) : "memory");
}
__device__ __forceinline__ ulonglong2 tagged_load2(const uint64_t *src)
{
    ulonglong2 w;
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(w.x), "=l"(w.y) : "l"(src) : "memory");
    return w;
}
__device__ __forceinline__ ulonglong2 tagged_load2_sys(const uint64_t *src)
{
    ulonglong2 w;
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(w.x), "=l"(w.y) : "l"(src) : "memory");
    return w;
}
__device__ __forceinline__ uint64_t tagged_load1_sys(const uint64_t *src)
{
    uint64_t w;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(src) : "memory");
    return w;
}
__device__ __forceinline__ bool tags_are(ulonglong2 w, uint32_t tag)
{
    return uint32_t(w.x >> 32) == tag && uint32_t(w.y >> 32) == tag;
}
__device__ __forceinline__ float tagged_value(uint64_t w) { return __uint_as_float(uint32_t(w)); }

__device__ __forceinline__ float apply_softcap(float s, float cap)
{
    // extension: cap * tanh(s / cap), the formula the reference applies to final
    // logits (src/backend/vulkan/forward/arch/gemma4.rs:85-94)
    return cap > 0.f ? cap * tanhf(s / cap) : s;
}
#endif

}  // namespace vfkv
