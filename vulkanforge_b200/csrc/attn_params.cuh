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
    PeerFanout fan;
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

// Layout of one source rank's block inside an exchange buffer, in floats: m[n_rows], l[n_rows],
// padding to a multiple of 4, o[n_rows][head_dim]; the block itself is padded to a multiple of 4.
__host__ __device__ __forceinline__ uint64_t fanout_o_offset(uint32_t n_rows) { return (2ull * n_rows + 3) & ~3ull; }
__host__ __device__ __forceinline__ uint64_t fanout_block_floats(uint32_t n_rows, uint32_t head_dim)
{
    return (fanout_o_offset(n_rows) + uint64_t(n_rows) * head_dim + 3) & ~3ull;
}
// Where source rank `src`'s block of exchange number e lives inside any rank's exchange buffer.
struct FanoutSlot {
    uint32_t epoch;      // e
    uint64_t m;          // float offset of m[n_rows]; l follows at + n_rows
    uint64_t o;          // float offset of o[n_rows][head_dim] (16-byte aligned)
    uint64_t flags;      // 4-byte offset of this rank's flag row
};
__device__ __forceinline__ FanoutSlot fanout_slot(const PeerFanout &f, uint32_t head_dim, uint32_t src, uint32_t epoch)
{
    FanoutSlot s;
    s.epoch = epoch;
    const uint64_t packed = fanout_block_floats(f.n_rows, head_dim);
    const uint64_t blk = uint64_t(epoch & 1u) * f.world + src;
    s.m = blk * packed;
    s.o = s.m + fanout_o_offset(f.n_rows);
    s.flags = 2ull * f.world * packed + blk * f.n_groups;
    return s;
}
// Publishes flag `group` of this rank's block on every GPU.  Call after a CTA barrier that follows
// the CTA's stores of the block: the release at system scope is cumulative over them.
__device__ __forceinline__ void fanout_publish(const PeerFanout &f, const FanoutSlot &s, uint32_t group)
{
#pragma unroll
    for (uint32_t r = 0; r < 8; ++r) {          // static indices: the pointer table stays in the parameter bank
        if (threadIdx.x == r && r < f.world) {
            uint32_t *flag = reinterpret_cast<uint32_t *>(f.base[r]) + s.flags + group;
            asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(flag), "r"(s.epoch) : "memory");
        }
    }
}

__device__ __forceinline__ float apply_softcap(float s, float cap)
{
    // extension: cap * tanh(s / cap), the formula the reference applies to final
    // logits (src/backend/vulkan/forward/arch/gemma4.rs:85-94)
    return cap > 0.f ? cap * tanhf(s / cap) : s;
}
#endif

}  // namespace vfkv
