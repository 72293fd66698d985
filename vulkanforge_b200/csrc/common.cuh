// Shared internal declarations of libvfkv: context, workspace, kernel
// parameter blocks and the host-side launchers of each kernel family.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <string>
#include <vector>

#include "../../include/vfkv.h"
#include "kv_cache.hpp"

struct vfkv_ctx {
    int device = 0;
    int sm_count = 0;
    std::string last_error;
    uint32_t *d_status = nullptr;      // device word written by bounded waits that give up
    uint32_t attn_impl = 0;            // 0 auto, 1 CUDA-core only, 2 tensor-core only, 3 as 0 but mma.sync instead of tcgen05 (prefill)
    uint32_t tune_warps = 0, tune_stages = 0;   // tensor-core kernel shape, 0 = choose
    float *d_prefill_scratch = nullptr;         // pieces of prefill items cut between CTAs; allocated at first use
    uint32_t prefill_scratch_ctas = 0;
    uint32_t prefill_epoch = 0;                 // value the flags of the current spread prefill launch take
    uint32_t pdl = 0;                  // programmatic dependent launch mode of the attention kernel (0 / 1 / 2)
    // Layer slab (K base address) that the last launch on this context wrote cache rows into, or
    // null: a mode-2 launch that reads the same slab next waits before its K/V prefetch (mode 1).
    const void *last_written_slab = nullptr;
    uint64_t merge_wait_ns = 1000000000ull;   // limit of the merging CTA's wait for the other splits' partials
    uint32_t debug_fail_split = 0xFFFFFFFFu;  // failure injection for tests (vfkv_ctx_debug_fail_split)
    uint32_t cluster_merge = 0;        // 1: merge the splits inside a thread-block cluster where the device allows it
    uint64_t launches = 0;
    unsigned long long *d_trace = nullptr;   // caller-owned device buffer for kernel phase timestamps, or null
    uint32_t trace_ring = 1;                 // blocks in d_trace; launch k of the decode kernel writes block k % trace_ring
    uint64_t trace_seq = 0;
    void *encode_tiled = nullptr;      // cuTensorMapEncodeTiled, resolved at run time
    // per-kernel GPU timing, the analogue of the reference's ShaderProfiler
    // (src/backend/vulkan/profiler.rs:28-187); off unless vfkv_profile_enable(ctx, 1)
    bool profiling = false;
    struct ProfRec { uint32_t label; cudaEvent_t e0, e1; };
    std::vector<ProfRec> prof;
};

struct vfkv_cache {
    vfkv_ctx *ctx = nullptr;
    vfkv::KvCache kv;
    // per-layer TMA descriptors of the K and V slabs, encoded on first use (128 bytes each)
    struct alignas(64) TmapBytes { unsigned char b[128]; };
    std::vector<TmapBytes> tm_k, tm_v;
    std::vector<unsigned char> tm_state;   // 0 = not tried, 1 = ready, 2 = not encodable
};

struct vfkv_workspace {
    vfkv_ctx *ctx = nullptr;
    uint32_t max_seqs = 0, n_q_heads = 0, head_dim = 0, max_splits = 0;
    float *part_o = nullptr;    // [seq][q_head][split][head_dim]
    float *part_m = nullptr;    // [seq][q_head][split]
    float *part_l = nullptr;    // [seq][q_head][split]
    uint32_t *d_u32 = nullptr;  // staging for scalar-call slot/len/start and host-step arrays
    // Tensor-core kernel's split merge: per (sequence, kv-head) 256 ticket words, one per split count,
    // that only count up (ticket / n_splits = launch number, ticket % n_splits = place in the draw);
    // and the split partials as 8-byte words {f32 value, u32 tag}, the tag made of the host's launch
    // count and the device-side launch number, so that a reader that finds the tag has the value.
    unsigned long long *tickets = nullptr;
    uint64_t n_counters = 0;
    uint64_t *tag_part = nullptr;   // per (seq, kv_head): [slice of the output pairs][split][ o words of the slice | {m, l}[g] | pad ]
    uint64_t tag_words = 0;
    uint32_t launch_seq = 0;        // split launches issued on this workspace (the host's half of a tag)
    uint64_t bytes = 0;
    // staging for vfkv_decode_token_host, grown on first use
    float *stage_in = nullptr;
    float *stage_out = nullptr;
    uint64_t stage_in_bytes = 0, stage_out_bytes = 0;
    // vfkv_decode_token_host: the kernel sequence of one token, captured once per configuration and
    // replayed (the analogue of the reference's pre-recorded command buffers, forward/decode.rs:169-259)
    // The layers form up to kTokChunks groups with one graph each, so that a second stream moves the
    // next group's inputs and the previous group's outputs while a group computes.
    static constexpr uint32_t kTokChunks = 4;
    cudaGraphExec_t tok_graphs[kTokChunks] = {nullptr, nullptr, nullptr, nullptr};
    uint64_t tok_key[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t tok_events[2 * kTokChunks] = {};         // inputs there / group done, per group
    // vfkv_decode_token_host_submit / _wait: two tokens in flight, each with its own staging set and
    // its own recorded graph (the analogue of the reference's two command-buffer / fence pairs and
    // per-slot scratch, forward/decode.rs:169-259, forward/setup.rs:203-230).
    struct HostSlot {
        float *in = nullptr, *out = nullptr;
        uint32_t *u32 = nullptr;                         // positions, then slot ids
        uint64_t in_bytes = 0, out_bytes = 0;
        cudaGraphExec_t graph = nullptr;
        uint64_t key[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        cudaEvent_t ev_in = nullptr, ev_done = nullptr, ev_out = nullptr;
        uint64_t ticket = 0;                             // ticket in flight on this slot, 0 = free
        uint32_t launches = 0;
    };
    HostSlot host_slot[2];
    cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;
    uint64_t next_ticket = 1;
};

namespace vfkv {

int32_t set_error(vfkv_ctx *ctx, int32_t status, const std::string &msg);
int32_t check_cuda(vfkv_ctx *ctx, cudaError_t e, const char *what);

// One layer's slab(s) as seen by the attention kernels.
struct KvView {
    const void *k = nullptr;       // start of slot 0 of the layer
    const void *v = nullptr;
    const float *k_scales = nullptr;   // [slot][pos][kv_head] or null
    const float *v_scales = nullptr;
    uint64_t slot_stride_bytes = 0;    // bytes between consecutive slots (K or V)
    uint64_t slot_stride_scales = 0;   // floats between consecutive slots in the scale planes
    uint32_t max_seq = 0;              // rows per slot
    uint32_t n_slots = 1;
    uint32_t dtype = 0;
    uint32_t n_kv_heads = 0;
    uint32_t head_dim = 0;
    const void *tm_k = nullptr;        // pre-encoded CUtensorMap of k / v (host memory), or null
    const void *tm_v = nullptr;
};

// Per-sequence arguments: either device arrays (batch calls) or scalars.
struct SeqArgs {
    const uint32_t *slot_ids = nullptr;   // null -> slot = seq index + slot0
    const uint32_t *seq_lens = nullptr;   // null -> seq_len_scalar
    const uint32_t *kv_starts = nullptr;  // null -> kv_start_scalar, or derived from window
    const uint32_t *positions = nullptr;  // when set: seq_len = positions[i] + 1
    uint32_t slot0 = 0;
    uint32_t seq_len_scalar = 0;
    uint32_t kv_start_scalar = 0;
    uint32_t window = 0;                  // with positions: kv_start = max(0, pos+1-window)
    uint32_t n_seqs = 1;
    uint32_t max_len_hint = 0;
};

// Fan-out of the (m, l, o) partial to every GPU of a position-sharded group, written by the
// attention kernel itself.  base[r] is rank r's exchange buffer (peer memory except base[rank]),
// an array of 8-byte words {f32 value, u32 tag}:
//   [parity 2][source rank][ m[n_rows] | l[n_rows] | o[n_rows][head_dim] ]
// A kernel of exchange number e = *epoch + 1 uses parity e & 1 and tags every word with e.  A word
// is written by one 8-byte store, so a reader that sees the tag has the value: no flag, no fence.
struct PeerFanout {
    uint64_t *base[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    const uint32_t *epoch = nullptr;   // this GPU's count of completed exchanges (device memory)
    uint32_t world = 0;                // 0 = no fan-out
    uint32_t rank = 0;
    uint32_t n_rows = 0;               // sequences * q-heads
    uint32_t pad = 0;
    uint32_t *ctl = nullptr;           // [0] completed exchanges (== epoch), [1] ticket of the kernels that close an exchange
    uint64_t wait_ns = 1000000000ull;  // limit of a wait for the other ranks' words
};

struct AttnArgs {
    KvView kv;
    SeqArgs seq;
    const float *q = nullptr;     // [seq][q_head][head_dim]
    float *out = nullptr;         // [seq][q_head][head_dim]  (normalised)  or null
    float *out_m = nullptr;       // partial outputs for sharded use, or null
    float *out_l = nullptr;
    float *out_o = nullptr;
    uint32_t n_q_heads = 0;
    float scale = 1.f;
    float softcap = 0.f;
    uint32_t n_splits = 0;        // 0 = choose
    // decode step: the token to append at each sequence's last position, [seq][kv_head][dim] f32;
    // only the tensor-core kernel consumes these (it writes the cache rows itself)
    const float *k_new = nullptr;
    const float *v_new = nullptr;
    const PeerFanout *fan = nullptr;   // device copy of the group's fan-out table, or null (tensor-core kernel only)
    // with fan: the attention kernel also waits for the other ranks' blocks in its own buffer, merges
    // them and writes the final rows to `out` (one launch per layer); otherwise vfkv_exchange_merge does
    bool fan_merge = false;
};

// Brackets one kernel launch with a pair of events on its stream while profiling is on.
struct ProfScope {
    vfkv_ctx *ctx; cudaStream_t st; cudaEvent_t e1 = nullptr;
    ProfScope(vfkv_ctx *c, uint32_t label, cudaStream_t s) : ctx(c), st(s)
    {
        if (!ctx->profiling) return;
        vfkv_ctx::ProfRec r{label, nullptr, nullptr};
        if (cudaEventCreate(&r.e0) != cudaSuccess || cudaEventCreate(&r.e1) != cudaSuccess) return;
        cudaEventRecord(r.e0, st);
        e1 = r.e1;
        ctx->prof.push_back(r);
    }
    ~ProfScope() { if (e1) cudaEventRecord(e1, st); }
};

// Launchers (each returns a vfkv_status).
int32_t launch_store(vfkv_ctx *ctx, uint32_t dtype, const float *src, void *dst, uint64_t n,
                     cudaStream_t st);
int32_t launch_fp8_to_f16(vfkv_ctx *ctx, const void *src, void *dst, uint64_t n, cudaStream_t st);

struct AppendArgs {
    const float *k = nullptr, *v = nullptr;   // [n_rows][row_elems]
    void *k_dst = nullptr, *v_dst = nullptr;  // layer base (slot 0)
    float *k_scales = nullptr, *v_scales = nullptr;
    uint64_t slot_stride_bytes = 0, slot_stride_scales = 0;
    uint32_t row_elems = 0, head_dim = 0, n_kv_heads = 0, dtype = 0, max_seq = 0, n_slots = 1;
    // rows: either n_tokens consecutive positions of one slot, or one token per sequence
    uint32_t n_rows = 0;
    uint32_t slot = 0, base_pos = 0;           // consecutive mode
    const uint32_t *slot_ids = nullptr;        // batch mode (positions != null)
    const uint32_t *positions = nullptr;
    // consecutive mode on a position-sharded cache: base_pos is global, only this rank's rows are stored
    uint32_t shard_world = 0, shard_rank = 0, shard_page = 0;
};
int32_t launch_append(vfkv_ctx *ctx, const AppendArgs &a, cudaStream_t st);

int32_t launch_attention(vfkv_ctx *ctx, vfkv_workspace *ws, const AttnArgs &a, cudaStream_t st);
int32_t launch_merge_partials(vfkv_ctx *ctx, const float *m, const float *l, const float *o,
                              uint32_t n_parts, uint32_t n_rows, uint32_t head_dim, float *out,
                              cudaStream_t st);

int32_t launch_merge_partials_packed(vfkv_ctx *ctx, const float *packed, uint32_t n_parts, uint32_t n_rows,
                                     uint32_t head_dim, float *out, cudaStream_t st);

// prefill attention on tcgen05 (attn_prefill_tc5.cu); k / v point at the slot's rows of the layer
bool prefill_tc5_supported(uint32_t dtype, uint32_t head_dim, uint32_t group, bool has_scales);
// true when the tcgen05 kernel is expected to beat the 64-row mma.sync kernel on this chunk: enough
// 256-row blocks, or even shares of all K/V tiles over the SMs, or at least ten K/V tiles an item
bool prefill_tc5_pays(const vfkv_ctx *ctx, uint32_t n_q_heads, uint32_t n_kv_heads, uint32_t m, uint32_t q_start,
                      uint32_t n_kv, uint32_t kv_start, uint32_t window);
int32_t launch_prefill_tc5(vfkv_ctx *ctx, uint32_t dtype, const uint8_t *k, const uint8_t *v, const float *q, float *out,
                           uint64_t row_bytes, uint32_t n_q_heads, uint32_t n_kv_heads, uint32_t m, uint32_t q_start,
                           uint32_t n_kv, uint32_t kv_start, uint32_t window, float scale, float softcap,
                           cudaStream_t st);

// peer exchange of partials (exchange.cu)
int32_t launch_fanout_push(vfkv_ctx *ctx, const PeerFanout &fan, const float *staging, uint32_t head_dim,
                           cudaStream_t st);

// attention implementations
uint32_t choose_splits(const vfkv_ctx *ctx, const AttnArgs &a, uint32_t tile);
int32_t launch_attn_generic(vfkv_ctx *ctx, vfkv_workspace *ws, const AttnArgs &a, uint32_t n_splits,
                            cudaStream_t st);
bool attn_mma_supported(const AttnArgs &a);
bool encode_layer_maps(vfkv_ctx *ctx, const KvView &v, void *tm_k_out, void *tm_v_out);
int32_t launch_attn_mma(vfkv_ctx *ctx, vfkv_workspace *ws, const AttnArgs &a, uint32_t n_splits,
                        cudaStream_t st);
// merges ws partials [seq][head][split] into a.out (normalised) or a.out_{m,l,o}
int32_t launch_merge_ws(vfkv_ctx *ctx, vfkv_workspace *ws, const AttnArgs &a, uint32_t n_splits,
                        cudaStream_t st);

// vfkv_ctx::last_written_slab after a store whose destination is a raw pointer.
static const void *const kAnySlab = reinterpret_cast<const void *>(~uintptr_t(0));

// Sentinel of vk_shaders/flash_attn_split.comp:104 for masked scores.
constexpr float kMaskedScore = -1e30f;

}  // namespace vfkv

// One GPU's end of a peer exchange of partials (exchange.cu).
struct vfkv_exchange {
    vfkv_ctx *ctx = nullptr;
    vfkv::PeerFanout fan;          // base[], epoch pointer, world, rank, rows, groups
    uint32_t head_dim = 0;
    uint64_t *local = nullptr;     // this rank's buffer of tagged words
    uint64_t bytes = 0;
    uint32_t *ctl = nullptr;       // [0] completed exchanges, [1] merge ticket (never shared)
    vfkv::PeerFanout *d_fan = nullptr;   // device copy of `fan`, read by the attention kernel
    float *staging = nullptr;      // one block, for attention kernels that cannot fan out themselves
    bool imported[8] = {false, false, false, false, false, false, false, false};
    uint64_t wait_ns = 1000000000ull;
};
