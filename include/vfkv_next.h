/* vfkv_next.h -- entry points for the callers either side of the KV-cache hot path:
 * the decode attention routing, chunked-prefill causal attention over the cache, the fused
 * RoPE + append, and the host-side bookkeeping that moves the cache's length counter.
 * Same library and conventions as vfkv.h (status codes, caller's stream, device pointers
 * owned by the caller). */
#ifndef VFKV_NEXT_H
#define VFKV_NEXT_H

#include "vfkv.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- decode attention routing ---------------------------------------------------------- */

/* The single-workgroup shader vk_shaders/flash_attn.comp:110-212 (FlashAttn / FlashAttnFp16Kv /
 * FlashAttnFp8Kv, dispatched by run_scalar_attn, src/backend/vulkan/forward/runs.rs:776-821):
 * one pass over [kv_start, seq_len) with an online softmax, no scratch and no second dispatch.
 * Equal to vfkv_attend with n_splits = 1; needs no workspace. */
int32_t vfkv_flash_attn(vfkv_cache *cache, uint32_t layer, uint32_t kv_layer, const float *d_q,
                        float *d_out, uint32_t n_q_heads, uint32_t slot, uint32_t seq_len,
                        uint32_t kv_start, float scale, float softcap, void *stream);

/* Forward::run_scalar_attn (runs.rs:722-775): seq_len = position + 1; with FA_TILE = 64, two or
 * more tiles go to the split + reduce path (the split count is chosen by the library), fewer to
 * vfkv_flash_attn.  kv_layer and kv_start are the caller's gemma4_kv_read_layer /
 * gemma4_kv_start (vfkv_gemma4_kv_read_layer, vfkv_sliding_kv_start). */
int32_t vfkv_scalar_attn(vfkv_cache *cache, vfkv_workspace *ws, uint32_t layer, uint32_t kv_layer,
                         const float *d_q, float *d_out, uint32_t n_q_heads, uint32_t slot,
                         uint32_t position, uint32_t kv_start, float scale, float softcap,
                         void *stream);
/* 1 when vfkv_scalar_attn takes the split path at this position (runs.rs:766-775). */
uint32_t vfkv_scalar_attn_uses_split(uint32_t position);

/* ---- chunked-prefill causal attention over the cache ------------------------------------- */

/* vk_shaders/flash_attn_batch.comp:105-208 + Forward::run_flash_attn_batch (runs.rs:933-1010):
 * m queries d_q [m][n_q_heads][head_dim] f32 of one sequence; query i sits at position
 * q_start + i and attends over [kv_start, min(q_start + i + 1, n_kv)).  kv_start is one value
 * for the whole chunk, as in the reference (b_step_attention, executor/attention.rs:2215-2219,
 * uses the last query's window).  window != 0 (extension) applies the exact per-query bound
 * max(kv_start, q_start + i + 1 - window) instead.  d_out [m][n_q_heads][head_dim] f32.
 * The cache rows [0, n_kv) of `slot` must already hold the chunk (append precedes attention,
 * executor/attention.rs:2134-2190).
 * One or two kernel launches.  For head_dim 128, FP8 or F16 rows and long items the tcgen05
 * kernel may spread the work as even shares of K/V tiles over all SMs (vfkv_ctx_set_attn_tuning
 * in vfkv.h); the first such call on a context outside a stream capture allocates 39 MB of
 * device scratch (a synchronising cudaMalloc), owned and freed by the context. */
int32_t vfkv_attend_prefill(vfkv_cache *cache, uint32_t layer, uint32_t kv_layer, const float *d_q,
                            float *d_out, uint32_t n_q_heads, uint32_t slot, uint32_t m,
                            uint32_t q_start, uint32_t n_kv, uint32_t kv_start, uint32_t window,
                            float scale, float softcap, void *stream);

/* ---- fused RoPE + append -------------------------------------------------------------------- */

/* RoPE-NeoX parameters (vk_shaders/rope_funcs.glsl:73-107, host runs.rs:647-720):
 * theta_i = position * freq_base^(-2 i / n_dims) for pair (i, i + n_dims / 2); dims >= n_dims
 * pass through.  freq_scale multiplies the position (1.0 = none). */
typedef struct {
    uint32_t n_dims;       /* rotated dims per head (even, <= head_dim) */
    float freq_base;       /* e.g. 500000 */
    float freq_scale;
} vfkv_rope_params;

/* K rows are rotated at their positions and stored, V rows stored, in one launch
 * (executor/attention.rs:435-530 followed by :546-596 in the reference: rope dispatch, barrier,
 * two store dispatches).  d_k / d_v: [n_tokens][kv_heads][head_dim] f32, positions
 * base_pos .. base_pos + n_tokens - 1 of `slot`.  d_k_rot (nullable): receives the rotated K
 * rows in f32, for callers that still need them. */
int32_t vfkv_rope_append(vfkv_cache *cache, uint32_t layer, const float *d_k, const float *d_v,
                         uint32_t n_tokens, uint32_t slot, uint32_t base_pos,
                         const vfkv_rope_params *rope, float *d_k_rot, void *stream);
/* Decode batch: one token per sequence at positions[i] of slot_ids[i] (null: slot i). */
int32_t vfkv_rope_append_batch(vfkv_cache *cache, uint32_t layer, const float *d_k, const float *d_v,
                               const uint32_t *d_slot_ids, const uint32_t *d_positions,
                               uint32_t n_seqs, const vfkv_rope_params *rope, float *d_k_rot,
                               void *stream);
/* The same rotation for Q rows [n_rows][n_heads][head_dim] in place or into d_out; row r is
 * rotated at d_positions[r] (null: base_pos + r). */
int32_t vfkv_rope_neox(vfkv_ctx *ctx, const float *d_x, float *d_out, uint32_t n_rows,
                       uint32_t n_heads, uint32_t head_dim, const uint32_t *d_positions,
                       uint32_t base_pos, const vfkv_rope_params *rope, void *stream);

/* ---- bookkeeping around the cache --------------------------------------------------------- */

/* longest_common_prefix (src/server/state.rs:49-51). */
uint64_t vfkv_longest_common_prefix(const uint32_t *a, uint64_t n_a, const uint32_t *b, uint64_t n_b);

/* The "KV prepare" of ServerSession::generate_reuse (state.rs:199-229): with reuse != 0,
 * k = min(lcp(cached, full), n_full - 1); k == 0 or reuse == 0 resets the slot's counter, else
 * the counter becomes k and rows [0, k) are kept; the caller prefills full[k..] at base_pos k.
 * *start_pos receives k.  As in the reference, the environment variable VF_KV_REUSE_OVERSHOOT=n
 * (a test hook, state.rs:206-212) makes k overshoot the common prefix by n rows, bounded by
 * n_cached and n_full - 1, so that a test can show that a wrong reuse changes the cache. */
int32_t vfkv_kv_reuse_prepare(vfkv_cache *cache, uint32_t slot, const uint32_t *cached_tokens,
                              uint64_t n_cached, const uint32_t *full_tokens, uint64_t n_full,
                              int32_t reuse, uint32_t *start_pos);
/* kv_invalidate (state.rs:284-287): after a failed or cancelled generation. */
int32_t vfkv_kv_invalidate(vfkv_cache *cache, uint32_t slot);

/* compute_auto_ctx (src/server/auto_ctx.rs:107-141): min of (free - weights - reserve) /
 * kv_bytes_per_token, the model's maximum, a hardware cap and a sane cap, rounded down to a
 * multiple of 256 and floored at 512.  *bound: 0 VRAM, 1 model max, 2 hardware, 3 sane cap. */
int32_t vfkv_compute_auto_ctx(uint64_t free_bytes, uint64_t weight_bytes, uint64_t reserve_bytes,
                              uint64_t kv_bytes_per_token, uint32_t model_max_ctx, uint32_t hw_cap,
                              uint32_t sane_cap, uint32_t *ctx_out, uint32_t *bound,
                              uint64_t *avail_for_kv);

/* gemma4_kv_read_layer (src/backend/vulkan/forward/arch/gemma4.rs:27-49).  kv_source[i]:
 * 0 Own, 1 OwnAndPublishesSliding, 2 OwnAndPublishesFull, 3 SubscribesSliding, 4 SubscribesFull.
 * A subscriber reads the first layer that publishes its kind; everything else reads itself. */
uint32_t vfkv_gemma4_kv_read_layer(const uint32_t *kv_source, uint32_t n_layers, uint32_t layer);

#ifdef __cplusplus
}
#endif
#endif /* VFKV_NEXT_H */
