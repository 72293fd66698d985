/*
 * vfkv.h -- C ABI of libvfkv.so: VulkanForge's KV-cache hot path on NVIDIA B200
 * (sm_100a).  KV append (FP8 E4M3 / F16 / F32), the FP8->F16 cache read and
 * split-K GQA decode attention with its log-sum-exp merge.
 *
 * Each entry point cites the VulkanForge interface it stands in for, by the
 * file's path inside that project.  The reference-side binding (Rust `extern "C"`
 * block plus a `src/backend/cuda` module) lives under rust/ in this source tree.
 *
 * Conventions
 *   - Every function returns a vfkv_status (0 = OK) and never aborts; the text
 *     of the last failure on a context is available from vfkv_last_error().
 *   - All device work is enqueued on the caller's stream (a cudaStream_t passed
 *     as void*; NULL = the default stream).  Stream order replaces the pipeline
 *     barriers the reference records between these dispatches
 *     (src/backend/vulkan/forward/executor/attention.rs:554,583-596;
 *     src/backend/vulkan/forward/runs.rs:1541).
 *   - Pointers named d_* are device pointers, h_* host pointers.
 *   - The library does not advance sequence lengths inside append: the caller
 *     commits them after the step, as the reference does
 *     (src/backend/vulkan/forward/decode.rs:812, forward/prefill.rs:277).
 *   - A context and the objects made from it may be used from one thread at a
 *     time.
 */
#ifndef VFKV_H
#define VFKV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VFKV_ABI_VERSION 1

typedef enum {
    VFKV_OK = 0,
    VFKV_ERR_INVALID = 1,      /* bad argument (null, out of range, misaligned)          */
    VFKV_ERR_OVERFLOW = 2,     /* a size computation overflowed 64 bits                  */
    VFKV_ERR_OOM = 3,          /* device allocation failed                               */
    VFKV_ERR_CUDA = 4,         /* a CUDA runtime / driver call failed                    */
    VFKV_ERR_UNSUPPORTED = 5,  /* shape or dtype outside what the kernels cover          */
    VFKV_ERR_TIMEOUT = 6,      /* a bounded device-side wait gave up (see vfkv_ctx_poll) */
    VFKV_ERR_PRECISION = 7     /* refused by vfkv_guard_kv_precision                     */
} vfkv_status;

/* src/backend/vulkan/kv_cache.rs:42-74 (KvDtype; element_size 4 / 2 / 1) */
typedef enum { VFKV_F32 = 0, VFKV_F16 = 1, VFKV_F8 = 2 } vfkv_dtype;

/* FP8 scaling.  NONE is the reference's behaviour: kv_store_fp8.comp casts each
 * value directly and the readers dequantise without a scale
 * (vk_shaders/kv_store_fp8.comp:42-50, vk_shaders/flash_attn_split.comp:34-43).
 * PER_TOKEN_HEAD is an extension with no counterpart in the reference's KV
 * path: one f32 scale per (position, kv-head), computed with the recipe of the
 * reference's FP8 GEMM activation quantiser
 * (vk_shaders/mul_coopmat_fp8_native_bn32.comp:149-152,214). */
typedef enum { VFKV_SCALE_NONE = 0, VFKV_SCALE_PER_TOKEN_HEAD = 1 } vfkv_scale_mode;

typedef struct vfkv_ctx vfkv_ctx;
typedef struct vfkv_cache vfkv_cache;
typedef struct vfkv_workspace vfkv_workspace;
typedef struct vfkv_exchange vfkv_exchange;

/* src/backend/vulkan/kv_cache.rs:153-176 (KvCacheConfig) plus the two build-side
 * fields n_slots and scale_mode. */
typedef struct {
    uint32_t n_layers;
    uint32_t n_kv_heads;
    uint32_t head_dim;
    uint32_t max_seq_len;
    uint32_t dtype;                        /* vfkv_dtype */
    const uint32_t *per_layer_head_dim;    /* NULL, or n_layers entries */
    const uint32_t *per_layer_n_kv_heads;  /* NULL, or n_layers entries */
    uint32_t n_slots;                      /* independent sequences; 0 or 1 = the reference's single slab */
    uint32_t scale_mode;                   /* vfkv_scale_mode; must be NONE unless dtype is F8 */
} vfkv_cache_config;

/* ---------------------------------------------------------------------- */
/* context                                                                  */
/* ---------------------------------------------------------------------- */
/* Stands in for the VulkanDevice + PipelineRegistry pair every run_* helper
 * receives (src/backend/vulkan/forward/runs.rs:722-729). */
int32_t vfkv_ctx_create(int32_t device_ordinal, vfkv_ctx **out);
int32_t vfkv_ctx_destroy(vfkv_ctx *ctx);
const char *vfkv_last_error(const vfkv_ctx *ctx);   /* never NULL */
const char *vfkv_status_string(int32_t status);
uint32_t vfkv_abi_version(void);
/* Reads the device-side status word that bounded waits write into; clears it.
 * Returns VFKV_OK or VFKV_ERR_TIMEOUT.  Synchronises the given stream. */
int32_t vfkv_ctx_poll(vfkv_ctx *ctx, void *stream);

/* ---------------------------------------------------------------------- */
/* cache: allocation, layout, bookkeeping                                   */
/* ---------------------------------------------------------------------- */
/* KvCache::new (src/backend/vulkan/kv_cache.rs:224-338): two device buffers,
 * position-major [layer][slot][pos][kv_head][dim]; with one slot this is the
 * reference's [layer][pos][kv_head][dim].  Sizes use checked arithmetic
 * (:273-291) and overflow returns VFKV_ERR_OVERFLOW.  Unlike the reference the
 * dtype is an explicit field, not an environment variable (:85-101); see
 * vfkv_dtype_from_env. */
int32_t vfkv_cache_create(vfkv_ctx *ctx, const vfkv_cache_config *cfg, vfkv_cache **out);
/* KvCache::destroy (:496-499) */
int32_t vfkv_cache_destroy(vfkv_cache *cache);
/* KvCache::zero_fill (:357-376) and zero_layer (:384-407); asynchronous on `stream` */
int32_t vfkv_cache_zero_fill(vfkv_cache *cache, void *stream);
int32_t vfkv_cache_zero_layer(vfkv_cache *cache, uint32_t layer, void *stream);

/* KvCache::current_seq_len and reset() (:208,492-494), one counter per slot.
 * reset zeroes only the counter; cache bytes persist, as in the reference. */
int32_t vfkv_cache_reset(vfkv_cache *cache, uint32_t slot);
int32_t vfkv_cache_seq_len(const vfkv_cache *cache, uint32_t slot, uint32_t *out);
int32_t vfkv_cache_set_seq_len(vfkv_cache *cache, uint32_t slot, uint32_t seq_len);

/* Layout accessors (:412-490).  The *_bytes values are offsets into the K
 * buffer (identical for V).  With n_slots > 1, layer_offset_bytes is the start
 * of slot 0 of that layer and slot_offset_bytes the start of any slot. */
uint32_t vfkv_cache_head_dim_for(const vfkv_cache *cache, uint32_t layer);
uint32_t vfkv_cache_kv_heads_for(const vfkv_cache *cache, uint32_t layer);
uint64_t vfkv_cache_row_bytes(const vfkv_cache *cache, uint32_t layer);
uint64_t vfkv_cache_layer_size_bytes(const vfkv_cache *cache, uint32_t layer);
uint64_t vfkv_cache_layer_offset_bytes(const vfkv_cache *cache, uint32_t layer);
uint64_t vfkv_cache_layer_offset_elems(const vfkv_cache *cache, uint32_t layer);
uint64_t vfkv_cache_pos_offset_bytes(const vfkv_cache *cache, uint32_t layer, uint32_t pos);
uint64_t vfkv_cache_slot_offset_bytes(const vfkv_cache *cache, uint32_t layer, uint32_t slot);
uint64_t vfkv_cache_bytes_per_buffer(const vfkv_cache *cache);
uint32_t vfkv_cache_dtype(const vfkv_cache *cache);
int32_t  vfkv_cache_is_fp8(const vfkv_cache *cache);
int32_t  vfkv_cache_is_fp16(const vfkv_cache *cache);
/* public k_buffer / v_buffer fields (:205-206): raw device base pointers */
void *vfkv_cache_k_ptr(const vfkv_cache *cache);
void *vfkv_cache_v_ptr(const vfkv_cache *cache);
/* extension: [layer][slot][pos][kv_head] f32 scale planes, NULL when scale_mode is NONE */
float *vfkv_cache_k_scale_ptr(const vfkv_cache *cache);
float *vfkv_cache_v_scale_ptr(const vfkv_cache *cache);

/* free functions of kv_cache.rs */
/* kv_bytes_per_token (:186-202) */
uint64_t vfkv_kv_bytes_per_token(uint32_t n_layers, uint32_t n_kv_heads, uint32_t head_dim,
                                 const uint32_t *per_layer_head_dim,
                                 const uint32_t *per_layer_n_kv_heads, uint64_t elem_size);
/* KvDtype::element_size (:60-66) */
uint64_t vfkv_dtype_element_size(uint32_t dtype);
/* kv_dtype_from_env (:85-101): VULKANFORGE_KV_FP8=1|true -> F8, else
 * VULKANFORGE_FP16_KV=0 -> F32, else F16 */
uint32_t vfkv_dtype_from_env(void);
/* guard_kv_precision (:118-151); `force` is VULKANFORGE_ALLOW_BROKEN_KV */
int32_t vfkv_guard_kv_precision(int32_t is_gemma4_moe, uint32_t dtype, int32_t force);
/* gemma4_kv_start (src/backend/vulkan/forward/arch/gemma4.rs:59-73) for a sliding layer */
uint32_t vfkv_sliding_kv_start(uint32_t position, uint32_t sliding_window);

/* ---------------------------------------------------------------------- */
/* raw ops: the reference's dispatch level (buffers + push constants)        */
/* ---------------------------------------------------------------------- */
/* Forward::run_kv_store_fp8 (src/backend/vulkan/forward/runs.rs:2437-2478) +
 * vk_shaders/kv_store_fp8.comp: n_elements f32 -> E4M3 bytes at
 * d_dst + dst_byte_offset; offset 4-byte aligned (runs.rs:2448-2452); a ragged
 * tail is padded to a multiple of four with the code of 0.0. */
int32_t vfkv_kv_store_fp8(vfkv_ctx *ctx, const float *d_src, void *d_dst, uint32_t n_elements,
                          uint64_t dst_byte_offset, void *stream);
/* Forward::run_kv_copy_fp16 (runs.rs:2389-2430) + vk_shaders/kv_copy_fp16.comp */
int32_t vfkv_kv_copy_fp16(vfkv_ctx *ctx, const float *d_src, void *d_dst, uint32_t n_elements,
                          uint64_t dst_byte_offset, void *stream);
/* vk_shaders/kv_fp8_to_f16.comp, dispatched from run_flash_attn_cm_gemma_rs
 * (runs.rs:1103-1137): identity-indexed E4M3 -> binary16. */
int32_t vfkv_kv_fp8_to_f16(vfkv_ctx *ctx, const void *d_src, void *d_dst, uint64_t n_elements,
                           void *stream);

/* Forward::run_flash_attn_split_reduce (runs.rs:1463-1571) +
 * vk_shaders/flash_attn_split.comp + flash_attn_reduce.comp on raw buffers:
 * d_k / d_v point at one layer's slab [pos][kv_head][dim] of `dtype`
 * (the layer_offset_bytes binding of runs.rs:1475,1501-1502), d_q is
 * [n_heads][head_dim] f32, d_out likewise.  The push-constant fields of
 * FlashAttnSplitPushConstants (src/backend/vulkan/pipeline.rs:555-569) appear
 * as arguments; max_seq is the slab's row count.  n_splits replaces the
 * reference's fixed ceil(seq_len/64) partial count (0 = choose).  softcap is an
 * extension (0 = off = reference). */
int32_t vfkv_flash_attn_split_reduce(vfkv_ctx *ctx, vfkv_workspace *ws, const float *d_q,
                                     const void *d_k, const void *d_v, float *d_out,
                                     uint32_t dtype, uint32_t n_heads, uint32_t n_kv_heads,
                                     uint32_t head_dim, uint32_t seq_len, uint32_t max_seq,
                                     float scale, uint32_t kv_start, float softcap,
                                     uint32_t n_splits, void *stream);

/* The same attention on raw buffers for hosts that may not allocate device
 * memory while they run (an engine whose VRAM is one arena sized at start-up, a
 * latency-critical thread that cannot afford cudaMalloc's implicit device
 * synchronisation, a process whose memory budget belongs to someone else).  It
 * has no counterpart in the reference; it exists so such a host can use the
 * path without a vfkv_ctx or vfkv_workspace, both of which allocate.
 *   - The split-K scratch lives in a fixed device array inside the library
 *     (vfkv_noalloc_scratch_bytes(), about 2 MiB, held by every GPU that loads
 *     the library until the process exits).  The call is refused with
 *     VFKV_ERR_UNSUPPORTED when n_heads * n_splits * (head_dim + 2) exceeds
 *     524288 floats.  n_splits = 0 means 1.
 *   - No cudaMalloc, cudaFree or other allocating routine is called, here or in
 *     the kernels it launches.  It always runs the CUDA-core kernels.
 *   - It works on the calling thread's current device.  The first call on each
 *     device looks up the array's device address (a one-time set-up under a
 *     lock); make that first call outside any stream capture.
 *   - All calls on a device share the one array, which keeps the previous
 *     call's contents; the only word that must start at zero is cleared on the
 *     stream at the start of every call.  Two calls whose GPU work can overlap
 *     (different streams, or different threads) race on it: serialise them.
 *   - Errors: the return code, and vfkv_noalloc_last_error() for the text
 *     (per calling thread).  Every argument is a scalar checked on the host, so
 *     the device-side status word of the other entry points (out-of-range rows in
 *     device arrays, waits that ran out) has nothing to report on this path and
 *     there is nothing to poll: the word at the head of the array only exists
 *     because the kernels' parameter block wants a valid address. */
int32_t vfkv_flash_attn_split_reduce_noalloc(const float *d_q, const void *d_k, const void *d_v,
                                             float *d_out, uint32_t dtype, uint32_t n_heads,
                                             uint32_t n_kv_heads, uint32_t head_dim,
                                             uint32_t seq_len, uint32_t max_seq, float scale,
                                             uint32_t kv_start, float softcap, uint32_t n_splits,
                                             void *stream);
const char *vfkv_noalloc_last_error(void);
uint64_t vfkv_noalloc_scratch_bytes(void);

/* ---------------------------------------------------------------------- */
/* workspace: the split-K partials                                          */
/* ---------------------------------------------------------------------- */
/* fa_scratch_out / fa_scratch_max / fa_scratch_sum (src/backend/vulkan/forward/setup.rs:203-230),
 * one set per in-flight step.  Sized for max_seqs sequences x n_q_heads x
 * max_splits partials of head_dim floats. */
int32_t vfkv_workspace_create(vfkv_ctx *ctx, uint32_t max_seqs, uint32_t n_q_heads,
                              uint32_t head_dim, uint32_t max_splits, vfkv_workspace **out);
int32_t vfkv_workspace_destroy(vfkv_workspace *ws);
uint64_t vfkv_workspace_bytes(const vfkv_workspace *ws);
/* The tensor-core attention kernel merges its splits through the workspace without a second
 * launch.  Every CTA of a (sequence, kv-head) draws one ticket by adding 1 to a 64-bit word that
 * only ever counts up; there is one such word per split count, so ticket / n_splits is the number
 * of this launch on the word and ticket % n_splits the CTA's place in the draw.  Partials are
 * 8-byte words {f32 value, u32 tag} written by one store each, the tag made of a launch counter
 * kept by the host and the launch number on the word, and laid out by slice of the output rows so
 * that each of the last drawers (four; up to sixteen when a few kv-heads are cut into many splits)
 * finds its slice of every split in one block.  They accept only words that carry the tag of their own launch, waiting
 * at most the time set with vfkv_ctx_set_merge_wait_ms (a wait that runs out raises bit 1 (value 1) of
 * the status word).  Nothing is reset between launches, so a launch that gave up, a graph replay or
 * a change of geometry leaves nothing that a later launch could mistake for its own;
 * vfkv_workspace_reset puts tickets and tags back to zero, in stream order, for a host that
 * wants a known state after a kernel was killed from outside. */
int32_t vfkv_workspace_reset(vfkv_workspace *ws, void *stream);

/* ---------------------------------------------------------------------- */
/* cache-level ops: what the forward pass calls                             */
/* ---------------------------------------------------------------------- */
/* step_kv_write / b_step_kv_write (executor/attention.rs:546-596,2134-2190):
 * store n_tokens consecutive tokens of one sequence, f32
 * [n_tokens][kv_heads_for(layer)][head_dim_for(layer)], at positions
 * base_pos .. base_pos+n_tokens-1 of `slot`.  Both K and V in one launch.
 * Writing below the committed length overwrites (prefix reuse,
 * src/server/state.rs:199-229). */
int32_t vfkv_append(vfkv_cache *cache, uint32_t layer, const float *d_k, const float *d_v,
                    uint32_t n_tokens, uint32_t slot, uint32_t base_pos, void *stream);
/* The same chunk on a cache sharded by position (the plan of vfkv_shard_owner below): base_pos is
 * the global position of the first token; the rows whose page this rank owns are stored at their
 * local positions, the others are skipped -- one launch per chunk whatever the page size.  The
 * cache's max_seq_len is the rank's local capacity. */
int32_t vfkv_append_sharded(vfkv_cache *cache, uint32_t layer, const float *d_k, const float *d_v,
                            uint32_t n_tokens, uint32_t slot, uint32_t base_pos, uint32_t world,
                            uint32_t page, uint32_t rank, void *stream);
/* One token for each of n_seqs sequences: d_k/d_v are [n_seqs][kv_heads][head_dim],
 * d_slot_ids (NULL = 0..n_seqs-1) and d_positions are device arrays. */
int32_t vfkv_append_batch(vfkv_cache *cache, uint32_t layer, const float *d_k, const float *d_v,
                          const uint32_t *d_slot_ids, const uint32_t *d_positions,
                          uint32_t n_seqs, void *stream);

/* run_flash_attn_cm_gemma_rs' convert pre-pass (runs.rs:1103-1137): positions
 * [0, n_positions) of one layer of one slot, K and V, into caller buffers of
 * n_positions*kv_heads*head_dim halfs each (the k_f16_scratch / v_f16_scratch
 * of setup.rs:366-373). */
int32_t vfkv_fp8_to_f16(vfkv_cache *cache, uint32_t slot, uint32_t layer, uint32_t n_positions,
                        void *d_k_out, void *d_v_out, void *stream);

/* step_attention -> run_scalar_attn (runs.rs:722-821): decode attention of one
 * query token over positions [kv_start, seq_len) of kv_layer's slab
 * (kv_layer != layer only for Gemma-4 KV sharing, gemma4.rs:27-49).
 * d_q, d_out: [n_q_heads][head_dim_for(layer)] f32.  scale is explicit because
 * the reference's rule is per model (runs.rs:1483-1489).  Every seq_len >= 1
 * takes the same kernels, including the <= 64-token case the reference routes
 * to flash_attn.comp (runs.rs:766-821). */
int32_t vfkv_attend(vfkv_cache *cache, vfkv_workspace *ws, uint32_t layer, uint32_t kv_layer,
                    const float *d_q, float *d_out, uint32_t n_q_heads, uint32_t slot,
                    uint32_t seq_len, uint32_t kv_start, float scale, float softcap,
                    uint32_t n_splits, void *stream);
/* n_seqs independent sequences: d_q, d_out [n_seqs][n_q_heads][head_dim];
 * d_slot_ids (NULL = 0..n_seqs-1), d_seq_lens, d_kv_starts (NULL = 0) on device.
 * max_seq_len_hint bounds the largest seq_len (0 = the cache's max_seq_len) and
 * only steers the split count. */
int32_t vfkv_attend_batch(vfkv_cache *cache, vfkv_workspace *ws, uint32_t layer,
                          uint32_t kv_layer, const float *d_q, float *d_out, uint32_t n_q_heads,
                          const uint32_t *d_slot_ids, const uint32_t *d_seq_lens,
                          const uint32_t *d_kv_starts, uint32_t n_seqs,
                          uint32_t max_seq_len_hint, float scale, float softcap,
                          uint32_t n_splits, void *stream);

/* KvWrite followed by Attention, the order of the layer plan
 * (src/backend/vulkan/forward/layer_plan.rs:472-483), for one token per
 * sequence: append at d_positions[i], attend over
 * [kv_start_i, d_positions[i]+1).  window 0 = full history, else the sliding
 * rule of gemma4.rs:59-73. */
int32_t vfkv_decode_step(vfkv_cache *cache, vfkv_workspace *ws, uint32_t layer,
                         const float *d_q, const float *d_k, const float *d_v, float *d_out,
                         uint32_t n_q_heads, const uint32_t *d_slot_ids,
                         const uint32_t *d_positions, uint32_t n_seqs,
                         uint32_t max_seq_len_hint, uint32_t window, float scale,
                         float softcap, uint32_t n_splits, void *stream);

/* The decode step for every layer of one token, device buffers: d_q, d_out
 * [n_layers][n_seqs][n_q_heads][D]; d_k, d_v [n_layers][n_seqs][kv_heads][D].  One call records
 * what record_decode_dispatches (src/backend/vulkan/forward/decode.rs:43-82) records for this
 * path: per layer, KvWrite then Attention.  windows: NULL, or n_layers host entries (0 = global
 * layer).  Uniform-shape caches only.  Nothing in it synchronises or allocates, so a caller may
 * capture it in a CUDA graph (after one warm-up call) and replay it per token: positions and
 * slot ids are read from device memory at run time. */
int32_t vfkv_decode_token(vfkv_cache *cache, vfkv_workspace *ws, const float *d_q, const float *d_k,
                          const float *d_v, float *d_out, uint32_t n_q_heads,
                          const uint32_t *d_slot_ids, const uint32_t *d_positions, uint32_t n_seqs,
                          uint32_t max_seq_len_hint, const uint32_t *windows, float scale,
                          float softcap, uint32_t n_splits, void *stream);

/* Same step for every layer of one token with HOST buffers: copies
 * h_q [n_layers][n_seqs][n_q_heads][D], h_k, h_v [n_layers][n_seqs][kv_heads][D]
 * to the device, runs the layers in order, copies h_out
 * [n_layers][n_seqs][n_q_heads][D] back and waits.  Uniform-shape caches only.
 * h_positions / h_slot_ids (NULL = identity) are host arrays of n_seqs.
 * windows: NULL, or n_layers entries (0 = global layer).  This is the
 * forward_token boundary (src/backend/vulkan/forward/decode.rs:567-626) reduced
 * to the hot path.  On a non-default stream the layers run as up to four cached
 * CUDA graphs, and a second stream owned by the workspace copies the next
 * group's inputs and the previous group's outputs while a group computes; the
 * call returns when h_out is complete.  Pinned host buffers make the copies
 * asynchronous. */
int32_t vfkv_decode_token_host(vfkv_cache *cache, vfkv_workspace *ws, const float *h_q,
                               const float *h_k, const float *h_v, float *h_out,
                               uint32_t n_q_heads, const uint32_t *h_slot_ids,
                               const uint32_t *h_positions, uint32_t n_seqs,
                               const uint32_t *windows, float scale, float softcap,
                               uint32_t n_splits, void *stream);

/* The same step without waiting, for two tokens in flight: the counterpart of pre_record /
 * fill_embed_and_submit / wait_and_read_logits with their two command-buffer / fence pairs and
 * per-slot scratch (src/backend/vulkan/forward/decode.rs:169-259, forward/setup.rs:203-230).
 * submit enqueues the input copies (a stream of the workspace), the layers (one recorded CUDA
 * graph per staging set, on `stream`, which must not be the default stream) and the output copy
 * (another stream of the workspace), and returns a ticket at once; wait blocks until that
 * token's h_out is complete.  Arguments as vfkv_decode_token_host.  At most two tickets are in
 * flight (VFKV_ERR_INVALID for a third); the host buffers of a ticket must stay untouched until
 * its wait returns, and should be pinned.  The layers of consecutive submits run in submit order
 * on `stream`, so the cache sees the tokens in order; the copies of one token overlap the layers
 * of the other. */
int32_t vfkv_decode_token_host_submit(vfkv_cache *cache, vfkv_workspace *ws, const float *h_q,
                                      const float *h_k, const float *h_v, float *h_out,
                                      uint32_t n_q_heads, const uint32_t *h_slot_ids,
                                      const uint32_t *h_positions, uint32_t n_seqs,
                                      const uint32_t *windows, float scale, float softcap,
                                      uint32_t n_splits, void *stream, uint64_t *ticket);
int32_t vfkv_decode_token_host_wait(vfkv_workspace *ws, uint64_t ticket);

/* ---------------------------------------------------------------------- */
/* sequence-dimension sharding (no counterpart in the reference, which is    */
/* single-GPU): local partials and the merge of flash_attn_reduce.comp:51-80 */
/* ---------------------------------------------------------------------- */
/* Attention over positions [pos_begin, pos_end) only, unnormalised:
 * d_m, d_l [n_seqs][n_q_heads], d_o [n_seqs][n_q_heads][head_dim] with
 * o = sum exp(s - m) v.  An empty range gives m = -1e30, l = 0, o = 0. */
int32_t vfkv_attend_partial(vfkv_cache *cache, vfkv_workspace *ws, uint32_t layer,
                            uint32_t kv_layer, const float *d_q, uint32_t n_q_heads,
                            uint32_t slot, uint32_t pos_begin, uint32_t pos_end, float scale,
                            float softcap, uint32_t n_splits, float *d_m, float *d_l,
                            float *d_o, void *stream);
/* The partial of this rank's positions, an all-gather of every rank's partial, and the merge, in
 * one call, for a host that already holds an NCCL communicator over its GPUs: nccl_comm is its
 * ncclComm_t; d_packed is scratch of world * n_q_heads * (head_dim + 2) floats (block r = rank r's
 * m[rows], l[rows], o[rows][head_dim]); d_out [n_q_heads][head_dim] is complete on every rank.
 * ncclAllGather is resolved at run time in the NCCL the process has loaded (VFKV_ERR_UNSUPPORTED if
 * there is none); this library links no collective library itself.  Three launches and the
 * collective's latency: the peer exchange further down (vfkv_attend_exchange) is the fast path. */
int32_t vfkv_attend_allgather(vfkv_cache *cache, vfkv_workspace *ws, void *nccl_comm, uint32_t world,
                              uint32_t rank, uint32_t layer, uint32_t kv_layer, const float *d_q,
                              uint32_t n_q_heads, uint32_t slot, uint32_t pos_begin, uint32_t pos_end,
                              float scale, float softcap, uint32_t n_splits, float *d_packed,
                              float *d_out, void *stream);
/* d_m, d_l: [n_parts][n_rows]; d_o: [n_parts][n_rows][head_dim];
 * d_out: [n_rows][head_dim]; n_rows = sequences x q-heads. */
int32_t vfkv_merge_partials(vfkv_ctx *ctx, const float *d_m, const float *d_l, const float *d_o,
                            uint32_t n_parts, uint32_t n_rows, uint32_t head_dim, float *d_out,
                            void *stream);

/* The same merge over the buffer an all-gather of per-GPU partials produces: n_parts blocks of
 * n_rows*(head_dim+2) floats, each block m[n_rows], l[n_rows], o[n_rows][head_dim]. */
int32_t vfkv_merge_partials_packed(vfkv_ctx *ctx, const float *d_packed, uint32_t n_parts,
                                   uint32_t n_rows, uint32_t head_dim, float *d_out, void *stream);

/* ---- the sharding plan (host arithmetic only; no counterpart in the reference) ----------------
 *
 * By position: global position p of a sequence is held by rank (p / page) % world at local position
 * ((p / page) / world) * page + p % page, so appends rotate over the GPUs and every rank's share of
 * any context differs by at most one page.  local_len = how many of the positions [0, seq_len) a
 * rank holds (they occupy its local rows [0, local_len)); local_capacity = rows a rank's slab needs
 * for contexts up to max_seq_len.  world and page must be non-zero (0 is returned otherwise). */
uint32_t vfkv_shard_owner(uint32_t world, uint32_t page, uint64_t pos);
uint64_t vfkv_shard_local_pos(uint32_t world, uint32_t page, uint64_t pos);
uint64_t vfkv_shard_local_len(uint32_t world, uint32_t page, uint64_t seq_len, uint32_t rank);
uint64_t vfkv_shard_local_capacity(uint32_t world, uint32_t page, uint64_t max_seq_len);
/* By sequence: longest-first greedy balancing of n sequences over `world` ranks by context length
 * (ties: lower sequence index first, lower rank first); owner_out[i] = rank that owns sequence i. */
int32_t vfkv_assign_sequences(const uint32_t *lengths, uint32_t n, uint32_t world, uint32_t *owner_out);
/* By kv-head group: rank r of `world` owns kv-heads [first, first + count) and the q-heads
 * [first * g, (first + count) * g) that read them (the kvh = h / g mapping of
 * vk_shaders/flash_attn_split.comp:83-95); outputs are disjoint head slices, no exchange.  The
 * heads are dealt as evenly as n_kv_heads allows. */
int32_t vfkv_shard_kv_heads(uint32_t world, uint32_t rank, uint32_t n_kv_heads, uint32_t *first,
                            uint32_t *count);

/* ---- peer exchange of partials (position sharding without a library collective) -----------
 *
 * No counterpart in the reference.  Each GPU of the group owns one exchange buffer of 8-byte words
 * {f32 value, u32 tag}.  The attention kernel of vfkv_attend_push stores this GPU's (m, l, o)
 * block into the buffer of EVERY rank with plain peer stores, each word tagged with the number of
 * the exchange (8-byte accesses are single-copy atomic, so a reader that finds the tag has the
 * value: no flags, no fences).  vfkv_exchange_merge polls the words of all ranks in its own
 * buffer -- at most the time set with vfkv_exchange_set_timeout_ms (default 1000 ms); a wait that
 * runs out sets bit 8 of the status word read by vfkv_ctx_poll and writes zeros -- and applies the
 * flash_attn_reduce.comp:51-80 merge.  Blocks are double-buffered by the parity of a device-side
 * exchange counter, so the calls can be captured in a CUDA graph and replayed.  Every rank must
 * make the same sequence of exchanges: one vfkv_exchange_merge per vfkv_attend_push, or
 * vfkv_attend_exchange alone.  vfkv_attend_exchange does both steps in ONE launch where the
 * tensor-core kernel covers the shape: the CTA that has merged a kv-head's splits stores the block
 * to every rank, then polls its own buffer for the other ranks' words of the same rows and writes
 * the final rows.  That needs the ranks' kernels to run at the same time, i.e. one GPU per rank;
 * ranks that share a GPU (tests) use the two-call form, whose producers all run first.
 *
 * Set-up: create on every rank with the same shape; make each rank's buffer known to the others,
 * either through vfkv_exchange_export / vfkv_exchange_import (CUDA IPC handles, one process per
 * GPU) or vfkv_exchange_set_peer (pointers the caller has mapped itself, or several ranks of one
 * process); synchronise the ranks once (the buffers are zeroed by create) before the first push.
 * world <= 8; n_rows = q-heads of the sequence; head_dim a multiple of 4. */
int32_t vfkv_exchange_create(vfkv_ctx *ctx, uint32_t world, uint32_t rank, uint32_t n_rows,
                             uint32_t head_dim, vfkv_exchange **out);
void vfkv_exchange_destroy(vfkv_exchange *ex);
uint64_t vfkv_exchange_bytes(const vfkv_exchange *ex);
void *vfkv_exchange_local_ptr(const vfkv_exchange *ex);
int32_t vfkv_exchange_export(vfkv_exchange *ex, uint8_t handle[64]);
int32_t vfkv_exchange_import(vfkv_exchange *ex, uint32_t rank, const uint8_t handle[64]);
int32_t vfkv_exchange_set_peer(vfkv_exchange *ex, uint32_t rank, void *d_peer_buffer);
int32_t vfkv_exchange_set_timeout_ms(vfkv_exchange *ex, uint32_t ms);
/* 1 once every rank's buffer is known. */
uint32_t vfkv_exchange_ready(const vfkv_exchange *ex);
/* Attention of one query token over local positions [pos_begin, pos_end) of `slot`, the partial
 * delivered to every rank (arguments as vfkv_attend_partial).  d_k_new / d_v_new: null, or -- on
 * the rank that owns the new token -- its K and V rows [kv_heads][head_dim] f32, stored at local
 * position pos_end - 1 before the attention reads it (KvWrite + Attention of one layer in one
 * launch where the tensor-core kernel covers the shape). */
int32_t vfkv_attend_push(vfkv_cache *cache, vfkv_workspace *ws, vfkv_exchange *ex, uint32_t layer,
                         uint32_t kv_layer, const float *d_q, const float *d_k_new,
                         const float *d_v_new, uint32_t n_q_heads, uint32_t slot,
                         uint32_t pos_begin, uint32_t pos_end, float scale, float softcap,
                         uint32_t n_splits, void *stream);
/* Waits for all ranks' blocks of the current exchange and writes d_out [n_rows][head_dim]. */
int32_t vfkv_exchange_merge(vfkv_exchange *ex, float *d_out, void *stream);
/* vfkv_attend_push and vfkv_exchange_merge as one step (one launch where the tensor-core kernel
 * covers the shape and d_out is 16-byte aligned, else the two calls in a row). */
int32_t vfkv_attend_exchange(vfkv_cache *cache, vfkv_workspace *ws, vfkv_exchange *ex,
                             uint32_t layer, uint32_t kv_layer, const float *d_q,
                             const float *d_k_new, const float *d_v_new, uint32_t n_q_heads,
                             uint32_t slot, uint32_t pos_begin, uint32_t pos_end, float scale,
                             float softcap, uint32_t n_splits, float *d_out, void *stream);

/* ---------------------------------------------------------------------- */
/* device-memory helpers for hosts without a CUDA binding of their own       */
/* ---------------------------------------------------------------------- */
int32_t vfkv_malloc(vfkv_ctx *ctx, uint64_t bytes, void **d_out);
int32_t vfkv_free(vfkv_ctx *ctx, void *d_ptr);
int32_t vfkv_malloc_host(vfkv_ctx *ctx, uint64_t bytes, void **h_out);   /* pinned */
int32_t vfkv_free_host(vfkv_ctx *ctx, void *h_ptr);
int32_t vfkv_memcpy_h2d(vfkv_ctx *ctx, void *d_dst, const void *h_src, uint64_t bytes, void *stream);
int32_t vfkv_memcpy_d2h(vfkv_ctx *ctx, void *h_dst, const void *d_src, uint64_t bytes, void *stream);
int32_t vfkv_memset(vfkv_ctx *ctx, void *d_dst, int32_t byte, uint64_t bytes, void *stream);
int32_t vfkv_stream_synchronize(vfkv_ctx *ctx, void *stream);

/* ---------------------------------------------------------------------- */
/* profiling hooks: the ShaderProfiler labels (src/backend/vulkan/profiler.rs:28-187) */
/* ---------------------------------------------------------------------- */
/* Selects the attention implementation for subsequent calls on this context:
 * 0 = automatic, 1 = CUDA-core kernel only, 2 = tensor-core kernel only
 * (VFKV_ERR_UNSUPPORTED from attend when the shape is outside it), 3 = automatic, but
 * vfkv_attend_prefill takes its mma.sync kernel where it would take the tcgen05 one. */
int32_t vfkv_ctx_set_attn_impl(vfkv_ctx *ctx, uint32_t impl);
/* Shape of the tensor-core attention kernel for subsequent calls: warps per CTA x TMA stages per
 * warp; 4x1, 4x2, 4x3, 8x1 or 8x3, 0x0 = choose per call (4 warps, or 8x3 when the grid has at most
 * one CTA per SM).  The reference has fixed workgroup shapes; this is a measurement knob.  The
 * stage count also picks the form of the tcgen05 prefill kernel of vfkv_attend_prefill: 1 the
 * simple one, 2 the pipelined one, 3 the one with the roles on separate warps (F16 rows by TMA
 * when the driver offers tensor maps), 0 = the last (the pipelined one for F16 caches without
 * tensor maps).  The specialised form runs either one CTA per
 * (kv-head, block of 256 rows) item -- always with 4x3 -- or one CTA per SM, each taking an even
 * share of all items' K/V tiles -- with 8x3 whenever the call allows it (every query sees at
 * least one position, at most 512 row blocks, at least 8 tiles a share), with 0x0 when in
 * addition one CTA per item would leave a twentieth of the SM time unused and an item averages 96
 * tiles or more, or the items are at most half the SMs and the shares are ten tiles shorter than
 * the longest item.  Items cut between CTAs
 * are put together by the CTA holding the item's head (a cooperative launch, at most four
 * pieces an item, not inside a stream capture) or by a small second kernel.  The shares need
 * 39 MB of device scratch, which the context allocates at the first such call outside a stream
 * capture and frees in vfkv_ctx_destroy; calls that would use it must not run concurrently on
 * two streams of one context. */
int32_t vfkv_ctx_set_attn_tuning(vfkv_ctx *ctx, uint32_t warps, uint32_t stages);
/* Programmatic dependent launch of the tensor-core attention kernel, the CUDA counterpart of
 * relaxing the full pipeline barrier the reference records between dispatches
 * (src/backend/vulkan/forward/runs.rs:1541, executor/attention.rs:583-596) to the buffers that
 * really depend on one another.
 *   0  off: a kernel starts when the previous work in the stream has finished (default).
 *   1  the kernel may be scheduled while its predecessor in the stream drains; it waits for the
 *      predecessor before it reads or writes any global memory.  Always safe.
 *   2  as 1, but it reads the position / slot arrays and prefetches this layer's K/V rows before
 *      that wait.  The caller promises that the kernel enqueued immediately before on the stream
 *      writes neither those arrays nor this layer's cache rows (true for consecutive layers of a
 *      decode step, and for a forward pass whose preceding kernel is a projection or RoPE).
 *      Only that one kernel matters: a mode-2 kernel releases its successor after its own wait,
 *      so an early prefetch never overlaps anything older than the direct predecessor.  When the
 *      direct predecessor was launched through this context and wrote rows of the slab this call
 *      reads (the same layer twice in a row, a subscriber layer right after its publisher's
 *      append, any raw store), the library itself falls back to mode 1 for that launch.
 *      Q, the token to append and all outputs are still touched only after the wait. */
int32_t vfkv_ctx_set_dependent_launch(vfkv_ctx *ctx, uint32_t mode);
/* Latency analysis of the tensor-core attention kernel: while d_buffer is non-NULL, thread 0 of
 * every CTA stores 16 x uint64 nanosecond timestamps (globaltimer) at fixed phases -- 0 entry,
 * 1 range known, 2 barriers ready, 3 Q ready, 4 first tile landed, 5 stream done, 6 CTA joined,
 * 7 partial stored, 8 splits merged, 9 rows written, 10 every split's partial seen, 11 first round of
 * copies staged (8, 10 and 11: merging CTAs only) -- at CTA index * 16.  The buffer
 * must hold 16 x 8 bytes per CTA of the largest grid.  NULL switches it off.
 * The tcgen05 prefill kernel (vfkv_attend_prefill) uses the same buffer: thread 0 of each of its
 * two warpgroups stores, at its 4th K/V tile, 0 tile start, 1 loads issued and previous P V
 * complete, 2 K/V converted, 3 CTA barrier passed, 4 S issued, 5 S complete, 6 row maximum,
 * 7 rescale decided, 8 P written, 9 P V issued -- at (CTA index * 2 + warpgroup) * 16.  Its
 * specialised form stores 32 slots per CTA at its 4th tile: 0 and 12 the MMA thread
 * (tile top, all of the tile's products issued); 16-23 thread 0 of the softmax
 * warps (tile top; per half: S there, maximum known, P handed over); 24-26 the first K/V thread
 * (tile top, K placed, V placed); and once per CTA, for its first item or share segment, by thread
 * 0: 13 start, 14 Q placed, 15 first S there, 27 last tile's softmax done, 28 last P V complete,
 * 29 rows written. */
/* Split merge inside a thread-block cluster (tensor-core kernel, 2..16 splits): the CTAs of one
 * (sequence, kv-head) exchange their partials through distributed shared memory instead of
 * global scratch and a ticket.  Taken only when every cluster of the grid can be resident at
 * once; otherwise the call falls back to the scratch + ticket form.  0 = off (default), 1 = on. */
int32_t vfkv_ctx_set_cluster_merge(vfkv_ctx *ctx, uint32_t on);
/* Time limit of the merging CTA's wait for the other splits' partials, and of the prefill kernel's
 * wait for the other pieces of an item cut between CTAs (1..10000 ms, default 1000). */
int32_t vfkv_ctx_set_merge_wait_ms(vfkv_ctx *ctx, uint32_t ms);
/* Host-side failure injection for tests of the bounded waits: in later launches of the tensor-core
 * attention kernel the CTA of (sequence 0, kv-head 0, split `split`) behaves as if its wait for a
 * TMA tile had run out -- it raises bit 1 of the status word and publishes no partial -- so the
 * merging CTA's own wait runs out as well.  In the prefill kernel's even-shares form the CTA with
 * index `split` does not announce its piece of a cut item, so the wait of the CTA that holds the
 * item's head runs out (status bit 1, that item's rows are zeros).  Nothing faults or hangs.
 * 0xFFFFFFFF = off (default). */
int32_t vfkv_ctx_debug_fail_split(vfkv_ctx *ctx, uint32_t split);
int32_t vfkv_ctx_set_trace_buffer(vfkv_ctx *ctx, void *d_buffer);
/* With n_blocks > 1 the k-th launch of the decode attention kernel after this call (or after the
 * buffer was set) writes block k % n_blocks of the buffer, a block being 16 x 8 bytes per CTA of
 * that launch's grid: the phases of consecutive layers of one token side by side, on the GPU's
 * common nanosecond clock.  The blocks of one ring must belong to launches with equal grids. */
int32_t vfkv_ctx_set_trace_ring(vfkv_ctx *ctx, uint32_t n_blocks);
/* Kernels this context has launched since creation (for launch accounting). */
uint64_t vfkv_ctx_launch_count(const vfkv_ctx *ctx);

/* Per-kernel GPU timing with the reference's profiler labels
 * (executor/attention.rs:560-573, runs.rs:1527,1561,1127; enabled there by
 * VF_GPU_TIMER).  While enabled every kernel launch is bracketed by a pair of
 * CUDA events on its stream.  Labels: */
typedef enum {
    VFKV_PROF_KV_STORE = 0,      /* kv_store_fp8_k/_v, kv_copy_fp16_k/_v (one launch covers K and V) */
    VFKV_PROF_FP8_TO_F16 = 1,    /* fa_cm_rs_cvt */
    VFKV_PROF_FA_SPLIT = 2,      /* fa_split */
    VFKV_PROF_FA_REDUCE = 3,     /* fa_reduce */
    VFKV_PROF_LABELS = 4
} vfkv_prof_label;
int32_t vfkv_profile_enable(vfkv_ctx *ctx, int32_t on);
/* Waits for the recorded events, returns count / total / minimum milliseconds of
 * one label and, when `reset` is non-zero, forgets all records of every label. */
int32_t vfkv_profile_collect(vfkv_ctx *ctx, uint32_t label, uint64_t *count, double *total_ms,
                             double *min_ms, int32_t reset);

#ifdef __cplusplus
}
#endif
#endif /* VFKV_H */
