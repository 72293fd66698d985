/*
 * vfkv_oracle.h -- CPU restatement of VulkanForge's KV-cache hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This is the checker the CUDA library is compared
 * against (and the timed CPU baseline).  Nothing in the product package links
 * or loads it; only the test-suite, the smoke check and the benchmark's CPU leg
 * do.
 *
 * Parity status:
 *   - E4M3 codec: pinned against the reference's known-answer tests
 *     (src/backend/vulkan/fp8_ext.rs:225-263).
 *   - Cache layout arithmetic: pinned against the integers asserted in
 *     src/backend/vulkan/kv_cache.rs:519-586.
 *   - Attention: restates tests/correctness.rs:2567-2617 (the reference's own
 *     CPU attention, f64 accumulators); pinned by the reference's analytic
 *     cases (seq_len 1 => out == V, tests/correctness.rs:1003-1123; constant
 *     K/V at a non-zero layer offset, :899-998) and by the tiled == naive
 *     property (tests/flash_attn_tiled_ref.rs:238-303).
 *   - F16 store rounding: PARITY UNPINNED in the reference (packHalf2x16 is
 *     driver-defined, vk_shaders/kv_copy_fp16.comp:50); this file uses
 *     round-to-nearest-even like the reference's tests do through the `half`
 *     crate (tests/coopmat_fa_gemma.rs:74,212).
 *   - The Rust reference cannot be compiled in this environment (no rustc /
 *     cargo), so there is no machine-made output of the reference itself.
 */
#ifndef VFKV_ORACLE_H
#define VFKV_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of the cache, numbering shared with include/vfkv.h */
enum { VFO_F32 = 0, VFO_F16 = 1, VFO_F8 = 2 };

/* ---- scalar codecs ---------------------------------------------------- */
uint8_t  vfo_f32_to_e4m3(float x);
float    vfo_e4m3_to_f32(uint8_t b);
uint16_t vfo_f32_to_f16(float x);
float    vfo_f16_to_f32(uint16_t h);

/* bulk forms (OpenMP) used by the exhaustive converter sweeps */
void vfo_f32_bits_to_e4m3_range(uint32_t first_bits, uint64_t count, uint8_t *dst);
void vfo_f32_bits_to_f16_range(uint32_t first_bits, uint64_t count, uint16_t *dst);

/* ---- append / convert ops --------------------------------------------- */
/* writes 4*ceil(n/4) bytes */
void vfo_kv_store_fp8(const float *src, uint32_t n_elements, uint8_t *dst);
/* writes 2*ceil(n/2) halfs */
void vfo_kv_copy_fp16(const float *src, uint32_t n_elements, uint16_t *dst);
void vfo_kv_fp8_to_f16(const uint8_t *src, uint32_t n_elements, uint16_t *dst);
/* extension: per-(token, kv-head) absmax scale; writes n_heads scales and
 * n_heads*head_dim bytes */
void vfo_kv_store_fp8_scaled(const float *src, uint32_t n_heads, uint32_t head_dim,
                             uint8_t *dst, float *scales);

/* ---- cache layout ------------------------------------------------------ */
typedef struct {
    uint32_t n_layers, n_kv_heads, head_dim, max_seq_len;
    uint32_t dtype;                         /* VFO_F32 / VFO_F16 / VFO_F8 */
    const uint32_t *per_layer_head_dim;     /* NULL or n_layers entries */
    const uint32_t *per_layer_n_kv_heads;   /* NULL or n_layers entries */
} vfo_layout;

uint64_t vfo_elem_size(uint32_t dtype);
uint32_t vfo_head_dim_for(const vfo_layout *c, uint32_t layer);
uint32_t vfo_kv_heads_for(const vfo_layout *c, uint32_t layer);
uint64_t vfo_row_bytes(const vfo_layout *c, uint32_t layer);
uint64_t vfo_layer_size_bytes(const vfo_layout *c, uint32_t layer);
uint64_t vfo_layer_offset_bytes(const vfo_layout *c, uint32_t layer);
uint64_t vfo_pos_offset_bytes(const vfo_layout *c, uint32_t layer, uint32_t pos);
/* returns 0 and writes *bytes, or -1 on overflow */
int      vfo_bytes_per_buffer(const vfo_layout *c, uint64_t *bytes);
uint64_t vfo_kv_bytes_per_token(uint32_t n_layers, uint32_t n_kv_heads, uint32_t head_dim,
                                const uint32_t *per_layer_head_dim,
                                const uint32_t *per_layer_n_kv_heads, uint64_t elem_size);
uint32_t vfo_sliding_kv_start(uint32_t position, uint32_t window);

/* ---- RoPE (input preparation) ------------------------------------------ */
void vfo_rope_neox(float *x, uint32_t n_heads, uint32_t head_dim, uint32_t n_dims,
                   uint32_t pos, float freq_base);

/* ---- attention ---------------------------------------------------------- */
/* k, v: one layer's slab for one sequence, [pos][kv_head][dim] in `dtype`.
 * k_scales / v_scales: NULL, or [pos][kv_head] f32 multipliers (extension).
 * softcap 0 => none. */
void vfo_attention_ref(const float *q, const void *k, const void *v, uint32_t dtype,
                       uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                       uint32_t seq_len, uint32_t kv_start, float scale, float softcap,
                       const float *k_scales, const float *v_scales, float *out);

/* the two shaders, f32 arithmetic in shader order; tile = positions per partial */
void vfo_flash_attn_split(const float *q, const void *k, const void *v, uint32_t dtype,
                          uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                          uint32_t seq_len, uint32_t kv_start, float scale, uint32_t tile,
                          uint32_t n_tiles, float *scratch_out, float *scratch_max,
                          float *scratch_sum);
void vfo_flash_attn_reduce(const float *scratch_out, const float *scratch_max,
                           const float *scratch_sum, uint32_t n_heads, uint32_t head_dim,
                           uint32_t n_tiles, float *out);

/* batched decode step used as the timed CPU baseline: for every sequence,
 * append one token (k_new/v_new f32 [seq][kv_head][dim]) at position
 * seq_lens[i]-1 of its slab and attend over [kv_starts[i], seq_lens[i]).
 * slabs are n_seqs consecutive slabs of slab_positions rows each. */
void vfo_decode_step(const float *q, const float *k_new, const float *v_new,
                     void *k_slabs, void *v_slabs, uint32_t dtype,
                     uint32_t n_seqs, uint64_t slab_positions,
                     uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                     const uint32_t *seq_lens, const uint32_t *kv_starts,
                     float scale, float softcap, float *out);

int vfo_num_threads(void);
void vfo_set_num_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
