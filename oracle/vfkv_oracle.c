/*
 * vfkv_oracle.c -- CPU restatement of VulkanForge's KV-cache hot path.
 * TEST INFRASTRUCTURE ONLY (see vfkv_oracle.h for the parity status of each part).
 *
 * Every function names the reference source it follows, by the file's path
 * inside the VulkanForge tree.
 */
#include "vfkv_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline uint32_t f32_bits(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static inline float bits_f32(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }

int vfo_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Launchers such as torch.distributed.run export OMP_NUM_THREADS=1; a timed CPU run sets
 * the count it wants explicitly. */
void vfo_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ===================================================================== */
/* E4M3 ("FN": no Inf, one NaN code, max 448)                             */
/* ===================================================================== */

/* src/backend/vulkan/fp8_ext.rs:104-122 */
float vfo_e4m3_to_f32(uint8_t b)
{
    uint32_t sign = (b >> 7) & 1u, e = (b >> 3) & 0xFu, m = b & 7u;
    float sf = sign ? -1.0f : 1.0f;
    if (e == 0xF && m == 7) return sf * NAN;
    if (e == 0) return sf * ((float)m / 8.0f) * ldexpf(1.0f, -6);
    return sf * (1.0f + (float)m / 8.0f) * ldexpf(1.0f, (int)e - 7);
}

/* src/backend/vulkan/fp8_ext.rs:189-211: keep the top 3 of 23 mantissa bits
 * after `extra` additional right shifts, round to nearest, ties to even.
 * Returns 0..8; 8 means the mantissa carried out. */
static uint32_t round_mant3(uint32_t mant, uint32_t extra)
{
    uint32_t shift = 20u + extra;
    if (shift >= 32u) return 0;
    uint32_t trunc = mant >> shift;
    uint32_t rbit = (mant >> (shift - 1u)) & 1u;
    int sticky = (mant & ((1u << (shift - 1u)) - 1u)) != 0;
    if (rbit && (sticky || (trunc & 1u))) trunc += 1u;
    return trunc;
}

/* src/backend/vulkan/fp8_ext.rs:126-187: NaN -> 0x7F, signed zero kept,
 * |x| >= 448 -> 0x7E, RNE in the normal and subnormal ranges, a carry to
 * exponent 16 clamps to 0x7E, more than 23 bits of underflow -> signed zero. */
uint8_t vfo_f32_to_e4m3(float x)
{
    uint32_t u = f32_bits(x);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7F;
    uint8_t s = (u >> 31) ? 0x80 : 0x00;
    uint32_t a = u & 0x7FFFFFFFu;
    if (a == 0) return s;
    if (bits_f32(a) >= 448.0f) return s | 0x7E;
    int32_t e = (int32_t)((a >> 23) & 0xFF) - 127 + 7;
    uint32_t mant = a & 0x007FFFFFu;
    if (e >= 1 && e <= 15) {
        uint32_t m3 = round_mant3(mant, 0);
        if (m3 == 8) {
            if (e + 1 == 16) return s | 0x7E;
            return s | (uint8_t)((e + 1) << 3);
        }
        return s | (uint8_t)(e << 3) | (uint8_t)m3;
    }
    if (e <= 0) {
        uint32_t shift = (uint32_t)(1 - e);
        if (shift > 23) return s;
        uint32_t m3 = round_mant3(0x00800000u | mant, shift);
        if (m3 == 8) return s | 0x08;
        return s | (uint8_t)m3;
    }
    return s | 0x7E;
}

/* ===================================================================== */
/* IEEE binary16, round to nearest even (the `half` crate's from_f32,     */
/* which the reference's tests use to mirror the F16 cache:               */
/* tests/coopmat_fa_gemma.rs:74,212)                                      */
/* ===================================================================== */
uint16_t vfo_f32_to_f16(float x)
{
    uint32_t u = f32_bits(x);
    uint16_t s = (uint16_t)((u >> 16) & 0x8000u);
    uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return s | 0x7E00 | (uint16_t)((a >> 13) & 0x3FF); /* NaN, quiet */
    if (a >= 0x47800000u) return s | 0x7C00;            /* >= 65536 (incl. Inf) -> Inf */
    int32_t e = (int32_t)(a >> 23) - 127;
    uint32_t mant = a & 0x007FFFFFu;
    if (e >= -14) {
        uint32_t h = ((uint32_t)(e + 15) << 10) | (mant >> 13);
        uint32_t rem = mant & 0x1FFFu;
        if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h += 1u; /* may carry to Inf */
        return s | (uint16_t)h;
    }
    if (e < -25) return s;                               /* below half the min subnormal */
    uint32_t full = 0x00800000u | mant;
    uint32_t shift = (uint32_t)(-14 - e) + 13u;          /* 14..24 */
    uint32_t h = full >> shift;
    uint32_t rem = full & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1u);
    if (rem > halfway || (rem == halfway && (h & 1u))) h += 1u;
    return s | (uint16_t)h;
}

float vfo_f16_to_f32(uint16_t h)
{
    uint32_t s = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
    if (e == 0x1F) return bits_f32(s | 0x7F800000u | (m << 13));
    if (e == 0) {
        float v = ldexpf((float)m, -24);
        return s ? -v : v;
    }
    return bits_f32(s | ((e + 112u) << 23) | (m << 13));
}

void vfo_f32_bits_to_e4m3_range(uint32_t first_bits, uint64_t count, uint8_t *dst)
{
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)count; ++i)
        dst[i] = vfo_f32_to_e4m3(bits_f32(first_bits + (uint32_t)i));
}

void vfo_f32_bits_to_f16_range(uint32_t first_bits, uint64_t count, uint16_t *dst)
{
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)count; ++i)
        dst[i] = vfo_f32_to_f16(bits_f32(first_bits + (uint32_t)i));
}

/* ===================================================================== */
/* append / convert ops                                                   */
/* ===================================================================== */

/* vk_shaders/kv_store_fp8.comp:42-66: four codes per 32-bit word, first
 * element in the low byte; a ragged tail is padded with the code of 0.0. */
void vfo_kv_store_fp8(const float *src, uint32_t n, uint8_t *dst)
{
    uint32_t padded = (n + 3u) & ~3u;
    for (uint32_t i = 0; i < padded; ++i)
        dst[i] = vfo_f32_to_e4m3(i < n ? src[i] : 0.0f);
}

/* vk_shaders/kv_copy_fp16.comp:40-50: two halfs per word, first element low. */
void vfo_kv_copy_fp16(const float *src, uint32_t n, uint16_t *dst)
{
    uint32_t padded = (n + 1u) & ~1u;
    for (uint32_t i = 0; i < padded; ++i)
        dst[i] = vfo_f32_to_f16(i < n ? src[i] : 0.0f);
}

/* vk_shaders/kv_fp8_to_f16.comp:28-34: identity index; every E4M3 value is
 * exactly representable in binary16, so the narrowing never rounds. */
void vfo_kv_fp8_to_f16(const uint8_t *src, uint32_t n, uint16_t *dst)
{
    for (uint32_t i = 0; i < n; ++i)
        dst[i] = vfo_f32_to_f16(vfo_e4m3_to_f32(src[i]));
}

/* Extension (not in kv_store_fp8.comp, which has no scale).  The recipe is the
 * reference's only absmax/448 quantiser, the FP8 GEMM activation path:
 * vk_shaders/mul_coopmat_fp8_native_bn32.comp:149-152 (scale, reciprocal) and
 * :214 (multiply, clamp, cast).  One scale per (token, kv-head). */
void vfo_kv_store_fp8_scaled(const float *src, uint32_t n_heads, uint32_t head_dim,
                             uint8_t *dst, float *scales)
{
    for (uint32_t h = 0; h < n_heads; ++h) {
        const float *x = src + (size_t)h * head_dim;
        float amax = 0.0f;
        for (uint32_t d = 0; d < head_dim; ++d) {
            float a = fabsf(x[d]);
            if (a > amax) amax = a;              /* NaN never raises the max */
        }
        float sc = fmaxf(amax * (1.0f / 448.0f), 1e-12f);
        float inv = 1.0f / sc;
        scales[h] = sc;
        for (uint32_t d = 0; d < head_dim; ++d) {
            float y = x[d] * inv;
            y = fminf(fmaxf(y, -448.0f), 448.0f);
            if (x[d] != x[d]) y = x[d];          /* keep NaN a NaN */
            dst[(size_t)h * head_dim + d] = vfo_f32_to_e4m3(y);
        }
    }
}

/* ===================================================================== */
/* cache layout: src/backend/vulkan/kv_cache.rs                           */
/* ===================================================================== */

uint64_t vfo_elem_size(uint32_t dtype)            /* kv_cache.rs:60-66 */
{
    return dtype == VFO_F32 ? 4u : dtype == VFO_F16 ? 2u : 1u;
}

uint32_t vfo_head_dim_for(const vfo_layout *c, uint32_t layer)   /* :412-417 */
{
    return c->per_layer_head_dim ? c->per_layer_head_dim[layer] : c->head_dim;
}

uint32_t vfo_kv_heads_for(const vfo_layout *c, uint32_t layer)   /* :422-427 */
{
    return c->per_layer_n_kv_heads ? c->per_layer_n_kv_heads[layer] : c->n_kv_heads;
}

uint64_t vfo_row_bytes(const vfo_layout *c, uint32_t layer)      /* :456-460 */
{
    return (uint64_t)vfo_kv_heads_for(c, layer) * vfo_head_dim_for(c, layer) *
           vfo_elem_size(c->dtype);
}

uint64_t vfo_layer_size_bytes(const vfo_layout *c, uint32_t layer)  /* :485-490 */
{
    return (uint64_t)c->max_seq_len * vfo_row_bytes(c, layer);
}

/* :243-283 (cumulative table when any per-layer override is present) and
 * :431-440,466-472 (closed form otherwise) */
uint64_t vfo_layer_offset_bytes(const vfo_layout *c, uint32_t layer)
{
    if (c->per_layer_head_dim || c->per_layer_n_kv_heads) {
        uint64_t acc = 0;
        for (uint32_t i = 0; i < layer; ++i) acc += vfo_layer_size_bytes(c, i);
        return acc;
    }
    return (uint64_t)layer * c->n_kv_heads * c->max_seq_len * c->head_dim *
           vfo_elem_size(c->dtype);
}

uint64_t vfo_pos_offset_bytes(const vfo_layout *c, uint32_t layer, uint32_t pos)  /* :446-450 */
{
    return vfo_layer_offset_bytes(c, layer) + (uint64_t)pos * vfo_row_bytes(c, layer);
}

static int mul_ovf(uint64_t a, uint64_t b, uint64_t *r) { return __builtin_mul_overflow(a, b, r); }
static int add_ovf(uint64_t a, uint64_t b, uint64_t *r) { return __builtin_add_overflow(a, b, r); }

int vfo_bytes_per_buffer(const vfo_layout *c, uint64_t *bytes)   /* :243-292, checked_mul */
{
    uint64_t acc = 0;
    for (uint32_t i = 0; i < c->n_layers; ++i) {
        uint64_t t;
        if (mul_ovf(c->max_seq_len, vfo_kv_heads_for(c, i), &t)) return -1;
        if (mul_ovf(t, vfo_head_dim_for(c, i), &t)) return -1;
        if (mul_ovf(t, vfo_elem_size(c->dtype), &t)) return -1;
        if (add_ovf(acc, t, &acc)) return -1;
    }
    *bytes = acc;
    return 0;
}

uint64_t vfo_kv_bytes_per_token(uint32_t n_layers, uint32_t n_kv_heads, uint32_t head_dim,
                                const uint32_t *plhd, const uint32_t *plkv,
                                uint64_t elem_size)              /* :186-202 */
{
    uint64_t elems = 0;
    for (uint32_t i = 0; i < n_layers; ++i) {
        uint64_t hd = plhd ? plhd[i] : head_dim, kvh = plkv ? plkv[i] : n_kv_heads;
        elems += kvh * hd;
    }
    return elems * elem_size * 2u;
}

/* src/backend/vulkan/forward/arch/gemma4.rs:59-73 (sliding layers) */
uint32_t vfo_sliding_kv_start(uint32_t position, uint32_t window)
{
    uint32_t seq_len = position + 1u;
    return seq_len > window ? seq_len - window : 0u;
}

/* ===================================================================== */
/* RoPE-NeoX: CPU form in tests/correctness.rs:827-838; theta_scale as in  */
/* src/backend/vulkan/forward/setup.rs:786-788                            */
/* ===================================================================== */
void vfo_rope_neox(float *x, uint32_t n_heads, uint32_t head_dim, uint32_t n_dims,
                   uint32_t pos, float freq_base)
{
    uint32_t half = n_dims / 2u;
    float theta_scale = powf(1.0f / freq_base, 2.0f / (float)n_dims);
    for (uint32_t h = 0; h < n_heads; ++h) {
        float *v = x + (size_t)h * head_dim;
        float freq = 1.0f;
        for (uint32_t i = 0; i < half; ++i) {
            float theta = (float)pos * freq;
            float c = cosf(theta), s = sinf(theta);
            float a = v[i], b = v[i + half];
            v[i] = a * c - b * s;
            v[i + half] = a * s + b * c;
            freq *= theta_scale;
        }
    }
}

/* ===================================================================== */
/* attention                                                              */
/* ===================================================================== */

static inline float load_kv(const void *p, uint32_t dtype, size_t idx)
{
    /* the three load_k/load_v variants of vk_shaders/flash_attn_split.comp:28-58 */
    switch (dtype) {
    case VFO_F32: return ((const float *)p)[idx];
    case VFO_F16: return vfo_f16_to_f32(((const uint16_t *)p)[idx]);
    default:      return vfo_e4m3_to_f32(((const uint8_t *)p)[idx]);
    }
}

/* decode table so the timed baseline does not pay the scalar decoder per byte */
static float g_e4m3_lut[256];
static int g_lut_ready = 0;
static void ensure_lut(void)
{
    if (!g_lut_ready) {
#pragma omp critical
        {
            for (int i = 0; i < 256; ++i) g_e4m3_lut[i] = vfo_e4m3_to_f32((uint8_t)i);
            g_lut_ready = 1;
        }
    }
}

/* One q-head of tests/correctness.rs:2567-2617: scores with an f64 dot
 * product, cast to f32, times scale; max; exp in f32; f64 sum; f64 weighted V
 * sum; multiply by the f32 reciprocal.  Added parameters, all neutral at their
 * defaults: kv_start (vk_shaders/flash_attn_split.comp:102), softcap
 * (extension: cap*tanh(s/cap), the formula of forward/arch/gemma4.rs:85-94
 * applied to scores), per-(pos, head) scales (extension). */
static void attend_one_head(const float *qh, const void *k, const void *v, uint32_t dtype,
                            uint32_t kvh, uint32_t n_kv_heads, uint32_t head_dim,
                            uint32_t seq_len, uint32_t kv_start, float scale, float softcap,
                            const float *k_scales, const float *v_scales,
                            float *scores, float *krow, float *out)
{
    size_t pos_stride = (size_t)n_kv_heads * head_dim, head_off = (size_t)kvh * head_dim;
    float max_score = -INFINITY;
    for (uint32_t t = kv_start; t < seq_len; ++t) {
        size_t kt = (size_t)t * pos_stride + head_off;
        double s = 0.0;
        if (dtype == VFO_F8) {
            const uint8_t *kb = (const uint8_t *)k + kt;
            for (uint32_t d = 0; d < head_dim; ++d) krow[d] = g_e4m3_lut[kb[d]];
        } else {
            for (uint32_t d = 0; d < head_dim; ++d) krow[d] = load_kv(k, dtype, kt + d);
        }
        if (k_scales) {
            float ks = k_scales[(size_t)t * n_kv_heads + kvh];
            for (uint32_t d = 0; d < head_dim; ++d) krow[d] *= ks;
        }
        for (uint32_t d = 0; d < head_dim; ++d) s += (double)qh[d] * (double)krow[d];
        float sf = (float)s * scale;
        if (softcap > 0.0f) sf = softcap * tanhf(sf / softcap);
        scores[t] = sf;
        if (sf > max_score) max_score = sf;
    }
    double sum = 0.0;
    for (uint32_t t = kv_start; t < seq_len; ++t) {
        scores[t] = expf(scores[t] - max_score);
        sum += (double)scores[t];
    }
    float inv = 1.0f / (float)sum;
    /* position-outer order keeps the V stream sequential; each out[d] still
     * accumulates in f64 in ascending position order, as the reference does */
    double *acc = (double *)calloc(head_dim, sizeof(double));
    for (uint32_t t = kv_start; t < seq_len; ++t) {
        size_t vt = (size_t)t * pos_stride + head_off;
        double p = (double)scores[t];
        float vs = v_scales ? v_scales[(size_t)t * n_kv_heads + kvh] : 1.0f;
        if (dtype == VFO_F8) {
            const uint8_t *vb = (const uint8_t *)v + vt;
            if (v_scales) for (uint32_t d = 0; d < head_dim; ++d) acc[d] += p * (double)(g_e4m3_lut[vb[d]] * vs);
            else          for (uint32_t d = 0; d < head_dim; ++d) acc[d] += p * (double)g_e4m3_lut[vb[d]];
        } else {
            for (uint32_t d = 0; d < head_dim; ++d) {
                float x = load_kv(v, dtype, vt + d);
                if (v_scales) x *= vs;
                acc[d] += p * (double)x;
            }
        }
    }
    for (uint32_t d = 0; d < head_dim; ++d) out[d] = (float)(acc[d] * (double)inv);
    free(acc);
}

void vfo_attention_ref(const float *q, const void *k, const void *v, uint32_t dtype,
                       uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                       uint32_t seq_len, uint32_t kv_start, float scale, float softcap,
                       const float *k_scales, const float *v_scales, float *out)
{
    ensure_lut();
    uint32_t group = n_heads / n_kv_heads;
#pragma omp parallel
    {
        float *scores = (float *)malloc(sizeof(float) * (seq_len ? seq_len : 1));
        float *krow = (float *)malloc(sizeof(float) * head_dim);
#pragma omp for schedule(dynamic, 1)
        for (int32_t h = 0; h < (int32_t)n_heads; ++h)
            attend_one_head(q + (size_t)h * head_dim, k, v, dtype, (uint32_t)h / group,
                            n_kv_heads, head_dim, seq_len, kv_start, scale, softcap,
                            k_scales, v_scales, scores, krow, out + (size_t)h * head_dim);
        free(scores);
        free(krow);
    }
}

/* vk_shaders/flash_attn_split.comp:82-161 with the tile width as a parameter
 * (the shader hard-codes 64).  f32 arithmetic, d ascending in the dot product,
 * positions ascending in the V sum, -1e30 for masked lanes. */
void vfo_flash_attn_split(const float *q, const void *k, const void *v, uint32_t dtype,
                          uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                          uint32_t seq_len, uint32_t kv_start, float scale, uint32_t tile,
                          uint32_t n_tiles, float *scratch_out, float *scratch_max,
                          float *scratch_sum)
{
    uint32_t group = n_heads / n_kv_heads;
    size_t pos_stride = (size_t)n_kv_heads * head_dim;
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
    for (int32_t h = 0; h < (int32_t)n_heads; ++h) {
        for (int32_t ti = 0; ti < (int32_t)n_tiles; ++ti) {
            size_t head_off = (size_t)((uint32_t)h / group) * head_dim;
            uint32_t base = (uint32_t)ti * tile;
            float *p = (float *)malloc(sizeof(float) * tile);
            float tmax = -1e30f;
            for (uint32_t i = 0; i < tile; ++i) {
                uint32_t t = base + i;
                float sc = -1e30f;
                if (t < seq_len && t >= kv_start) {
                    float s = 0.0f;
                    for (uint32_t d = 0; d < head_dim; ++d)
                        s += q[(size_t)h * head_dim + d] *
                             load_kv(k, dtype, (size_t)t * pos_stride + head_off + d);
                    sc = s * scale;
                }
                p[i] = sc;
                if (sc > tmax) tmax = sc;
            }
            float tsum = 0.0f;
            for (uint32_t i = 0; i < tile; ++i) {
                uint32_t t = base + i;
                int valid = t < seq_len && t >= kv_start;
                p[i] = valid ? expf(p[i] - tmax) : 0.0f;
                tsum += p[i];
            }
            size_t pidx = (size_t)h * n_tiles + (size_t)ti;
            scratch_max[pidx] = tmax;
            scratch_sum[pidx] = tsum;
            uint32_t tsize = base < seq_len ? (seq_len - base < tile ? seq_len - base : tile) : 0;
            for (uint32_t d = 0; d < head_dim; ++d) {
                float acc = 0.0f;
                for (uint32_t i = 0; i < tsize; ++i)
                    acc += p[i] * load_kv(v, dtype, (size_t)(base + i) * pos_stride + head_off + d);
                scratch_out[pidx * head_dim + d] = acc;
            }
            free(p);
        }
    }
}

/* vk_shaders/flash_attn_reduce.comp:51-80 */
void vfo_flash_attn_reduce(const float *scratch_out, const float *scratch_max,
                           const float *scratch_sum, uint32_t n_heads, uint32_t head_dim,
                           uint32_t n_tiles, float *out)
{
    for (uint32_t h = 0; h < n_heads; ++h) {
        for (uint32_t d = 0; d < head_dim; ++d) {
            float gmax = -1e30f, gsum = 0.0f, acc = 0.0f;
            for (uint32_t t = 0; t < n_tiles; ++t) {
                size_t pidx = (size_t)h * n_tiles + t;
                float tm = scratch_max[pidx], ts = scratch_sum[pidx];
                float nm = fmaxf(gmax, tm);
                float ko = expf(gmax - nm), kn = expf(tm - nm);
                acc = acc * ko + scratch_out[pidx * head_dim + d] * kn;
                gsum = gsum * ko + ts * kn;
                gmax = nm;
            }
            out[(size_t)h * head_dim + d] = acc * (1.0f / gsum);
        }
    }
}

/* Timed CPU baseline: the decode step of the forward loop for a batch of
 * independent sequences -- append (executor/attention.rs:546-596 calling the
 * store shaders) then attention (tests/correctness.rs:2567-2617). */
void vfo_decode_step(const float *q, const float *k_new, const float *v_new,
                     void *k_slabs, void *v_slabs, uint32_t dtype,
                     uint32_t n_seqs, uint64_t slab_positions,
                     uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                     const uint32_t *seq_lens, const uint32_t *kv_starts,
                     float scale, float softcap, float *out)
{
    ensure_lut();
    uint32_t kv_dim = n_kv_heads * head_dim, group = n_heads / n_kv_heads;
    uint64_t es = vfo_elem_size(dtype);
    uint64_t slab_bytes = slab_positions * kv_dim * es;
    for (uint32_t s = 0; s < n_seqs; ++s) {
        if (seq_lens[s] == 0) continue;
        uint64_t off = (uint64_t)s * slab_bytes + (uint64_t)(seq_lens[s] - 1u) * kv_dim * es;
        const float *kn = k_new + (size_t)s * kv_dim, *vn = v_new + (size_t)s * kv_dim;
        if (dtype == VFO_F8) {
            vfo_kv_store_fp8(kn, kv_dim, (uint8_t *)k_slabs + off);
            vfo_kv_store_fp8(vn, kv_dim, (uint8_t *)v_slabs + off);
        } else if (dtype == VFO_F16) {
            vfo_kv_copy_fp16(kn, kv_dim, (uint16_t *)((uint8_t *)k_slabs + off));
            vfo_kv_copy_fp16(vn, kv_dim, (uint16_t *)((uint8_t *)v_slabs + off));
        } else {
            memcpy((uint8_t *)k_slabs + off, kn, kv_dim * 4u);
            memcpy((uint8_t *)v_slabs + off, vn, kv_dim * 4u);
        }
    }
    uint32_t max_len = 1;
    for (uint32_t s = 0; s < n_seqs; ++s) if (seq_lens[s] > max_len) max_len = seq_lens[s];
#pragma omp parallel
    {
        float *scores = (float *)malloc(sizeof(float) * max_len);
        float *krow = (float *)malloc(sizeof(float) * head_dim);
#pragma omp for schedule(dynamic, 1)
        for (int64_t w = 0; w < (int64_t)n_seqs * n_heads; ++w) {
            uint32_t s = (uint32_t)(w / n_heads), h = (uint32_t)(w % n_heads);
            float *o = out + ((size_t)s * n_heads + h) * head_dim;
            if (seq_lens[s] == 0) { memset(o, 0, sizeof(float) * head_dim); continue; }
            attend_one_head(q + ((size_t)s * n_heads + h) * head_dim,
                            (const uint8_t *)k_slabs + (uint64_t)s * slab_bytes,
                            (const uint8_t *)v_slabs + (uint64_t)s * slab_bytes, dtype,
                            h / group, n_kv_heads, head_dim, seq_lens[s],
                            kv_starts ? kv_starts[s] : 0u, scale, softcap, NULL, NULL,
                            scores, krow, o);
        }
        free(scores);
        free(krow);
    }
}
