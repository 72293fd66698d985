// Layout arithmetic of the KV cache; see kv_cache.hpp.
#include "kv_cache.hpp"

#include <cstdlib>
#include <cstring>
#include <strings.h>

namespace vfkv {

static bool env_truthy(const char *name)
{
    const char *v = std::getenv(name);
    return v && (std::strcmp(v, "1") == 0 || strcasecmp(v, "true") == 0);
}

// kv_cache.rs:85-101.  The reference also sets VULKANFORGE_ENABLE_FP8 as a side
// effect (a Vulkan device-feature opt-in); there is no such feature bit here.
KvDtype kv_dtype_from_env()
{
    if (env_truthy("VULKANFORGE_KV_FP8")) return KvDtype::F8;
    const char *v = std::getenv("VULKANFORGE_FP16_KV");
    if (v && std::strcmp(v, "0") == 0) return KvDtype::F32;
    return KvDtype::F16;
}

// kv_cache.rs:126-151
bool guard_kv_precision(bool is_gemma4_moe, KvDtype kv_dtype, bool force, std::string *msg)
{
    if (!is_gemma4_moe || kv_dtype == KvDtype::F8) return true;
    if (msg) {
        *msg = std::string("gemma-4-MoE (26B) requires VULKANFORGE_KV_FP8=1 -- non-FP8 KV (here: ") +
               label(kv_dtype) +
               ") is known-broken for this model; only FP8 (E4M3) KV is correct. Set "
               "VULKANFORGE_KV_FP8=1, or VULKANFORGE_ALLOW_BROKEN_KV=1 to force.";
    }
    return force;
}

// kv_cache.rs:186-202 (saturating arithmetic)
uint64_t kv_bytes_per_token(uint32_t n_layers, uint32_t n_kv_heads, uint32_t head_dim,
                            const uint32_t *plhd, const uint32_t *plkv, uint64_t elem_size)
{
    auto sat_mul = [](uint64_t a, uint64_t b) {
        uint64_t r;
        return __builtin_mul_overflow(a, b, &r) ? UINT64_MAX : r;
    };
    auto sat_add = [](uint64_t a, uint64_t b) {
        uint64_t r;
        return __builtin_add_overflow(a, b, &r) ? UINT64_MAX : r;
    };
    uint64_t elems = 0;
    for (uint32_t i = 0; i < n_layers; ++i) {
        uint64_t hd = plhd ? plhd[i] : head_dim, kvh = plkv ? plkv[i] : n_kv_heads;
        elems = sat_add(elems, sat_mul(kvh, hd));
    }
    return sat_mul(sat_mul(elems, elem_size), 2u);
}

// kv_cache.rs:243-292
bool KvCache::plan(const KvCacheConfig &cfg_in, KvDtype dtype, KvCache *out, std::string *err)
{
    KvCacheConfig cfg = cfg_in;
    if (cfg.n_slots == 0) cfg.n_slots = 1;
    auto fail = [&](const char *m) {
        if (err) *err = m;
        return false;
    };
    if (cfg.n_layers == 0 || cfg.max_seq_len == 0) return fail("n_layers and max_seq_len must be non-zero");
    if (cfg.per_layer_head_dim && cfg.per_layer_head_dim->size() != cfg.n_layers)
        return fail("per_layer_head_dim length must equal n_layers");
    if (cfg.per_layer_n_kv_heads && cfg.per_layer_n_kv_heads->size() != cfg.n_layers)
        return fail("per_layer_n_kv_heads length must equal n_layers");
    if (cfg.scale_mode > 1) return fail("unknown scale_mode");
    if (cfg.scale_mode != 0 && dtype != KvDtype::F8) return fail("scale_mode requires an FP8 cache");

    out->config = cfg;
    out->kv_dtype = dtype;
    out->current_seq_len.assign(cfg.n_slots, 0);
    const uint64_t es = element_size(dtype);
    const bool any_per_layer = cfg.per_layer_head_dim || cfg.per_layer_n_kv_heads;

    std::vector<uint64_t> offsets, soffsets;
    offsets.reserve(cfg.n_layers + 1);
    soffsets.reserve(cfg.n_layers + 1);
    uint64_t acc = 0, sacc = 0;
    offsets.push_back(0);
    soffsets.push_back(0);
    for (uint32_t i = 0; i < cfg.n_layers; ++i) {
        uint64_t hd = out->head_dim_for(i), kvh = out->kv_heads_for(i), t, s;
        if (__builtin_mul_overflow(uint64_t(cfg.max_seq_len), kvh, &s) ||
            __builtin_mul_overflow(s, uint64_t(cfg.n_slots), &s))
            return fail("kv-cache per-layer size overflow");
        if (__builtin_mul_overflow(s, hd, &t) || __builtin_mul_overflow(t, es, &t))
            return fail("kv-cache per-layer size overflow");
        if (__builtin_add_overflow(acc, t, &acc) || __builtin_add_overflow(sacc, s, &sacc))
            return fail("kv-cache total size overflow");
        // 16-byte rows keep every vectorised store and every TMA box aligned
        if ((kvh * hd * es) % 16u != 0 && kvh * hd != 0)
            return fail("kv_heads*head_dim*element_size must be a multiple of 16 bytes");
        offsets.push_back(acc);
        soffsets.push_back(sacc);
    }
    out->bytes = acc;
    out->scale_floats = cfg.scale_mode ? sacc : 0;
    out->scale_layer_offsets_ = soffsets;
    if (any_per_layer) out->layer_byte_offsets = offsets;
    else out->layer_byte_offsets.reset();
    return true;
}

// kv_cache.rs:431-440,466-472
uint64_t KvCache::layer_offset_bytes(uint32_t layer) const
{
    if (layer_byte_offsets) return (*layer_byte_offsets)[layer];
    return uint64_t(layer) * config.n_slots * config.n_kv_heads * config.max_seq_len *
           config.head_dim * element_size(kv_dtype);
}

uint64_t KvCache::scale_offset(uint32_t layer, uint32_t slot, uint32_t pos) const
{
    return scale_layer_offsets_[layer] +
           (uint64_t(slot) * config.max_seq_len + pos) * kv_heads_for(layer);
}

}  // namespace vfkv
