// Host-side mirror of VulkanForge's KvCache (src/backend/vulkan/kv_cache.rs),
// kept in the reference's own vocabulary so a maintainer can map one onto the
// other method by method.  Pure layout arithmetic and bookkeeping; the device
// buffers are plain CUDA allocations owned by this object.
#pragma once

#include <cstdint>
#include <optional>
#include <string>
#include <vector>

namespace vfkv {

// kv_cache.rs:42-74
enum class KvDtype : uint32_t { F32 = 0, F16 = 1, F8 = 2 };

inline uint64_t element_size(KvDtype d)
{
    return d == KvDtype::F32 ? 4u : d == KvDtype::F16 ? 2u : 1u;
}
inline const char *label(KvDtype d)
{
    return d == KvDtype::F32 ? "FP32" : d == KvDtype::F16 ? "FP16" : "FP8";
}

// kv_cache.rs:85-101
KvDtype kv_dtype_from_env();
// kv_cache.rs:126-151 (the pure core; `force` is the env override of :118-123)
bool guard_kv_precision(bool is_gemma4_moe, KvDtype kv_dtype, bool force, std::string *msg);
// kv_cache.rs:186-202
uint64_t kv_bytes_per_token(uint32_t n_layers, uint32_t n_kv_heads, uint32_t head_dim,
                            const uint32_t *per_layer_head_dim,
                            const uint32_t *per_layer_n_kv_heads, uint64_t elem_size);
// forward/arch/gemma4.rs:59-73, sliding layers
inline uint32_t sliding_kv_start(uint32_t position, uint32_t window)
{
    uint32_t seq_len = position + 1u;
    return seq_len > window ? seq_len - window : 0u;
}

// kv_cache.rs:153-176
struct KvCacheConfig {
    uint32_t n_layers = 0;
    uint32_t n_kv_heads = 0;
    uint32_t head_dim = 0;
    uint32_t max_seq_len = 0;
    std::optional<std::vector<uint32_t>> per_layer_head_dim;
    std::optional<std::vector<uint32_t>> per_layer_n_kv_heads;
    // build-side additions
    uint32_t n_slots = 1;      // independent sequences, each a full copy of the reference's slab
    uint32_t scale_mode = 0;   // 0 = none (reference); 1 = per-(token, kv-head) absmax, FP8 only
};

// kv_cache.rs:204-221.  Layout is [layer][slot][pos][kv_head][dim]; with one
// slot it is the reference's [layer][pos][kv_head][dim].
struct KvCache {
    void *k_buffer = nullptr;
    void *v_buffer = nullptr;
    float *k_scales = nullptr;   // [layer][slot][pos][kv_head], scale_mode 1 only
    float *v_scales = nullptr;
    KvCacheConfig config;
    std::vector<uint32_t> current_seq_len;              // one counter per slot (:208 has one)
    KvDtype kv_dtype = KvDtype::F16;
    // :219-221 -- n_layers+1 cumulative entries when any per-layer override is set
    std::optional<std::vector<uint64_t>> layer_byte_offsets;
    uint64_t bytes = 0;                                  // per buffer, all slots
    uint64_t scale_floats = 0;                           // per scale plane

    // Computes sizes with checked arithmetic (:243-292).  Returns false and sets
    // *err on overflow or an inconsistent config; allocates nothing.
    static bool plan(const KvCacheConfig &cfg, KvDtype dtype, KvCache *out, std::string *err);

    uint64_t bytes_per_buffer() const { return bytes; }                   // :379-381
    uint32_t head_dim_for(uint32_t layer) const                           // :412-417
    {
        return config.per_layer_head_dim ? (*config.per_layer_head_dim)[layer] : config.head_dim;
    }
    uint32_t kv_heads_for(uint32_t layer) const                           // :422-427
    {
        return config.per_layer_n_kv_heads ? (*config.per_layer_n_kv_heads)[layer]
                                           : config.n_kv_heads;
    }
    uint64_t row_bytes(uint32_t layer) const                              // :456-460
    {
        return uint64_t(kv_heads_for(layer)) * head_dim_for(layer) * element_size(kv_dtype);
    }
    uint64_t layer_size_bytes(uint32_t layer) const                       // :485-490 (one slot)
    {
        return uint64_t(config.max_seq_len) * row_bytes(layer);
    }
    // :431-440 / :466-472 scaled by the slot count: start of slot 0 of `layer`
    uint64_t layer_offset_bytes(uint32_t layer) const;
    uint64_t layer_offset_elems(uint32_t layer) const
    {
        return layer_offset_bytes(layer) / element_size(kv_dtype);
    }
    uint64_t slot_offset_bytes(uint32_t layer, uint32_t slot) const
    {
        return layer_offset_bytes(layer) + uint64_t(slot) * layer_size_bytes(layer);
    }
    uint64_t pos_offset_bytes(uint32_t layer, uint32_t pos) const          // :446-450
    {
        return layer_offset_bytes(layer) + uint64_t(pos) * row_bytes(layer);
    }
    // scale planes: float index of (layer, slot, pos, head 0)
    uint64_t scale_offset(uint32_t layer, uint32_t slot, uint32_t pos) const;
    bool is_fp8() const { return kv_dtype == KvDtype::F8; }               // :474-476
    bool is_fp16() const { return kv_dtype == KvDtype::F16; }             // :478-480
    void reset(uint32_t slot) { current_seq_len[slot] = 0; }              // :492-494

private:
    std::vector<uint64_t> scale_layer_offsets_;   // n_layers+1, in floats
};

}  // namespace vfkv
