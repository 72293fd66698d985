// Host-side entry points around the hot path (declared in include/vfkv_next.h): the decode
// attention routing of Forward::run_scalar_attn (src/backend/vulkan/forward/runs.rs:722-821) and
// the bookkeeping that moves the cache's length counter (src/server/state.rs:183-290,
// src/server/auto_ctx.rs:107-141, src/backend/vulkan/forward/arch/gemma4.rs:27-49).
// Everything here goes through the public C ABI of vfkv.h; no kernels.
#include <algorithm>
#include <cstdlib>
#include <vector>
#include "../../include/vfkv_next.h"

namespace {
constexpr uint32_t kFaTile = 64;           // FA_TILE, runs.rs:766
constexpr uint32_t kMultiWgMinTiles = 2;   // MULTI_WG_MIN_TILES, runs.rs:767
constexpr uint32_t kRoundTo = 256;         // ROUND_TO, auto_ctx.rs:39
constexpr uint32_t kMinCtx = 512;          // MIN_CTX, auto_ctx.rs:45
}  // namespace

extern "C" {

int32_t vfkv_flash_attn(vfkv_cache *cache, uint32_t layer, uint32_t kv_layer, const float *d_q, float *d_out,
                        uint32_t n_q_heads, uint32_t slot, uint32_t seq_len, uint32_t kv_start, float scale,
                        float softcap, void *stream)
{
    return vfkv_attend(cache, nullptr, layer, kv_layer, d_q, d_out, n_q_heads, slot, seq_len, kv_start, scale,
                       softcap, 1, stream);
}

uint32_t vfkv_scalar_attn_uses_split(uint32_t position)
{
    const uint64_t seq_len = uint64_t(position) + 1;
    return (seq_len + kFaTile - 1) / kFaTile >= kMultiWgMinTiles ? 1u : 0u;
}

int32_t vfkv_scalar_attn(vfkv_cache *cache, vfkv_workspace *ws, uint32_t layer, uint32_t kv_layer, const float *d_q,
                         float *d_out, uint32_t n_q_heads, uint32_t slot, uint32_t position, uint32_t kv_start,
                         float scale, float softcap, void *stream)
{
    if (position == UINT32_MAX) return VFKV_ERR_INVALID;
    const uint32_t seq_len = position + 1;
    if (vfkv_scalar_attn_uses_split(position))
        return vfkv_attend(cache, ws, layer, kv_layer, d_q, d_out, n_q_heads, slot, seq_len, kv_start, scale,
                           softcap, 0, stream);
    return vfkv_flash_attn(cache, layer, kv_layer, d_q, d_out, n_q_heads, slot, seq_len, kv_start, scale, softcap,
                           stream);
}

uint64_t vfkv_longest_common_prefix(const uint32_t *a, uint64_t n_a, const uint32_t *b, uint64_t n_b)
{
    if (!a || !b) return 0;
    const uint64_t n = n_a < n_b ? n_a : n_b;
    uint64_t i = 0;
    while (i < n && a[i] == b[i]) ++i;
    return i;
}

int32_t vfkv_kv_reuse_prepare(vfkv_cache *cache, uint32_t slot, const uint32_t *cached_tokens, uint64_t n_cached,
                              const uint32_t *full_tokens, uint64_t n_full, int32_t reuse, uint32_t *start_pos)
{
    if (!cache || !start_pos) return VFKV_ERR_INVALID;
    *start_pos = 0;
    uint64_t k = 0;
    if (reuse) {
        const uint64_t lcp = vfkv_longest_common_prefix(cached_tokens, n_cached, full_tokens, n_full);
        const uint64_t cap = n_full ? n_full - 1 : 0;      // at least one token is always prefilled
        k = lcp < cap ? lcp : cap;
        // The reference's one fault-injection hook (state.rs:206-212, never set in production):
        // reuse more rows than the prompts have in common, bounded by the resident rows and the
        // new prompt, so that a test can show that a wrong reuse is caught.
        if (const char *extra = std::getenv("VF_KV_REUSE_OVERSHOOT")) {
            char *end = nullptr;
            const unsigned long long n = std::strtoull(extra, &end, 10);
            if (end != extra && *end == '\0') {
                k += n;
                if (k > n_cached) k = n_cached;
                if (k > cap) k = cap;
            }
        }
    }
    if (k == 0) return vfkv_cache_reset(cache, slot);
    if (k > UINT32_MAX) return VFKV_ERR_OVERFLOW;
    // rows [0, k) stay; the suffix prefill at base_pos = k overwrites the rest
    int32_t rc = vfkv_cache_set_seq_len(cache, slot, uint32_t(k));
    if (rc == VFKV_OK) *start_pos = uint32_t(k);
    return rc;
}

int32_t vfkv_kv_invalidate(vfkv_cache *cache, uint32_t slot) { return vfkv_cache_reset(cache, slot); }

int32_t vfkv_compute_auto_ctx(uint64_t free_bytes, uint64_t weight_bytes, uint64_t reserve_bytes,
                              uint64_t kv_bytes_per_token, uint32_t model_max_ctx, uint32_t hw_cap, uint32_t sane_cap,
                              uint32_t *ctx_out, uint32_t *bound, uint64_t *avail_for_kv)
{
    if (!ctx_out) return VFKV_ERR_INVALID;
    uint64_t avail = free_bytes > weight_bytes ? free_bytes - weight_bytes : 0;       // saturating
    avail = avail > reserve_bytes ? avail - reserve_bytes : 0;
    const uint64_t bpt = kv_bytes_per_token ? kv_bytes_per_token : 1;
    const uint64_t by_vram = avail / bpt;
    uint32_t ctx = by_vram > UINT32_MAX ? UINT32_MAX : uint32_t(by_vram);
    uint32_t which = 0;
    if (model_max_ctx < ctx) { ctx = model_max_ctx; which = 1; }
    if (hw_cap < ctx) { ctx = hw_cap; which = 2; }
    if (sane_cap < ctx) { ctx = sane_cap; which = 3; }
    ctx = ctx / kRoundTo * kRoundTo;
    if (ctx < kMinCtx) ctx = kMinCtx;
    *ctx_out = ctx;
    if (bound) *bound = which;
    if (avail_for_kv) *avail_for_kv = avail;
    return VFKV_OK;
}

uint32_t vfkv_gemma4_kv_read_layer(const uint32_t *kv_source, uint32_t n_layers, uint32_t layer)
{
    if (!kv_source || layer >= n_layers) return layer;
    uint32_t want;
    switch (kv_source[layer]) {
    case 3: want = 1; break;       // SubscribesSliding -> OwnAndPublishesSliding
    case 4: want = 2; break;       // SubscribesFull    -> OwnAndPublishesFull
    default: return layer;
    }
    for (uint32_t i = 0; i < n_layers; ++i)
        if (kv_source[i] == want) return i;
    return layer;
}


/* ---- the sharding plan ----------------------------------------------------------------------- */

uint32_t vfkv_shard_owner(uint32_t world, uint32_t page, uint64_t pos)
{
    return world && page ? uint32_t((pos / page) % world) : 0u;
}

uint64_t vfkv_shard_local_pos(uint32_t world, uint32_t page, uint64_t pos)
{
    return world && page ? ((pos / page) / world) * page + pos % page : 0ull;
}

uint64_t vfkv_shard_local_len(uint32_t world, uint32_t page, uint64_t seq_len, uint32_t rank)
{
    if (!world || !page || rank >= world) return 0;
    const uint64_t full_pages = seq_len / page, rest = seq_len % page;
    uint64_t n = (full_pages / world) * page;
    const uint64_t extra = full_pages % world;      // ranks below it hold one more full page, it holds the rest
    if (rank < extra) n += page;
    else if (rank == extra) n += rest;
    return n;
}

uint64_t vfkv_shard_local_capacity(uint32_t world, uint32_t page, uint64_t max_seq_len)
{
    if (!world || !page) return 0;
    const uint64_t pages = (max_seq_len + page - 1) / page;
    return ((pages + world - 1) / world) * page;
}

int32_t vfkv_assign_sequences(const uint32_t *lengths, uint32_t n, uint32_t world, uint32_t *owner_out)
{
    if (!world || (n && (!lengths || !owner_out))) return VFKV_ERR_INVALID;
    std::vector<uint32_t> order(n);
    for (uint32_t i = 0; i < n; ++i) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return lengths[a] > lengths[b]; });
    std::vector<uint64_t> load(world, 0);
    for (uint32_t i : order) {
        uint32_t best = 0;
        for (uint32_t r = 1; r < world; ++r)
            if (load[r] < load[best]) best = r;
        owner_out[i] = best;
        load[best] += lengths[i];
    }
    return VFKV_OK;
}

int32_t vfkv_shard_kv_heads(uint32_t world, uint32_t rank, uint32_t n_kv_heads, uint32_t *first, uint32_t *count)
{
    if (!world || rank >= world || !first || !count) return VFKV_ERR_INVALID;
    const uint32_t base = n_kv_heads / world, extra = n_kv_heads % world;   // the first `extra` ranks hold one more
    *count = base + (rank < extra ? 1u : 0u);
    *first = rank * base + (rank < extra ? rank : extra);
    return VFKV_OK;
}

}  // extern "C"
