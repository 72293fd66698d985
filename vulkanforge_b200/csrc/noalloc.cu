// Split-K decode attention for callers that must not allocate device memory.
//
// Some hosts cannot call cudaMalloc once they are running: an engine that carves
// all of its VRAM out of one arena at start-up and treats any later allocation as
// a bug (VulkanForge itself sizes every buffer in its setup phase), a serving
// thread for which the implicit device synchronisation of cudaMalloc / cudaFree
// is a latency fault, or a process whose memory budget is owned by another
// component.  For them this file offers the raw-buffer attention entry point
// with its split-K scratch (the per-split max / sum / partial output, plus the
// status word the kernels report into) living in a file-scope __device__ array
// instead of a vfkv_workspace.  The caller still passes Q, K, V and the output.
//
// Cost: every GPU that loads libvfkv.so carries kScratchBytes (about 2 MiB) of
// device memory for the lifetime of the process, whether or not this entry
// point is ever used.
#include <mutex>

#include "common.cuh"

namespace vfkv {
namespace {

constexpr uint64_t kHeaderBytes = 256;                       // status word, padded
constexpr uint64_t kPartialFloats = 512u * 1024u;            // m, l and o of every (head, split)
constexpr uint64_t kScratchBytes = kHeaderBytes + kPartialFloats * sizeof(float);
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for the runtime to look up; it is not
// an address a kernel can use.  The device address is fetched once per device
// with cudaGetSymbolAddress below and that pointer is what the kernels receive.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

std::mutex g_mutex;
unsigned char *g_scratch_ptr[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};
thread_local char g_last_error[256] = "";

int32_t fail(int32_t status, const char *msg)
{
    snprintf(g_last_error, sizeof(g_last_error), "%s", msg);
    return status;
}

// One-time set-up for the calling thread's current device.
int32_t scratch_for_current_device(unsigned char **out, int *sm_count)
{
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(VFKV_ERR_CUDA, cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(VFKV_ERR_UNSUPPORTED, "device ordinal beyond the 64 this entry point tracks");
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_scratch_ptr[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            snprintf(g_last_error, sizeof(g_last_error), "cudaGetSymbolAddress(scratch) failed: %s", cudaGetErrorString(e));
            return VFKV_ERR_CUDA;
        }
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return fail(VFKV_ERR_CUDA, cudaGetErrorString(e));
        g_sm_count[dev] = sms;
        g_scratch_ptr[dev] = static_cast<unsigned char *>(p);
    }
    *out = g_scratch_ptr[dev];
    *sm_count = g_sm_count[dev];
    return VFKV_OK;
}

}  // namespace
}  // namespace vfkv

using namespace vfkv;

extern "C" {

const char *vfkv_noalloc_last_error(void) { return g_last_error; }

uint64_t vfkv_noalloc_scratch_bytes(void) { return kScratchBytes; }

int32_t vfkv_flash_attn_split_reduce_noalloc(const float *d_q, const void *d_k, const void *d_v, float *d_out,
                                             uint32_t dtype, uint32_t n_heads, uint32_t n_kv_heads,
                                             uint32_t head_dim, uint32_t seq_len, uint32_t max_seq, float scale,
                                             uint32_t kv_start, float softcap, uint32_t n_splits, void *stream)
{
    g_last_error[0] = 0;
    if (!d_q || !d_k || !d_v || !d_out) return fail(VFKV_ERR_INVALID, "null buffer");
    if (dtype > VFKV_F8) return fail(VFKV_ERR_INVALID, "unknown dtype");
    if (n_heads == 0 || n_kv_heads == 0 || n_heads % n_kv_heads != 0)
        return fail(VFKV_ERR_INVALID, "n_heads must be a non-zero multiple of n_kv_heads");
    if (head_dim != 64 && head_dim != 128 && head_dim != 256 && head_dim != 512)
        return fail(VFKV_ERR_UNSUPPORTED, "head_dim must be 64, 128, 256 or 512");
    if (seq_len > max_seq || kv_start > seq_len) return fail(VFKV_ERR_INVALID, "need kv_start <= seq_len <= max_seq");
    if ((reinterpret_cast<uintptr_t>(d_k) | reinterpret_cast<uintptr_t>(d_v)) % 16 != 0)
        return fail(VFKV_ERR_INVALID, "K/V slabs must be 16-byte aligned");
    if (n_splits == 0) n_splits = 1;
    // the fixed scratch bounds the problem: (m, l, o[head_dim]) per (head, split)
    const uint64_t need = uint64_t(n_heads) * n_splits * (uint64_t(head_dim) + 2);
    if (need > kPartialFloats) {
        snprintf(g_last_error, sizeof(g_last_error),
                 "n_heads*n_splits*(head_dim+2) = %llu floats exceeds the built-in scratch of %llu floats; "
                 "lower n_splits or use vfkv_flash_attn_split_reduce with a workspace",
                 (unsigned long long)need, (unsigned long long)kPartialFloats);
        return VFKV_ERR_UNSUPPORTED;
    }
    unsigned char *base = nullptr;
    int sms = 0;
    int32_t rc = scratch_for_current_device(&base, &sms);
    if (rc != VFKV_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    // Stack-only stand-ins for the context and workspace objects; they point into the scratch.
    vfkv_ctx ctx;
    ctx.sm_count = sms;
    ctx.d_status = reinterpret_cast<uint32_t *>(base);
    vfkv_workspace ws;
    ws.ctx = &ctx;
    ws.max_seqs = 1; ws.n_q_heads = n_heads; ws.head_dim = head_dim; ws.max_splits = n_splits;
    float *f = reinterpret_cast<float *>(base + kHeaderBytes);
    const uint64_t parts = uint64_t(n_heads) * n_splits;
    ws.part_m = f;
    ws.part_l = f + parts;
    ws.part_o = f + 2 * parts;

    // The array keeps whatever the previous call left.  The partials are fully rewritten by
    // the split kernel before the merge reads them; only the status word must start at zero.
    // (Nothing can raise it here -- the CUDA-core kernels only report out-of-range entries of
    // device arrays, and this entry point passes host-checked scalars -- so no call reads it back.)
    cudaError_t e = cudaMemsetAsync(base, 0, sizeof(uint32_t), st);
    if (e != cudaSuccess) return fail(VFKV_ERR_CUDA, cudaGetErrorString(e));

    AttnArgs a;
    a.kv.k = d_k; a.kv.v = d_v; a.kv.max_seq = max_seq; a.kv.n_slots = 1; a.kv.dtype = dtype;
    a.kv.n_kv_heads = n_kv_heads; a.kv.head_dim = head_dim;
    a.seq.n_seqs = 1; a.seq.seq_len_scalar = seq_len; a.seq.kv_start_scalar = kv_start;
    a.q = d_q; a.out = d_out; a.n_q_heads = n_heads; a.scale = scale; a.softcap = softcap;
    rc = launch_attn_generic(&ctx, &ws, a, n_splits, st);
    if (rc == VFKV_OK && n_splits > 1) rc = launch_merge_ws(&ctx, &ws, a, n_splits, st);
    if (rc != VFKV_OK) snprintf(g_last_error, sizeof(g_last_error), "%s", ctx.last_error.c_str());
    return rc;
}

}  // extern "C"
