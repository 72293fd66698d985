// Exchange of softmax partials between the GPUs of a position-sharded group over peer memory.
//
// No counterpart in the reference (it is single-GPU).  The math of the merge is
// vk_shaders/flash_attn_reduce.comp:51-80 over one part per GPU.  Every GPU owns one exchange
// buffer of 8-byte words {f32 value, u32 tag}.  The attention kernel of rank r stores its (m, l, o)
// block into the buffer of every rank with plain peer stores, every word tagged with the number of
// the exchange; a word is written by a single 8-byte store, so a reader that finds the tag has
// the value, and neither a flag nor a fence is needed.  The merge kernel of each rank polls, with
// a time limit, the words of all source ranks in its own buffer and reduces them.  Blocks are
// double-buffered by the parity of the exchange number: a rank cannot be more than one exchange
// ahead of the slowest rank, because its own merge needs that rank's words first.
#include "attn_params.cuh"

#include <cstring>
#include <new>

namespace vfkv {

__device__ __forceinline__ uint64_t global_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Copies one staged block (plain floats: m[n_rows], l[n_rows], o[n_rows][head_dim]) into every
// rank's buffer as tagged words: the path of attention kernels without the fused fan-out.
__global__ void __launch_bounds__(256)
fanout_push_kernel(PeerFanout fan, const float *__restrict__ staging, uint32_t head_dim)
{
    const FanoutSlot fs = fanout_slot(fan, head_dim, fan.rank, *fan.epoch + 1u);
    const uint64_t n = fanout_block_words(fan.n_rows, head_dim);
    for (uint64_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += uint64_t(gridDim.x) * blockDim.x) {
        const float v = staging[i];
#pragma unroll
        for (uint32_t r = 0; r < 8; ++r)
            if (r < fan.world) fanout_store(fan.base[r] + fs.m + i, v, fs.epoch);
    }
}

__device__ __forceinline__ uint64_t load_word(const uint64_t *p)
{
    uint64_t w;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}

// Re-reads *p until it carries tag e or the time limit passes; returns false on a time-out.
__device__ __forceinline__ bool await_word(const uint64_t *p, uint64_t &w, uint32_t e, uint64_t t0, uint64_t wait_ns)
{
    while (uint32_t(w >> 32) != e) {
        if (global_ns() - t0 > wait_ns) return false;
        __nanosleep(32);
        w = load_word(p);
    }
    return true;
}

// One CTA per output row, thread t owning dims t, t+128, ...  All words a thread needs are
// requested at once; only those whose tag is not there yet are polled.  A wait that runs out sets
// bit 8 of the status word and the row is written as zeros.
__global__ void __launch_bounds__(128)
exchange_merge_kernel(PeerFanout fan, const uint64_t *__restrict__ local, uint32_t *__restrict__ ctl,
                      uint32_t head_dim, uint64_t wait_ns, float *__restrict__ out, uint32_t *__restrict__ status)
{
    constexpr int kMaxDims = 4, kMaxWorld = 8;
    __shared__ float s_m[kMaxWorld], s_l[kMaxWorld];
    __shared__ uint32_t s_bad;
    // Dependent launch: lets the next kernel of the stream start its prologue, and waits for the
    // attention kernel before it (and through it for the previous merge, which wrote ctl[0]).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t row = blockIdx.x;
    const uint32_t e = ctl[0] + 1u;
    const uint64_t t0 = global_ns();
    if (threadIdx.x == 0) s_bad = 0u;
    __syncthreads();

    uint64_t w[kMaxWorld][kMaxDims];
#pragma unroll
    for (uint32_t r = 0; r < kMaxWorld; ++r) {
        const FanoutSlot fs = fanout_slot(fan, head_dim, r, e);
#pragma unroll
        for (int j = 0; j < kMaxDims; ++j) {
            const uint32_t d = threadIdx.x + j * 128;
            w[r][j] = (r < fan.world && d < head_dim) ? load_word(local + fs.o + uint64_t(row) * head_dim + d) : 0ull;
        }
    }
    bool ok = true;
    if (threadIdx.x < 2 * fan.world) {                       // m and l of every source rank
        const uint32_t r = threadIdx.x >> 1, which = threadIdx.x & 1;
        const FanoutSlot fs = fanout_slot(fan, head_dim, r, e);
        const uint64_t *p = local + fs.m + uint64_t(which) * fan.n_rows + row;
        uint64_t v = load_word(p);
        ok = await_word(p, v, e, t0, wait_ns);
        (which ? s_l : s_m)[r] = __uint_as_float(uint32_t(v));
    }
#pragma unroll
    for (uint32_t r = 0; r < kMaxWorld; ++r) {
        const FanoutSlot fs = fanout_slot(fan, head_dim, r, e);
#pragma unroll
        for (int j = 0; j < kMaxDims; ++j) {
            const uint32_t d = threadIdx.x + j * 128;
            if (r < fan.world && d < head_dim)
                ok = await_word(local + fs.o + uint64_t(row) * head_dim + d, w[r][j], e, t0, wait_ns) && ok;
        }
    }
    if (!ok) atomicOr(&s_bad, 1u);
    __syncthreads();
    const bool bad = s_bad != 0u;
    if (bad && threadIdx.x == 0) atomicOr(status, 8u);

    float acc[kMaxDims] = {0.f, 0.f, 0.f, 0.f};
    float gmax = kMaskedScore, gsum = 0.f;
    if (!bad) {
#pragma unroll
        for (uint32_t r = 0; r < kMaxWorld; ++r)
            if (r < fan.world) gmax = fmaxf(gmax, s_m[r]);
#pragma unroll
        for (uint32_t r = 0; r < kMaxWorld; ++r) {
            if (r < fan.world) {
                const float kn = __expf(s_m[r] - gmax);
                gsum = fmaf(s_l[r], kn, gsum);
#pragma unroll
                for (int j = 0; j < kMaxDims; ++j) acc[j] = fmaf(__uint_as_float(uint32_t(w[r][j])), kn, acc[j]);
            }
        }
    }
    const float inv = gsum > 0.f ? 1.0f / gsum : 0.f;
#pragma unroll
    for (int j = 0; j < kMaxDims; ++j) {
        const uint32_t d = threadIdx.x + j * 128;
        if (d < head_dim) out[uint64_t(row) * head_dim + d] = acc[j] * inv;
    }
    // The CTA that finishes last closes the exchange: every CTA has read ctl[0] by then.
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t ticket = atomicAdd(&ctl[1], 1u);
        if (ticket == gridDim.x - 1) { ctl[1] = 0u; ctl[0] = e; }
    }
}

int32_t launch_fanout_push(vfkv_ctx *ctx, const PeerFanout &fan, const float *staging, uint32_t head_dim,
                           cudaStream_t st)
{
    const uint64_t n = fanout_block_words(fan.n_rows, head_dim);
    fanout_push_kernel<<<uint32_t((n + 255) / 256), 256, 0, st>>>(fan, staging, head_dim);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "fanout_push launch");
}

}  // namespace vfkv

using namespace vfkv;

namespace {
struct Guard {
    int prev = -1;
    explicit Guard(int dev) { cudaGetDevice(&prev); if (prev != dev) cudaSetDevice(dev); else prev = -1; }
    ~Guard() { if (prev >= 0) cudaSetDevice(prev); }
};
}  // namespace

extern "C" {

int32_t vfkv_exchange_create(vfkv_ctx *ctx, uint32_t world, uint32_t rank, uint32_t n_rows, uint32_t head_dim,
                             vfkv_exchange **out)
{
    if (!ctx || !out) return VFKV_ERR_INVALID;
    *out = nullptr;
    if (world == 0 || world > 8 || rank >= world)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_exchange_create: world must be 1..8 and rank below it");
    if (n_rows == 0 || head_dim == 0 || head_dim > 512 || head_dim % 4 != 0)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_exchange_create: head_dim must be a multiple of 4 up to 512");
    Guard g(ctx->device);
    vfkv_exchange *ex = new (std::nothrow) vfkv_exchange();
    if (!ex) return set_error(ctx, VFKV_ERR_OOM, "vfkv_exchange_create: host allocation failed");
    ex->ctx = ctx;
    ex->head_dim = head_dim;
    const uint64_t block = fanout_block_words(n_rows, head_dim);
    ex->bytes = 2ull * world * block * 8;
    cudaError_t e = cudaMalloc(&ex->local, ex->bytes);
    if (e == cudaSuccess) e = cudaMalloc(&ex->ctl, 16);
    if (e == cudaSuccess) e = cudaMalloc(&ex->staging, block * 4);
    if (e == cudaSuccess) e = cudaMemset(ex->local, 0, ex->bytes);
    if (e == cudaSuccess) e = cudaMemset(ex->ctl, 0, 16);
    if (e == cudaSuccess) e = cudaMemset(ex->staging, 0, block * 4);
    if (e != cudaSuccess) {
        cudaGetLastError();
        cudaFree(ex->local); cudaFree(ex->ctl); cudaFree(ex->staging);
        delete ex;
        return set_error(ctx, e == cudaErrorMemoryAllocation ? VFKV_ERR_OOM : VFKV_ERR_CUDA,
                         std::string("vfkv_exchange_create: ") + cudaGetErrorString(e));
    }
    ex->fan.world = world; ex->fan.rank = rank; ex->fan.n_rows = n_rows;
    ex->fan.epoch = ex->ctl;
    ex->fan.ctl = ex->ctl;
    ex->fan.wait_ns = ex->wait_ns;
    ex->fan.base[rank] = ex->local;
    if (cudaMalloc(&ex->d_fan, sizeof(PeerFanout)) != cudaSuccess ||
        cudaMemcpy(ex->d_fan, &ex->fan, sizeof(PeerFanout), cudaMemcpyHostToDevice) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(ex->local); cudaFree(ex->ctl); cudaFree(ex->staging); cudaFree(ex->d_fan);
        delete ex;
        return set_error(ctx, VFKV_ERR_OOM, "vfkv_exchange_create: device allocation failed");
    }
    *out = ex;
    return VFKV_OK;
}

void vfkv_exchange_destroy(vfkv_exchange *ex)
{
    if (!ex) return;
    Guard g(ex->ctx->device);
    for (uint32_t r = 0; r < 8; ++r)
        if (ex->imported[r] && ex->fan.base[r]) cudaIpcCloseMemHandle(ex->fan.base[r]);
    cudaFree(ex->local); cudaFree(ex->ctl); cudaFree(ex->staging); cudaFree(ex->d_fan);
    cudaGetLastError();
    delete ex;
}

uint64_t vfkv_exchange_bytes(const vfkv_exchange *ex) { return ex ? ex->bytes : 0; }

void *vfkv_exchange_local_ptr(const vfkv_exchange *ex) { return ex ? ex->local : nullptr; }

int32_t vfkv_exchange_export(vfkv_exchange *ex, uint8_t handle[64])
{
    if (!ex || !handle) return VFKV_ERR_INVALID;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    Guard g(ex->ctx->device);
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, ex->local);
    if (e != cudaSuccess) return check_cuda(ex->ctx, e, "vfkv_exchange_export");
    std::memcpy(handle, &h, 64);
    return VFKV_OK;
}

int32_t vfkv_exchange_import(vfkv_exchange *ex, uint32_t rank, const uint8_t handle[64])
{
    if (!ex || !handle) return VFKV_ERR_INVALID;
    if (rank >= ex->fan.world || rank == ex->fan.rank)
        return set_error(ex->ctx, VFKV_ERR_INVALID, "vfkv_exchange_import: rank must be another member of the group");
    if (ex->fan.base[rank]) return set_error(ex->ctx, VFKV_ERR_INVALID, "vfkv_exchange_import: rank already set");
    Guard g(ex->ctx->device);
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, 64);
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return check_cuda(ex->ctx, e, "vfkv_exchange_import");
    ex->fan.base[rank] = static_cast<uint64_t *>(p);
    ex->imported[rank] = true;
    return check_cuda(ex->ctx, cudaMemcpy(ex->d_fan, &ex->fan, sizeof(PeerFanout), cudaMemcpyHostToDevice),
                      "vfkv_exchange_import");
}

int32_t vfkv_exchange_set_peer(vfkv_exchange *ex, uint32_t rank, void *d_peer_buffer)
{
    if (!ex || !d_peer_buffer) return VFKV_ERR_INVALID;
    if (rank >= ex->fan.world || rank == ex->fan.rank)
        return set_error(ex->ctx, VFKV_ERR_INVALID, "vfkv_exchange_set_peer: rank must be another member of the group");
    if (reinterpret_cast<uintptr_t>(d_peer_buffer) % 16 != 0)
        return set_error(ex->ctx, VFKV_ERR_INVALID, "vfkv_exchange_set_peer: buffer must be 16-byte aligned");
    ex->fan.base[rank] = static_cast<uint64_t *>(d_peer_buffer);
    ex->imported[rank] = false;
    Guard g(ex->ctx->device);
    return check_cuda(ex->ctx, cudaMemcpy(ex->d_fan, &ex->fan, sizeof(PeerFanout), cudaMemcpyHostToDevice),
                      "vfkv_exchange_set_peer");
}

int32_t vfkv_exchange_set_timeout_ms(vfkv_exchange *ex, uint32_t ms)
{
    if (!ex || ms == 0 || ms > 10000) return VFKV_ERR_INVALID;
    ex->wait_ns = uint64_t(ms) * 1000000ull;
    ex->fan.wait_ns = ex->wait_ns;
    Guard g(ex->ctx->device);
    return check_cuda(ex->ctx, cudaMemcpy(ex->d_fan, &ex->fan, sizeof(PeerFanout), cudaMemcpyHostToDevice),
                      "vfkv_exchange_set_timeout_ms");
}

uint32_t vfkv_exchange_ready(const vfkv_exchange *ex)
{
    if (!ex) return 0;
    for (uint32_t r = 0; r < ex->fan.world; ++r)
        if (!ex->fan.base[r]) return 0;
    return 1;
}

int32_t vfkv_exchange_merge(vfkv_exchange *ex, float *d_out, void *stream)
{
    if (!ex || !d_out) return VFKV_ERR_INVALID;
    vfkv_ctx *ctx = ex->ctx;
    Guard g(ctx->device);
    ProfScope ps(ctx, VFKV_PROF_FA_REDUCE, static_cast<cudaStream_t>(stream));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ex->fan.n_rows);
    cfg.blockDim = dim3(128);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    cudaError_t le = cudaLaunchKernelEx(&cfg, exchange_merge_kernel, ex->fan, static_cast<const uint64_t *>(ex->local),
                                        ex->ctl, ex->head_dim, ex->wait_ns, d_out, ctx->d_status);
    if (le != cudaSuccess) return check_cuda(ctx, le, "exchange_merge launch");
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "exchange_merge launch");
}

}  // extern "C"
