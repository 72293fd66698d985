// Exchange of softmax partials between the GPUs of a position-sharded group over peer memory.
//
// No counterpart in the reference (it is single-GPU).  The math of the merge is
// vk_shaders/flash_attn_reduce.comp:51-80 over one part per GPU.  Every GPU owns one exchange
// buffer; the attention kernel of rank r stores its (m, l, o) block into the buffer of every rank
// (plain peer stores) and then sets that block's arrival flags with a release at system scope.
// The merge kernel of each rank waits, with a time limit, for the flags of all source ranks in its
// own buffer and reduces the blocks.  Blocks and flags are double-buffered by the parity of the
// exchange number: a rank cannot be more than one exchange ahead of the slowest rank, because its
// own merge needs that rank's flags first.
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

// Copies one staged block into every rank's buffer and publishes its flags (the path of attention
// kernels without the fused fan-out).  One CTA per group so the flag follows that group's rows.
__global__ void __launch_bounds__(256)
fanout_push_kernel(PeerFanout fan, const float *__restrict__ staging, uint32_t head_dim)
{
    const uint32_t group = blockIdx.x;
    const uint32_t g = fan.n_rows / fan.n_groups;
    const FanoutSlot fs = fanout_slot(fan, head_dim, fan.rank, *fan.epoch + 1u);
    const uint64_t o_off = fanout_o_offset(fan.n_rows);
    for (uint32_t idx = threadIdx.x; idx < g * head_dim; idx += blockDim.x) {
        const uint32_t row = group * g + idx / head_dim, d = idx % head_dim;
        const float o = staging[o_off + uint64_t(row) * head_dim + d];
        const float m = staging[row], l = staging[fan.n_rows + row];
#pragma unroll
        for (uint32_t r = 0; r < 8; ++r) {
            if (r < fan.world) {
                float *dst = fan.base[r];
                dst[fs.o + uint64_t(row) * head_dim + d] = o;
                if (d == 0) { dst[fs.m + row] = m; dst[fs.m + fan.n_rows + row] = l; }
            }
        }
    }
    __syncthreads();
    fanout_publish(fan, fs, group);
}

// One CTA per output row.  Thread r < world waits for source rank r's flag of this row's group;
// a wait that runs out sets bit 8 of the status word and the row is written as zeros.
__global__ void __launch_bounds__(128)
exchange_merge_kernel(PeerFanout fan, const float *__restrict__ local, uint32_t *__restrict__ ctl,
                      uint32_t head_dim, uint64_t wait_ns, float *__restrict__ out, uint32_t *__restrict__ status)
{
    __shared__ uint32_t s_bad;
    const uint32_t row = blockIdx.x;
    const uint32_t g = fan.n_rows / fan.n_groups;
    const uint32_t e = ctl[0] + 1u;
    if (threadIdx.x == 0) s_bad = 0u;
    __syncthreads();
    if (threadIdx.x < fan.world) {
        const FanoutSlot fs = fanout_slot(fan, head_dim, threadIdx.x, e);
        const uint32_t *flag = reinterpret_cast<const uint32_t *>(local) + fs.flags + row / g;
        const uint64_t t0 = global_ns();
        for (;;) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if (int32_t(v - e) >= 0) break;
            if (global_ns() - t0 > wait_ns) { atomicOr(&s_bad, 1u); break; }
            __nanosleep(64);
        }
    }
    __syncthreads();
    const bool bad = s_bad != 0u;
    if (bad && threadIdx.x == 0) atomicOr(status, 8u);

    constexpr int kMaxDims = 4;
    float acc[kMaxDims] = {0.f, 0.f, 0.f, 0.f};
    float gmax = kMaskedScore, gsum = 0.f;
    if (!bad) {
        for (uint32_t r = 0; r < fan.world; ++r) {
            const FanoutSlot fs = fanout_slot(fan, head_dim, r, e);
            gmax = fmaxf(gmax, __ldcg(local + fs.m + row));
        }
        for (uint32_t r = 0; r < fan.world; ++r) {
            const FanoutSlot fs = fanout_slot(fan, head_dim, r, e);
            const float kn = __expf(__ldcg(local + fs.m + row) - gmax);
            gsum = fmaf(__ldcg(local + fs.m + fan.n_rows + row), kn, gsum);
#pragma unroll
            for (int j = 0; j < kMaxDims; ++j) {
                const uint32_t d = threadIdx.x + j * 128;
                const float t = d < head_dim ? __ldcg(local + fs.o + uint64_t(row) * head_dim + d) : 0.f;
                acc[j] = fmaf(t, kn, acc[j]);
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
    fanout_push_kernel<<<fan.n_groups, 256, 0, st>>>(fan, staging, head_dim);
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

int32_t vfkv_exchange_create(vfkv_ctx *ctx, uint32_t world, uint32_t rank, uint32_t n_rows, uint32_t n_groups,
                             uint32_t head_dim, vfkv_exchange **out)
{
    if (!ctx || !out) return VFKV_ERR_INVALID;
    *out = nullptr;
    if (world == 0 || world > 8 || rank >= world)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_exchange_create: world must be 1..8 and rank below it");
    if (n_rows == 0 || n_groups == 0 || n_rows % n_groups != 0 || head_dim == 0 || head_dim > 512 || head_dim % 4 != 0)
        return set_error(ctx, VFKV_ERR_INVALID, "vfkv_exchange_create: rows must be a multiple of groups, head_dim a multiple of 4 up to 512");
    Guard g(ctx->device);
    vfkv_exchange *ex = new (std::nothrow) vfkv_exchange();
    if (!ex) return set_error(ctx, VFKV_ERR_OOM, "vfkv_exchange_create: host allocation failed");
    ex->ctx = ctx;
    ex->head_dim = head_dim;
    const uint64_t block = fanout_block_floats(n_rows, head_dim);
    ex->bytes = (2ull * world * block + 2ull * world * n_groups) * 4;
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
    ex->fan.world = world; ex->fan.rank = rank; ex->fan.n_rows = n_rows; ex->fan.n_groups = n_groups;
    ex->fan.epoch = ex->ctl;
    ex->fan.base[rank] = ex->local;
    *out = ex;
    return VFKV_OK;
}

void vfkv_exchange_destroy(vfkv_exchange *ex)
{
    if (!ex) return;
    Guard g(ex->ctx->device);
    for (uint32_t r = 0; r < 8; ++r)
        if (ex->imported[r] && ex->fan.base[r]) cudaIpcCloseMemHandle(ex->fan.base[r]);
    cudaFree(ex->local); cudaFree(ex->ctl); cudaFree(ex->staging);
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
    ex->fan.base[rank] = static_cast<float *>(p);
    ex->imported[rank] = true;
    return VFKV_OK;
}

int32_t vfkv_exchange_set_peer(vfkv_exchange *ex, uint32_t rank, void *d_peer_buffer)
{
    if (!ex || !d_peer_buffer) return VFKV_ERR_INVALID;
    if (rank >= ex->fan.world || rank == ex->fan.rank)
        return set_error(ex->ctx, VFKV_ERR_INVALID, "vfkv_exchange_set_peer: rank must be another member of the group");
    if (reinterpret_cast<uintptr_t>(d_peer_buffer) % 16 != 0)
        return set_error(ex->ctx, VFKV_ERR_INVALID, "vfkv_exchange_set_peer: buffer must be 16-byte aligned");
    ex->fan.base[rank] = static_cast<float *>(d_peer_buffer);
    ex->imported[rank] = false;
    return VFKV_OK;
}

int32_t vfkv_exchange_set_timeout_ms(vfkv_exchange *ex, uint32_t ms)
{
    if (!ex || ms == 0 || ms > 10000) return VFKV_ERR_INVALID;
    ex->wait_ns = uint64_t(ms) * 1000000ull;
    return VFKV_OK;
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
    exchange_merge_kernel<<<ex->fan.n_rows, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        ex->fan, ex->local, ex->ctl, ex->head_dim, ex->wait_ns, d_out, ctx->d_status);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "exchange_merge launch");
}

}  // extern "C"
