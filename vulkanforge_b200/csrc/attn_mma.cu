// Tensor-core split-K decode attention (placeholder until the kernel lands).
#include "attn_params.cuh"

namespace vfkv {

bool attn_mma_supported(const AttnArgs &) { return false; }

int32_t launch_attn_mma(vfkv_ctx *ctx, vfkv_workspace *, const AttnArgs &, uint32_t, cudaStream_t)
{
    return set_error(ctx, VFKV_ERR_UNSUPPORTED, "tensor-core attention is not built");
}

}  // namespace vfkv
