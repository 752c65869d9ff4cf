// Instantiates the tensor-core tree-attention kernels for bf16, head_dim 64.
#include "fst_attention_persist.cuh"

namespace fst {
cudaError_t launch_mma_bf16_d64(const AttnArgs &a, int variant, cudaStream_t stream) {
    if (variant == FST_KERNEL_PERSIST) return launch_persist_d<__nv_bfloat16, 64>(a, stream);
    if (variant == FST_KERNEL_TMA) {
        if (persist_pays(a)) {                             // many items per SM: the persistent kernel
            const cudaError_t e = launch_persist_d<__nv_bfloat16, 64>(a, stream);
            if (e != cudaErrorNotSupported) return e;
        }
        return launch_tma_d<__nv_bfloat16, 64>(a, 0, stream);
    }
    if (variant == FST_KERNEL_TMA_T32) return launch_tma_d<__nv_bfloat16, 64>(a, 32, stream);
    if (variant == FST_KERNEL_TMA_T64) return launch_tma_d<__nv_bfloat16, 64>(a, 64, stream);
    return launch_mma_d<__nv_bfloat16, 64>(a, variant, stream);
}
cudaError_t launch_combine_bf16_d64(const AttnArgs &a, cudaStream_t stream) {
    return launch_combine_t<__nv_bfloat16, 64>(a, stream);
}
}  // namespace fst
