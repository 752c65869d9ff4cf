// Instantiates the tensor-core tree-attention kernel for bf16, head_dim 64.
#include "fst_attention_mma.cuh"

namespace fst {
cudaError_t launch_mma_bf16_d64(const AttnArgs &a, int variant, cudaStream_t stream) {
    return launch_mma_d<__nv_bfloat16, 64>(a, variant, stream);
}
}  // namespace fst
