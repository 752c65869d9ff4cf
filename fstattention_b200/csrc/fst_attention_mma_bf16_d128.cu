// Instantiates the tensor-core tree-attention kernel for bf16, head_dim 128.
#include "fst_attention_mma.cuh"

namespace fst {
cudaError_t launch_mma_bf16_d128(const AttnArgs &a, int variant, cudaStream_t stream) {
    return launch_mma_d<__nv_bfloat16, 128>(a, variant, stream);
}
}  // namespace fst
