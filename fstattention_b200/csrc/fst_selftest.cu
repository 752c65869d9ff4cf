// Self-test of the bounded mbarrier wait every TMA / tcgen05 kernel here relies on: a kernel waits
// on a barrier nobody will ever arrive at.  The wait gives up after its time limit (about 50 ms),
// the kernel records FST_DEV_TIMEOUT in the status record and returns; the context stays usable.

#include "fst_attention_tma.cuh"

namespace fst {

__global__ void wait_timeout_kernel(int32_t *status, int32_t *done) {
    __shared__ __align__(8) unsigned long long bar;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(b, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        const bool arrived = mbar_wait(b, 0, status, 12345);      // nobody arrives: runs out
        *done = arrived ? 1 : 2;
    }
}

cudaError_t launch_wait_timeout(int32_t *status, int32_t *done, cudaStream_t stream) {
    wait_timeout_kernel<<<1, 32, 0, stream>>>(status, done);
    return cudaGetLastError();
}

}  // namespace fst
