// Depth-first renumbering of a tree on the device.
//
// The reference leaves node ordering as a TODO (README.md:19-20): its precompute
// (utils.py:104-129) takes whatever numbering the caller has, and with a breadth-first numbering
// a 64-row block of a deep tree has ancestors all over the tree.  Numbered depth first (pre-order,
// children in their old relative order) a block is a few root-to-leaf paths and gathers a
// fraction of the rows.  This kernel computes that numbering from a parent array that is already
// on the GPU, so a decoder that builds its tree on the device never goes back to the host:
//     order[i]      = old index of the node that becomes node i
//     new_parent[i] = its parent in the new numbering (still < i, or -1)
// One CTA per tree, everything in shared memory, integer arithmetic only:
//   1. size[a] = nodes in the subtree of a: every node climbs to its root adding one on the way;
//   2. off[i]  = sizes of the siblings of i with a smaller index (roots are siblings of one
//      another): one warp sweeps the nodes in index order, 32 at a time, keeping a running sum
//      per parent;
//   3. pos[i]  = off[i] + sum over the ancestors a of i of (off[a] + 1): a second climb;
//   4. scatter.
// A malformed parent (parent[i] >= i or < -1) is reported through the status record and the
// outputs are left untouched.

#include "fst_common.cuh"

namespace fst {

constexpr int REORDER_THREADS = 512;
constexpr int REORDER_MAX_NODES = 8192;                   // four int arrays of that many nodes in shared memory

__global__ void __launch_bounds__(REORDER_THREADS)
dfs_order_kernel(const int32_t *__restrict__ parent, int n, int32_t *__restrict__ order,
                 int32_t *__restrict__ new_parent, int32_t *status) {
    extern __shared__ int32_t rs[];
    int32_t *par = rs;                                    // [n]
    int32_t *size = par + n;                              // [n]   subtree sizes, later final positions
    int32_t *off = size + n;                              // [n]
    int32_t *acc = off + n;                               // [n+1] running sum per parent; slot n = the roots
    __shared__ int bad;
    const int tree = blockIdx.x, tid = threadIdx.x;
    const int32_t *src = parent + size_t(tree) * n;
    if (tid == 0) bad = 0;
    __syncthreads();
    for (int i = tid; i < n; i += REORDER_THREADS) {
        const int32_t p = src[i];
        if (p >= i || p < -1) {
            report(status, FST_DEV_MALFORMED_TREE, i, int(p));
            bad = 1;
        }
        par[i] = p;
        size[i] = 1;
        acc[i] = 0;
    }
    if (tid == 0) acc[n] = 0;
    __syncthreads();
    if (bad) return;                                      // the climbs below rely on parent[i] < i

    for (int i = tid; i < n; i += REORDER_THREADS)
        for (int32_t a = par[i]; a >= 0; a = par[a]) atomicAdd(&size[a], 1);
    __syncthreads();

    if (tid < 32) {
        const int lane = tid;
        for (int base = 0; base < n; base += 32) {
            const int i = base + lane;
            const int32_t p = i < n ? par[i] : -2;        // -2 matches no real parent
            const int32_t sz = i < n ? size[i] : 0;
            int32_t before = 0, total = 0;
            bool first = true;                            // lowest lane of its sibling group
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int32_t pj = __shfl_sync(0xffffffffu, p, j), sj = __shfl_sync(0xffffffffu, sz, j);
                if (pj == p) {
                    total += sj;
                    if (j < lane) {
                        before += sj;
                        first = false;
                    }
                }
            }
            const int slot = p < 0 ? n : p;
            if (i < n) off[i] = acc[slot] + before;
            __syncwarp();
            if (i < n && first) acc[slot] += total;
            __syncwarp();
        }
    }
    __syncthreads();

    int32_t mine[REORDER_MAX_NODES / REORDER_THREADS];    // my nodes' positions (size[] is still being read)
#pragma unroll
    for (int k = 0; k < REORDER_MAX_NODES / REORDER_THREADS; ++k) {
        const int i = tid + k * REORDER_THREADS;
        int32_t s = 0;
        if (i < n) {
            s = off[i];
            for (int32_t a = par[i]; a >= 0; a = par[a]) s += off[a] + 1;
        }
        mine[k] = s;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < REORDER_MAX_NODES / REORDER_THREADS; ++k) {
        const int i = tid + k * REORDER_THREADS;
        if (i < n) size[i] = mine[k];                     // size[] now holds positions
    }
    __syncthreads();
    int32_t *ord = order + size_t(tree) * n, *npar = new_parent + size_t(tree) * n;
    for (int i = tid; i < n; i += REORDER_THREADS) {
        const int32_t at = size[i], p = par[i];
        ord[at] = i;
        npar[at] = p < 0 ? -1 : size[p];
    }
}

cudaError_t launch_dfs_order(const int32_t *parent, int n_trees, int n_nodes, int32_t *order,
                             int32_t *new_parent, int32_t *status, cudaStream_t stream) {
    if (n_nodes > REORDER_MAX_NODES) return cudaErrorInvalidValue;
    const size_t smem = (size_t(n_nodes) * 4 + 1) * sizeof(int32_t);
    static std::atomic<size_t> enabled[kMaxDevices];      // largest dynamic shared memory enabled, per device
    const int slot = current_device_slot();
    if (slot < 0) return cudaErrorInvalidDevice;
    if (smem > 48 * 1024 && smem > enabled[slot].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(dfs_order_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        enabled[slot].store(smem, std::memory_order_release);
    }
    dfs_order_kernel<<<n_trees, REORDER_THREADS, smem, stream>>>(parent, n_nodes, order, new_parent, status);
    return cudaGetLastError();
}

}  // namespace fst
