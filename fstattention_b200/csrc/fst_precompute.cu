// Tree precompute: parent array -> per-block ancestor list, row-by-ancestor mask, leaf list.
//
// Semantics follow the reference's create_fst_attention_kernel_inputs (utils.py:104-129):
//   A_b   = ascending unique strict ancestors of the rows of block b          (utils.py:119)
//   mask  = [row j][slot a] : A_b[a] is an ancestor of row j, or is row j     (utils.py:124-127)
//   leaf  = rows of the block that are not in A_b, rows past the last node
//           included                                                           (utils.py:121-122)
// The reference gets there with unique / isin over a lineage matrix in Python loops; here one
// CTA per (tree, block) marks ancestors by walking parent links (byte flags in shared memory,
// plain stores: many walkers hit the same few nodes and atomics on one word would serialise),
// packs the flags into a bitmap, ranks the set bits with a popcount prefix scan (which yields
// the ascending order of torch.unique without sorting) and walks each row's chain once more to
// set its mask bits.
// Integer work only; the reference-format outputs are bit-identical to the reference's.
//
// The packed form written for the attention kernels splits A_b in two: ancestors outside the
// block's own rows ("external", gathered row by row) and ancestors inside it, which the kernel
// reads from the block's contiguous K/V rows through a row-by-row bit mask that also carries
// the self bit (the reference's leaf path, utils.py:121-122, and its self-through-mask case,
// utils.py:124-127, become the diagonal of that mask).
//
// Also here: the converter from reference-format metadata tensors to the packed form.

#include <atomic>
#include <climits>

#include "fst_common.cuh"

namespace fst {

constexpr int PRE_THREADS = 256;
constexpr int PRE_WARPS = PRE_THREADS / 32;

// BYTE_FLAGS: ancestors are first marked as one byte per node and packed into the bitmap by
// ballots (the fast path: plain stores never serialise).  Without it the walkers set bitmap bits
// with atomicOr directly; that needs 1/9 of the shared memory and is what lets trees of a
// hundred thousand nodes and more fit (a CTA keeps a bitmap of every node below its last row).
template <bool BYTE_FLAGS>
__global__ void __launch_bounds__(PRE_THREADS)
precompute_kernel(const int32_t *__restrict__ parent_all, int n_nodes, int bm, int ma, int par_cap, int depth_cap,
                  int64_t *__restrict__ anc_idx_all, uint8_t *__restrict__ anc_mask_all,
                  int64_t *__restrict__ leaf_idx_all, unsigned char *__restrict__ packed_all,
                  size_t packed_stride, int32_t *status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int b = blockIdx.x, tree = blockIdx.y, nb = gridDim.x;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int row0 = b * bm;
    const int row_end = row0 + bm;                       // may run past the last node
    const int n_here = min(row_end, n_nodes);            // nodes that exist below row_end
    const int W = (row_end + 31) >> 5;                   // bitmap words, phantom rows included
    const int maw = (ma + 31) >> 5;

    uint32_t *bitmap = reinterpret_cast<uint32_t *>(smem_raw);
    int *rank = reinterpret_cast<int *>(bitmap + W);     // set bits in words below w
    const int bw = (bm + 31) >> 5;
    uint32_t *rowmask = reinterpret_cast<uint32_t *>(rank + W);      // [bm][maw] over all of A_b
    uint32_t *blkmask = rowmask + size_t(bm) * maw;                   // [bm][bw] over block rows
    int *warp_tot = reinterpret_cast<int *>(blkmask + size_t(bm) * bw);
    unsigned char *flag = reinterpret_cast<unsigned char *>(warp_tot + 40);   // [W*32] node is an ancestor
    int *chain = reinterpret_cast<int *>(flag + (BYTE_FLAGS ? size_t(W) * 32 : 0));   // [depth_cap][bm] ancestors of row j
    int *depth = chain + size_t(depth_cap) * bm;                      // [bm] recorded chain length
    int *s_par = depth + bm;

    const int32_t *parent = parent_all + size_t(tree) * n_nodes;
    const int cap = min(par_cap, n_here);
    // parents are checked once, here: a malformed entry is reported and treated as a root, so
    // every walk below ends
    auto checked = [&](int x, int p) -> int {
        if (p >= x || p < -1) {
            report(status, FST_DEV_MALFORMED_TREE, x, p);
            p = -1;
        }
        return p;
    };
    for (int i0 = tid; i0 < cap; i0 += 8 * PRE_THREADS) {    // eight loads in flight per thread
        int v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * PRE_THREADS;
            v[u] = i < cap ? __ldg(parent + i) : -1;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * PRE_THREADS;
            if (i < cap) s_par[i] = checked(i, v[u]);
        }
    }
    if (BYTE_FLAGS) {
        for (int i = tid; i < W * 8; i += PRE_THREADS) reinterpret_cast<uint32_t *>(flag)[i] = 0u;
    } else {
        for (int i = tid; i < W; i += PRE_THREADS) bitmap[i] = 0u;
    }
    for (int i = tid; i < bm * maw; i += PRE_THREADS) rowmask[i] = 0u;
    for (int i = tid; i < bm * bw; i += PRE_THREADS) blkmask[i] = 0u;
    __syncthreads();

    const bool all_staged = cap >= n_here;
    auto par = [&](int x) -> int {
        if (all_staged || x < cap) return s_par[x];
        return checked(x, __ldg(parent + x));
    };

    // 1. every row climbs to its root, recording the chain (its lineage) and flagging each node
    //    as an ancestor.  Flags are bytes written with plain stores: many rows hit the same few
    //    nodes and atomics on one word would serialise.  The loop body is kept minimal because
    //    its length times the depth of the tree is the critical path of this kernel.
    int too_deep = 0;
    for (int j = tid; j < bm; j += PRE_THREADS) {
        const int k = row0 + j;
        int n = 0;
        if (k < n_nodes) {
            int a = par(k);
            while (a >= 0) {
                if (n < depth_cap) chain[n * bm + j] = a;
                if (BYTE_FLAGS) flag[a] = 1;
                else atomicOr(&bitmap[a >> 5], 1u << (a & 31));
                ++n;
                a = par(a);
            }
        }
        depth[j] = n;
        too_deep |= n > depth_cap;
    }
    const bool walk_masks = __syncthreads_or(too_deep) != 0;          // also: flags complete
    // flags -> bitmap, one warp per word
    if (BYTE_FLAGS) {
        for (int w = wid; w < W; w += PRE_WARPS) {
            const uint32_t word = __ballot_sync(0xffffffffu, flag[w * 32 + lane] != 0);
            if (lane == 0) bitmap[w] = word;
        }
        __syncthreads();
    }

    // 2. exclusive popcount scan over the bitmap words -> rank[w]
    const int per = (W + PRE_THREADS - 1) / PRE_THREADS;
    const int w0 = min(W, tid * per), w1 = min(W, w0 + per);
    int mine = 0;
    for (int w = w0; w < w1; ++w) mine += __popc(bitmap[w]);
    int inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
    }
    if (lane == 31) warp_tot[wid] = inc;
    __syncthreads();
    if (wid == 0) {
        const int v = lane < PRE_WARPS ? warp_tot[lane] : 0;
        int iv = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, iv, o);
            if (lane >= o) iv += u;
        }
        warp_tot[lane] = iv - v;
        if (lane == 31) warp_tot[32] = iv;
    }
    __syncthreads();
    {
        int base = warp_tot[wid] + inc - mine;
        for (int w = w0; w < w1; ++w) {
            rank[w] = base;
            base += __popc(bitmap[w]);
        }
    }
    const int n_anc = warp_tot[32];
    const int n_keep = min(n_anc, ma);
    if (n_anc > ma && tid == 0) report(status, FST_DEV_ANCESTOR_OVERFLOW, tree * 65536 + b, n_anc);
    __syncthreads();
    // external ancestors are the ones below row0; they come first in ascending order
    const int n_ext = min(ma, rank[row0 >> 5] + __popc(bitmap[row0 >> 5] & ((1u << (row0 & 31)) - 1u)));

    const PackedLayout L = packed_layout(nb, bm, ma);
    unsigned char *blob = packed_all ? packed_all + size_t(tree) * packed_stride : nullptr;
    int32_t *p_count = blob ? reinterpret_cast<int32_t *>(blob + L.off_count) : nullptr;
    int32_t *p_idx = blob ? reinterpret_cast<int32_t *>(blob + L.off_idx) + size_t(b) * ma : nullptr;
    uint32_t *p_emask = blob ? reinterpret_cast<uint32_t *>(blob + L.off_emask) + size_t(b) * bm * maw
                             : nullptr;
    uint32_t *p_bmask = blob ? reinterpret_cast<uint32_t *>(blob + L.off_bmask) + size_t(b) * bm * bw
                             : nullptr;
    const size_t blk = size_t(tree) * nb + b;
    int64_t *o_idx = anc_idx_all ? anc_idx_all + blk * ma : nullptr;
    uint8_t *o_mask = anc_mask_all ? anc_mask_all + blk * size_t(bm) * ma : nullptr;
    int64_t *o_leaf = leaf_idx_all ? leaf_idx_all + blk * bm : nullptr;

    // 3. ascending ancestor list: slot = rank of the bit; one warp per word, one lane per node
    for (int w = wid; w < W; w += PRE_WARPS) {
        const uint32_t bits = bitmap[w];
        if ((bits >> lane) & 1u) {
            const int pos = rank[w] + __popc(bits & ((1u << lane) - 1u));
            if (pos < ma) {
                const int node = w * 32 + lane;
                if (p_idx && node < row0) p_idx[pos] = node;
                if (o_idx) o_idx[pos] = node;
            }
        }
    }
    if (p_idx)
        for (int a = n_ext + tid; a < ma; a += PRE_THREADS) p_idx[a] = -1;
    if (o_idx)
        for (int a = n_keep + tid; a < ma; a += PRE_THREADS) o_idx[a] = -1;
    if (tid == 0 && p_count) p_count[b] = n_ext;

    // 4. mask rows: bit (row, slot of node) for the row itself, when it is somebody's ancestor
    //    here, and for every node of its chain; plus the same in block-column space.
    if (!walk_masks) {
        // one work item per recorded (row, chain step), spread over all threads
        for (int j = tid; j < bm; j += PRE_THREADS) {
            const int k = row0 + j;
            atomicOr(&blkmask[j * bw + (j >> 5)], 1u << (j & 31));     // every row attends to itself
            if (k < n_nodes && ((bitmap[k >> 5] >> (k & 31)) & 1u)) {
                const int pos = rank[k >> 5] + __popc(bitmap[k >> 5] & ((1u << (k & 31)) - 1u));
                if (pos < ma) atomicOr(&rowmask[j * maw + (pos >> 5)], 1u << (pos & 31));
            }
        }
        int dmax = 0;
        for (int j = lane; j < bm; j += 32) dmax = max(dmax, depth[j]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dmax = max(dmax, __shfl_xor_sync(0xffffffffu, dmax, o));
        for (int i = tid; i < dmax * bm; i += PRE_THREADS) {
            const int sidx = i / bm, j = i - sidx * bm;
            if (sidx < depth[j]) {
                const int x = chain[i];
                const uint32_t word = bitmap[x >> 5];
                const int pos = rank[x >> 5] + __popc(word & ((1u << (x & 31)) - 1u));
                if (pos < ma) atomicOr(&rowmask[j * maw + (pos >> 5)], 1u << (pos & 31));
                if (x >= row0) atomicOr(&blkmask[j * bw + ((x - row0) >> 5)], 1u << ((x - row0) & 31));
            }
        }
    } else {
        // a chain longer than the recording space: walk every row's chain again
        for (int j = tid; j < bm; j += PRE_THREADS) {
            const int k = row0 + j;
            blkmask[j * bw + (j >> 5)] |= 1u << (j & 31);
            if (k < n_nodes) {
                int x = k;
                while (x >= 0) {
                    const uint32_t word = bitmap[x >> 5];
                    const uint32_t bit = 1u << (x & 31);
                    const int up = par(x);
                    if (word & bit) {
                        const int pos = rank[x >> 5] + __popc(word & (bit - 1u));
                        if (pos < ma) rowmask[j * maw + (pos >> 5)] |= 1u << (pos & 31);
                        if (x >= row0) blkmask[j * bw + ((x - row0) >> 5)] |= 1u << ((x - row0) & 31);
                    }
                    x = up;
                }
            }
        }
    }
    __syncthreads();

    if (p_emask) {
        for (int i = tid; i < bm * maw; i += PRE_THREADS) {
            const int w = i % maw, lo = w * 32;           // keep the bits of external slots only
            const uint32_t keep = n_ext >= lo + 32 ? 0xffffffffu : (n_ext > lo ? (1u << (n_ext - lo)) - 1u : 0u);
            p_emask[i] = rowmask[i] & keep;
        }
        for (int i = tid; i < bm * bw; i += PRE_THREADS) p_bmask[i] = blkmask[i];
    }
    if (o_mask) {
        if ((ma & 3) == 0) {                             // four bool bytes per store
            uint32_t *o32 = reinterpret_cast<uint32_t *>(o_mask);
            const int n4 = bm * ma / 4;
            for (int i = tid; i < n4; i += PRE_THREADS) {
                const int e = i * 4, j = e / ma, a = e - j * ma;
                const uint32_t nib = (rowmask[j * maw + (a >> 5)] >> (a & 31)) & 0xFu;
                o32[i] = (nib & 1u) | ((nib & 2u) << 7) | ((nib & 4u) << 14) | ((nib & 8u) << 21);
            }
        } else {
            for (int i = tid; i < bm * ma; i += PRE_THREADS) {
                const int j = i / ma, a = i - j * ma;
                o_mask[i] = (rowmask[j * maw + (a >> 5)] >> (a & 31)) & 1u;
            }
        }
    }

    // 5. leaves: block rows that are not in the ancestor set (rows past the last node too)
    if (o_leaf)
        for (int j = tid; j < bm; j += PRE_THREADS) {
            const int k = row0 + j;
            const bool leaf = !((bitmap[k >> 5] >> (k & 31)) & 1u);
            o_leaf[j] = leaf ? int64_t(k) : int64_t(-1);
        }
}

// -------------------------------------------------------------------------------------------
// reference-format tensors -> packed blob
// -------------------------------------------------------------------------------------------
constexpr int PACK_THREADS = 128;

__global__ void __launch_bounds__(PACK_THREADS)
pack_kernel(const int64_t *__restrict__ anc_idx_all, const uint8_t *__restrict__ anc_mask_all,
            const int64_t *__restrict__ leaf_idx_all, int bm, int ma, int64_t index_base,
            unsigned char *__restrict__ packed_all, size_t packed_stride, int32_t *status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int b = blockIdx.x, tree = blockIdx.y, nb = gridDim.x;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int maw = (ma + 31) >> 5, bw = (bm + 31) >> 5;
    // slot -> external position (>= 0), or -1 - column for an ancestor inside the block, or
    // INT_MIN for padding
    int *slot_map = reinterpret_cast<int *>(smem_raw);               // [ma]
    __shared__ int s_warp[PACK_THREADS / 32];
    __shared__ int s_base;
    if (tid == 0) s_base = 0;
    __syncthreads();

    const PackedLayout L = packed_layout(nb, bm, ma);
    unsigned char *blob = packed_all + size_t(tree) * packed_stride;
    int32_t *p_count = reinterpret_cast<int32_t *>(blob + L.off_count);
    int32_t *p_idx = reinterpret_cast<int32_t *>(blob + L.off_idx) + size_t(b) * ma;
    uint32_t *p_emask = reinterpret_cast<uint32_t *>(blob + L.off_emask) + size_t(b) * bm * maw;
    uint32_t *p_bmask = reinterpret_cast<uint32_t *>(blob + L.off_bmask) + size_t(b) * bm * bw;
    const size_t blk = size_t(tree) * nb + b;
    const int64_t *g_idx = anc_idx_all + blk * ma;
    const uint8_t *g_mask = anc_mask_all + blk * size_t(bm) * ma;
    const int64_t *g_leaf = leaf_idx_all + blk * bm;
    const int64_t row0 = int64_t(b) * bm;

    // external slots keep their order; an exclusive scan of the "is external" flags places them
    for (int a0 = 0; a0 < ma; a0 += PACK_THREADS) {
        const int a = a0 + tid;
        bool ext = false;
        int node = -1;
        int code = INT_MIN;
        if (a < ma) {
            const int64_t v = g_idx[a];
            const int64_t rel = v - index_base;
            if (v >= 0 && rel >= 0) {
                if (rel > 0x7fffffffLL) {
                    report(status, FST_DEV_INDEX_RANGE, tree * 65536 + b, a);
                } else if (rel >= row0 && rel < row0 + bm) {
                    code = -1 - int(rel - row0);
                } else {
                    ext = true;
                    node = int(rel);
                }
            }
        }
        const uint32_t votes = __ballot_sync(0xffffffffu, ext);
        if (lane == 0) s_warp[wid] = __popc(votes);
        __syncthreads();
        int pos = s_base + __popc(votes & ((1u << lane) - 1u));
        for (int w = 0; w < wid; ++w) pos += s_warp[w];
        if (ext) {
            code = pos;
            p_idx[pos] = node;
        }
        if (a < ma) slot_map[a] = code;
        __syncthreads();
        if (tid == 0) {
            int add = 0;
            for (int w = 0; w < PACK_THREADS / 32; ++w) add += s_warp[w];
            s_base += add;
        }
        __syncthreads();
    }
    const int n_ext = s_base;
    for (int a = n_ext + tid; a < ma; a += PACK_THREADS) p_idx[a] = -1;
    if (tid == 0) p_count[b] = n_ext;

    // one thread per row: scatter its mask bytes into the two bit masks
    for (int j = tid; j < bm; j += PACK_THREADS) {
        uint32_t *er = p_emask + size_t(j) * maw, *br = p_bmask + size_t(j) * bw;
        for (int w = 0; w < maw; ++w) er[w] = 0u;
        for (int w = 0; w < bw; ++w) br[w] = 0u;
        const int64_t leaf = g_leaf[j];
        const bool is_leaf = leaf >= 0 && leaf >= index_base;
        if (is_leaf && leaf - index_base != row0 + j)
            report(status, FST_DEV_INDEX_RANGE, tree * 65536 + b, -1 - j);
        if (is_leaf) br[j >> 5] |= 1u << (j & 31);
        const uint8_t *src = g_mask + size_t(j) * ma;
        for (int a = 0; a < ma; ++a) {
            if (!src[a]) continue;
            const int code = slot_map[a];
            if (code >= 0) er[code >> 5] |= 1u << (code & 31);
            else if (code != INT_MIN) br[(-1 - code) >> 5] |= 1u << ((-1 - code) & 31);
        }
    }
}

// largest dynamic shared memory enabled so far, per device and kernel variant
static std::atomic<size_t> g_pre_smem_set[2][kMaxDevices];
static std::atomic<size_t> g_pack_smem_set[kMaxDevices];

cudaError_t launch_precompute(const int32_t *parent, int n_trees, int n_nodes, int bm, int ma,
                              int64_t *anc_idx, uint8_t *anc_mask, int64_t *leaf_idx,
                              void *packed, size_t packed_stride, int32_t *status,
                              cudaStream_t stream) {
    const int nb = (n_nodes + bm - 1) / bm;
    const int maw = (ma + 31) / 32;
    const size_t W = (size_t(nb) * bm + 31) / 32;
    const size_t budget = 200 * 1024;
    // bitmap + ranks + the two row masks + scan scratch + chain lengths
    const size_t base = (2 * W + size_t(bm) * maw + size_t(bm) * ((bm + 31) / 32) + 40 + size_t(bm)) * 4;
    // recording space for the rows' chains: as deep as 48 KB allows, at most 1024 levels
    int depth_cap = int((48 * 1024) / (size_t(bm) * 4));
    if (depth_cap > 1024) depth_cap = 1024;
    if (depth_cap < 1) depth_cap = 1;
    // Byte flags (one byte per node below the last row) while they leave room to stage a good
    // part of the parent array; beyond that the walkers set bitmap bits with atomics.
    bool byte_flags = base + W * 32 + size_t(depth_cap) * bm * 4 + 16 * 1024 <= budget;
    size_t fixed = base + (byte_flags ? W * 32 : 0) + size_t(depth_cap) * bm * 4;
    while (fixed + 1024 > budget && depth_cap > 1) {     // a tight budget: record shallower chains
        depth_cap = depth_cap / 2;                         // (deeper rows are walked a second time)
        fixed = base + size_t(depth_cap) * bm * 4;
    }
    if (fixed + 1024 > budget) return cudaErrorInvalidConfiguration;
    const size_t cap = (budget - fixed) / 4;
    const int par_cap = int(cap < size_t(n_nodes) ? cap : size_t(n_nodes));
    const size_t smem = fixed + size_t(par_cap) * 4;
    const int slot = current_device_slot();
    if (slot < 0) return cudaErrorInvalidDevice;
    auto kernel = byte_flags ? precompute_kernel<true> : precompute_kernel<false>;
    std::atomic<size_t> &enabled = g_pre_smem_set[byte_flags ? 1 : 0][slot];
    if (smem > 48 * 1024 && smem > enabled.load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        enabled.store(smem, std::memory_order_release);
    }
    dim3 grid(nb, n_trees);
    kernel<<<grid, PRE_THREADS, smem, stream>>>(
        parent, n_nodes, bm, ma, par_cap, depth_cap, anc_idx, anc_mask, leaf_idx,
        static_cast<unsigned char *>(packed), packed_stride, status);
    return cudaGetLastError();
}

cudaError_t launch_pack(const int64_t *anc_idx, const uint8_t *anc_mask, const int64_t *leaf_idx,
                        int n_trees, int nb, int bm, int ma, int64_t index_base, void *packed,
                        size_t packed_stride, int32_t *status, cudaStream_t stream) {
    const size_t smem = size_t(ma) * 4;
    const int slot = current_device_slot();
    if (slot < 0) return cudaErrorInvalidDevice;
    if (smem > 48 * 1024 && smem > g_pack_smem_set[slot].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(pack_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        g_pack_smem_set[slot].store(smem, std::memory_order_release);
    }
    dim3 grid(nb, n_trees);
    pack_kernel<<<grid, PACK_THREADS, smem, stream>>>(
        anc_idx, anc_mask, leaf_idx, bm, ma, index_base, static_cast<unsigned char *>(packed),
        packed_stride, status);
    return cudaGetLastError();
}

}  // namespace fst
