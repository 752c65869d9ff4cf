// Shared declarations for the fstattn_b200 kernels: packed-metadata layout, status record,
// small device helpers.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <stdint.h>
#include <stddef.h>

#include "../../include/fstattn_b200.h"

namespace fst {

// Offsets (bytes) of the four arrays inside one packed-metadata blob.
//   count[nb]            external ancestors of the block (nodes outside the block's own rows)
//   idx  [nb][ma]        their node indices, ascending, -1 padded
//   emask[nb][bm][maw]   bit a of row j: row j attends to external ancestor slot a
//   bmask[nb][bm][bw]    bit c of row j: row j attends to row c of its own block (c == j always
//                        set; other bits are ancestors that live inside the block)
struct PackedLayout {
    int nb, bm, ma, maw, bw;
    size_t off_count, off_idx, off_emask, off_bmask, total;
};

__host__ __device__ inline size_t align16(size_t x) { return (x + 15) & ~size_t(15); }

__host__ __device__ inline PackedLayout packed_layout(int nb, int bm, int ma) {
    PackedLayout L;
    L.nb = nb; L.bm = bm; L.ma = ma;
    L.maw = (ma + 31) / 32;
    L.bw = (bm + 31) / 32;
    L.off_count = 0;
    L.off_idx = align16(size_t(nb) * 4);
    L.off_emask = L.off_idx + align16(size_t(nb) * ma * 4);
    L.off_bmask = L.off_emask + align16(size_t(nb) * bm * L.maw * 4);
    L.total = L.off_bmask + align16(size_t(nb) * bm * L.bw * 4);
    return L;
}

// First error wins; later ones are dropped.
__device__ inline void report(int32_t *status, int code, int where, int detail) {
    if (status == nullptr) return;
    if (atomicCAS(status, 0, code) == 0) {
        status[1] = where;
        status[2] = detail;
    }
}

// Index of the current device, for per-device caches of launch configuration (a function
// attribute set on one device says nothing about another).  -1 when it cannot be told.
constexpr int kMaxDevices = 64;
inline int current_device_slot() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
    return dev;
}

// One-time per-device launch set-up of a kernel instantiation (the dynamic shared memory
// attribute is per device); safe from several host threads.
struct DeviceOnce {
    // (static storage: zero-initialised)
    std::atomic<bool> done[kMaxDevices];
    template <typename F>
    cudaError_t run(F &&f) {
        const int slot = current_device_slot();
        if (slot < 0) return cudaErrorInvalidDevice;
        if (done[slot].load(std::memory_order_acquire)) return cudaSuccess;
        const cudaError_t e = f();                        // idempotent: a second thread may repeat it
        if (e == cudaSuccess) done[slot].store(true, std::memory_order_release);
        return e;
    }
};

// Kernel launchers (defined in the .cu files, called from fst_api.cu)
cudaError_t launch_precompute(const int32_t *parent, int n_trees, int n_nodes, int bm, int ma,
                              int64_t *anc_idx, uint8_t *anc_mask, int64_t *leaf_idx,
                              void *packed, size_t packed_stride, int32_t *status,
                              cudaStream_t stream);

cudaError_t launch_wait_timeout(int32_t *status, int32_t *done, cudaStream_t stream);

cudaError_t launch_dfs_order(const int32_t *parent, int n_trees, int n_nodes, int32_t *order,
                             int32_t *new_parent, int32_t *status, cudaStream_t stream);

// levels (depth + 1) a device-built forest may have
constexpr int kMaxTreeLevels = 32;
long long tree_topk_nodes(int depth, int topk, double left_weight_factor);
cudaError_t launch_build_tree_topk(const float *scores, int n_trees, int depth, int topk,
                                   double left_weight_factor, int max_nodes, int32_t *parent, int32_t *choice,
                                   float *node_score, cudaStream_t stream);

cudaError_t launch_pack(const int64_t *anc_idx, const uint8_t *anc_mask, const int64_t *leaf_idx,
                        int n_trees, int nb, int bm, int ma, int64_t index_base, void *packed,
                        size_t packed_stride, int32_t *status, cudaStream_t stream);

struct AttnArgs {
    const void *q, *k, *v;
    void *o;
    float *lse;
    const unsigned char *packed;
    size_t meta_stride;
    int Z, H, n_q, n_kv, D, prefix;
    int kv_group;          // query heads per K/V head (grouped-query attention); K and V have H / kv_group heads
    int64_t qs_z, qs_h, qs_n, ks_z, ks_h, ks_n, vs_z, vs_h, vs_n, os_z, os_h, os_n;
    int bm, ma, nb;
    float scale_log2;      // sm_scale * log2(e)
    int32_t *status;
    // split of the shared prefix over n_splits CTAs per (block, head, batch): partial outputs
    // [n_splits][Z][H][n_q][D] (float, normalised) and their base-2 log-sum-exps; 1 = no split
    int n_splits;
    float *part_o;
    float *part_lse;
    // skip_prefix: the tree kernel leaves the prefix to the tcgen05 prefix kernel and writes its
    // own result as partial slot 0; part_slots: how many partial slots the merge kernel reads
    int skip_prefix;
    int part_slots;
    // the packed metadata was complete before the launch ahead of this one in the stream began:
    // a kernel launched with programmatic stream serialisation may read it before its dependency wait
    int meta_stable;
    // grid order of the TMA tree kernel: heads fastest and blocks from the last one down (grids of a few waves)
    int heads_first;
    // Delivery of the output to every GPU of a sharded problem (n_out > 0): o_ranks[r] is rank r's
    // copy of the full output tensor [out_Z][out_H][n_q][D] as mapped into this process, os_*
    // are that tensor's strides, and this call's (z, h) land at (z + out_z0, h + out_h0).
    int n_out, out_rank, out_z0, out_h0, out_Z, out_H;      // out_rank: which of o_ranks is this GPU's own
    const void *o_ranks[8];
};
constexpr int kMaxRanks = 8;

// Prefix rows held in a page pool (a KV cache): pages of page_size rows, pool strides in elements.
struct PagedArgs {
    const void *k_pool, *v_pool;
    const int32_t *block_table;          // [Z][table_stride] page numbers
    const int32_t *prefix_lens;          // [Z] prefix rows of every batch element
    int table_stride, page_size, n_pages;
    int64_t stride_page, stride_row, stride_head;
};

cudaError_t launch_attention_simt(const AttnArgs &a, int dtype, cudaStream_t stream);
// returns cudaErrorNotSupported when no tensor-core instantiation fits
cudaError_t launch_attention_mma(const AttnArgs &a, int dtype, int variant, cudaStream_t stream);
// dense prefix on tcgen05: partial results of n_runs runs into slots first_slot..; D = 64 or 128
cudaError_t launch_prefix_umma(const AttnArgs &a, int dtype, int n_runs, int first_slot, cudaStream_t stream);
cudaError_t launch_prefix_umma_paged(const AttnArgs &a, const PagedArgs &pg, int dtype, int n_runs, int first_slot,
                                     cudaStream_t stream);
// merge a.part_slots partial results into o (and lse)
cudaError_t launch_combine(const AttnArgs &a, int dtype, cudaStream_t stream);

}  // namespace fst
