// C ABI of fstattn_b200: argument checks and kernel dispatch.  See include/fstattn_b200.h.
#include <atomic>
#include <cmath>
#include <cstdio>

#include "fst_common.cuh"

namespace fst {
cudaError_t launch_mma_f16_d64(const AttnArgs &, int, cudaStream_t);
cudaError_t launch_mma_f16_d128(const AttnArgs &, int, cudaStream_t);
cudaError_t launch_mma_bf16_d64(const AttnArgs &, int, cudaStream_t);
cudaError_t launch_mma_bf16_d128(const AttnArgs &, int, cudaStream_t);
cudaError_t launch_combine_f16_d64(const AttnArgs &, cudaStream_t);
cudaError_t launch_combine_f16_d128(const AttnArgs &, cudaStream_t);
cudaError_t launch_combine_bf16_d64(const AttnArgs &, cudaStream_t);
cudaError_t launch_combine_bf16_d128(const AttnArgs &, cudaStream_t);

cudaError_t launch_combine(const AttnArgs &a, int dtype, cudaStream_t stream) {
    if (dtype == FST_F16 && a.D == 64) return launch_combine_f16_d64(a, stream);
    if (dtype == FST_F16 && a.D == 128) return launch_combine_f16_d128(a, stream);
    if (dtype == FST_BF16 && a.D == 64) return launch_combine_bf16_d64(a, stream);
    if (dtype == FST_BF16 && a.D == 128) return launch_combine_bf16_d128(a, stream);
    return cudaErrorNotSupported;
}

cudaError_t launch_attention_mma(const AttnArgs &a, int dtype, int variant, cudaStream_t stream) {
    if (dtype == FST_F16 && a.D == 64) return launch_mma_f16_d64(a, variant, stream);
    if (dtype == FST_F16 && a.D == 128) return launch_mma_f16_d128(a, variant, stream);
    if (dtype == FST_BF16 && a.D == 64) return launch_mma_bf16_d64(a, variant, stream);
    if (dtype == FST_BF16 && a.D == 128) return launch_mma_bf16_d128(a, variant, stream);
    return cudaErrorNotSupported;
}

static int elem_size(int dtype) { return dtype == FST_F32 ? 4 : 2; }
static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
static bool mma_ok(int dtype, int D, int bm) {
    return (dtype == FST_F16 || dtype == FST_BF16) && (D == 64 || D == 128) &&
           (bm == 16 || bm == 32 || bm == 64 || bm == 128);
}

// A second stream with a fork and a join event, per host thread and device, so that two
// independent kernels of one call can run side by side.  Created on first use and kept for the
// life of the thread; never created while the caller's stream is being captured into a graph
// (the call then simply runs its kernels in order).
struct SideStream {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
};
static SideStream *side_stream(cudaStream_t caller) {
    thread_local SideStream per_device[kMaxDevices];
    const int slot = current_device_slot();
    if (slot < 0) return nullptr;
    SideStream &s = per_device[slot];
    if (s.stream != nullptr) return &s;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(caller, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
        (void)cudaGetLastError();
        return nullptr;
    }
    SideStream made;
    if (cudaStreamCreateWithFlags(&made.stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&made.fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&made.join, cudaEventDisableTiming) != cudaSuccess) {
        if (made.join != nullptr) cudaEventDestroy(made.join);
        if (made.fork != nullptr) cudaEventDestroy(made.fork);
        if (made.stream != nullptr) cudaStreamDestroy(made.stream);
        (void)cudaGetLastError();
        return nullptr;
    }
    s = made;
    return &s;
}

static int cuda_status(cudaError_t e) {
    if (e == cudaSuccess) return FST_OK;
    if (e == cudaErrorNotSupported) return FST_ERR_UNSUPPORTED;
    if (e == cudaErrorInvalidConfiguration) return FST_ERR_TOO_LARGE;   // what a launcher returns when the sizes do not fit an SM
    return FST_ERR_CUDA;
}
}  // namespace fst

using namespace fst;

// Scratch for fst_attention_fwd_ref_static: lives in the library's device image, so every GPU
// that loads the library carries these bytes until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[FST_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch on the current device.  In host code the array's name is
// only a handle for the runtime, not something a kernel can dereference, so the address is
// asked for once per device and remembered.
static int static_scratch_address(void **out) {
    static std::atomic<void *> cached[kMaxDevices];       // two threads racing here store the same address
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FST_ERR_CUDA;
    void *ptr = cached[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr)
            return FST_ERR_CUDA;
        cached[dev].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return FST_OK;
}

extern "C" {

int fst_version(void) { return FST_VERSION; }

const char *fst_status_string(int s) {
    switch (s) {
        case FST_OK: return "ok";
        case FST_ERR_INVALID_ARG: return "invalid argument";
        case FST_ERR_UNSUPPORTED: return "unsupported dtype / head_dim / block_m combination";
        case FST_ERR_ALIGNMENT: return "pointer or stride not 16-byte aligned";
        case FST_ERR_WORKSPACE: return "workspace too small";
        case FST_ERR_CUDA: return "CUDA runtime error";
        case FST_ERR_TOO_LARGE: return "size beyond the supported limit (or beyond the built-in scratch)";
        case FST_DEV_MALFORMED_TREE: return "malformed tree: parent[i] must be -1 or an earlier node";
        case FST_DEV_ANCESTOR_OVERFLOW: return "a block has more unique ancestors than max_ancestors";
        case FST_DEV_INDEX_RANGE: return "metadata index outside the K/V rows";
        case FST_DEV_TIMEOUT: return "a bounded wait on an asynchronous copy ran out";
        default: return "unknown status";
    }
}

size_t fst_packed_meta_bytes(int n_blocks, int block_m, int max_ancestors) {
    if (n_blocks <= 0 || block_m <= 0 || max_ancestors <= 0) return 0;
    return packed_layout(n_blocks, block_m, max_ancestors).total;
}

int fst_precompute(const int32_t *parent, int n_trees, int n_nodes, int block_m, int max_ancestors,
                   int64_t *ancestor_idx, uint8_t *ancestor_mask, int64_t *leaf_idx, void *packed,
                   size_t packed_tree_stride, int32_t *status, void *stream) {
    if (!parent || n_trees <= 0 || n_nodes <= 0 || block_m <= 0 || max_ancestors <= 0)
        return FST_ERR_INVALID_ARG;
    if (block_m > 1024 || n_nodes > 262144 || n_trees > 65535 || max_ancestors > 65536)
        return FST_ERR_TOO_LARGE;
    if (size_t(block_m) * ((max_ancestors + 31) / 32) * 4 > 64 * 1024) return FST_ERR_TOO_LARGE;
    const int nb = (n_nodes + block_m - 1) / block_m;
    if (packed) {
        if (!aligned16(packed) || (packed_tree_stride & 15)) return FST_ERR_ALIGNMENT;
        if (n_trees > 1 && packed_tree_stride < packed_layout(nb, block_m, max_ancestors).total)
            return FST_ERR_INVALID_ARG;
    }
    if ((max_ancestors & 3) == 0 && ancestor_mask && (reinterpret_cast<uintptr_t>(ancestor_mask) & 3))
        return FST_ERR_ALIGNMENT;
    return cuda_status(launch_precompute(parent, n_trees, n_nodes, block_m, max_ancestors,
                                         ancestor_idx, ancestor_mask, leaf_idx, packed,
                                         packed_tree_stride, status,
                                         static_cast<cudaStream_t>(stream)));
}

int fst_selftest_wait_timeout(int32_t *status, int32_t *done, void *stream) {
    if (!status || !done) return FST_ERR_INVALID_ARG;
    return cuda_status(launch_wait_timeout(status, done, static_cast<cudaStream_t>(stream)));
}

int fst_dfs_order(const int32_t *parent, int n_trees, int n_nodes, int32_t *order,
                  int32_t *new_parent, int32_t *status, void *stream) {
    if (!parent || !order || !new_parent || n_trees <= 0 || n_nodes <= 0) return FST_ERR_INVALID_ARG;
    if (n_nodes > 8192 || n_trees > 65535) return FST_ERR_TOO_LARGE;
    return cuda_status(launch_dfs_order(parent, n_trees, n_nodes, order, new_parent, status,
                                        static_cast<cudaStream_t>(stream)));
}

long long fst_tree_topk_nodes(int depth, int topk, double left_weight_factor) {
    if (!(left_weight_factor >= 0.0) || !(left_weight_factor <= 1.0)) return -1;
    return tree_topk_nodes(depth, topk, left_weight_factor);
}

int fst_build_tree_topk(const float *scores, int n_trees, int depth, int topk, double left_weight_factor,
                        int max_nodes, int32_t *parent, int32_t *choice, float *node_score, void *stream) {
    if (!scores || !parent || n_trees <= 0 || depth < 0 || topk <= 0 || max_nodes <= 0 ||
        !(left_weight_factor >= 0.0) || !(left_weight_factor <= 1.0))
        return FST_ERR_INVALID_ARG;
    if (n_trees > 65535 || depth + 1 > kMaxTreeLevels || tree_topk_nodes(depth, topk, left_weight_factor) < 0)
        return FST_ERR_TOO_LARGE;
    return cuda_status(launch_build_tree_topk(scores, n_trees, depth, topk, left_weight_factor, max_nodes,
                                              parent, choice, node_score, static_cast<cudaStream_t>(stream)));
}

int fst_pack_metadata(const int64_t *ancestor_idx, const uint8_t *ancestor_mask,
                      const int64_t *leaf_idx, int n_trees, int n_blocks, int block_m,
                      int max_ancestors, int64_t index_base, void *packed,
                      size_t packed_tree_stride, int32_t *status, void *stream) {
    if (!ancestor_idx || !ancestor_mask || !leaf_idx || !packed || n_trees <= 0 || n_blocks <= 0 ||
        block_m <= 0 || max_ancestors <= 0)
        return FST_ERR_INVALID_ARG;
    if (n_trees > 65535 || max_ancestors > 32768) return FST_ERR_TOO_LARGE;   // one slot map per CTA in shared memory
    if (!aligned16(packed) || (packed_tree_stride & 15)) return FST_ERR_ALIGNMENT;
    if (n_trees > 1 && packed_tree_stride < packed_layout(n_blocks, block_m, max_ancestors).total)
        return FST_ERR_INVALID_ARG;
    return cuda_status(launch_pack(ancestor_idx, ancestor_mask, leaf_idx, n_trees, n_blocks, block_m,
                                   max_ancestors, index_base, packed, packed_tree_stride, status,
                                   static_cast<cudaStream_t>(stream)));
}

size_t fst_attention_split_workspace_bytes(int Z, int H, int n_q, int head_dim, int kv_splits) {
    if (Z <= 0 || H <= 0 || n_q <= 0 || head_dim <= 0 || kv_splits < 1) return 0;
    return size_t(kv_splits + 1) * Z * H * n_q * (size_t(head_dim) + 1) * sizeof(float);
}

// where a call's output goes when it is delivered to every rank of a sharded problem
struct ScatterTo {
    void *const *o_ranks;
    int n_ranks, rank, z0, h0, Z_total, H_total;
};

static int attention_fwd_impl(const void *q, const void *k, const void *v, void *o, float *lse,
                      const void *packed, size_t meta_tree_stride, int Z, int H, int H_kv, int n_q, int n_kv,
                      int head_dim, int64_t q_stride_z, int64_t q_stride_h, int64_t q_stride_n,
                      int64_t k_stride_z, int64_t k_stride_h, int64_t k_stride_n,
                      int64_t v_stride_z, int64_t v_stride_h, int64_t v_stride_n,
                      int64_t o_stride_z, int64_t o_stride_h, int64_t o_stride_n, int block_m,
                      int max_ancestors, float sm_scale, int dtype, int kernel, int kv_splits,
                      void *workspace, size_t workspace_bytes, int32_t *status, void *stream,
                      const ScatterTo *scatter = nullptr) {
    if (!q || !k || !v || !o || !packed || Z <= 0 || H <= 0 || n_q <= 0 || n_kv < n_q ||
        block_m <= 0 || max_ancestors <= 0)
        return FST_ERR_INVALID_ARG;
    if (dtype != FST_F16 && dtype != FST_BF16 && dtype != FST_F32) return FST_ERR_INVALID_ARG;
    if (head_dim != 16 && head_dim != 32 && head_dim != 64 && head_dim != 128)
        return FST_ERR_UNSUPPORTED;                       // the reference's set, fstattention.py:157
    if (H > 65535 || Z > 65535) return FST_ERR_TOO_LARGE;
    if (H_kv <= 0 || H % H_kv != 0) return FST_ERR_INVALID_ARG;
    if (!aligned16(packed) || (meta_tree_stride & 15)) return FST_ERR_ALIGNMENT;
    if (!std::isfinite(sm_scale)) return FST_ERR_INVALID_ARG;   // any finite factor is fine, either sign (fstattention.py:78)
    const int flags = kernel & ~FST_KERNEL_MASK;
    kernel &= FST_KERNEL_MASK;
    if (flags & ~FST_KERNEL_FLAG_META_STABLE) return FST_ERR_INVALID_ARG;

    AttnArgs a = {};
    a.q = q; a.k = k; a.v = v; a.o = o; a.lse = lse;
    a.packed = static_cast<const unsigned char *>(packed);
    a.meta_stride = meta_tree_stride;
    a.Z = Z; a.H = H; a.n_q = n_q; a.n_kv = n_kv; a.D = head_dim; a.prefix = n_kv - n_q;
    a.kv_group = H / H_kv;
    a.qs_z = q_stride_z; a.qs_h = q_stride_h; a.qs_n = q_stride_n;
    a.ks_z = k_stride_z; a.ks_h = k_stride_h; a.ks_n = k_stride_n;
    a.vs_z = v_stride_z; a.vs_h = v_stride_h; a.vs_n = v_stride_n;
    a.os_z = o_stride_z; a.os_h = o_stride_h; a.os_n = o_stride_n;
    a.bm = block_m; a.ma = max_ancestors; a.nb = (n_q + block_m - 1) / block_m;
    // A factor of zero would turn the -inf of a masked score into NaN inside the exponent's
    // multiply-add; a factor too small to move any finite score gives the same uniform weights.
    a.scale_log2 = sm_scale == 0.f ? 1e-30f : sm_scale * 1.4426950408889634f;
    a.status = status;
    a.n_splits = 1;
    a.part_o = nullptr;
    a.part_lse = nullptr;
    a.skip_prefix = 0;
    a.part_slots = 1;
    a.meta_stable = (flags & FST_KERNEL_FLAG_META_STABLE) ? 1 : 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    // the tensor-core kernel moves 16-byte pieces: every row must start on a 16-byte boundary
    const int es = elem_size(dtype);
    const int64_t strides[] = {q_stride_z, q_stride_h, q_stride_n, k_stride_z, k_stride_h, k_stride_n,
                               v_stride_z, v_stride_h, v_stride_n, o_stride_z, o_stride_h, o_stride_n};
    bool rows_aligned = aligned16(q) && aligned16(k) && aligned16(v) && aligned16(o);
    for (int64_t s : strides)
        if ((s * es) & 15) rows_aligned = false;

    if (scatter != nullptr) {
        // attention + all-gather in one kernel: the TMA tree kernel only, no shared prefix
        if (scatter->n_ranks < 1 || scatter->n_ranks > kMaxRanks || !scatter->o_ranks || scatter->rank < 0 ||
            scatter->rank >= scatter->n_ranks)
            return FST_ERR_INVALID_ARG;
        if (scatter->z0 < 0 || scatter->h0 < 0 || scatter->z0 + Z > scatter->Z_total || scatter->h0 + H > scatter->H_total)
            return FST_ERR_INVALID_ARG;
        if (kernel != FST_KERNEL_AUTO && kernel != FST_KERNEL_TMA && kernel != FST_KERNEL_TMA_T32 && kernel != FST_KERNEL_TMA_T64)
            return FST_ERR_UNSUPPORTED;
        if (a.prefix != 0 || !mma_ok(dtype, head_dim, block_m) || block_m < 32) return FST_ERR_UNSUPPORTED;
        for (int r = 0; r < scatter->n_ranks; ++r) {
            if (!scatter->o_ranks[r]) return FST_ERR_INVALID_ARG;
            if (!aligned16(scatter->o_ranks[r])) rows_aligned = false;
            a.o_ranks[r] = scatter->o_ranks[r];
        }
        if (!rows_aligned) return FST_ERR_ALIGNMENT;
        a.n_out = scatter->n_ranks;
        a.out_rank = scatter->rank;
        a.out_z0 = scatter->z0; a.out_h0 = scatter->h0;
        a.out_Z = scatter->Z_total; a.out_H = scatter->H_total;
        return cuda_status(launch_attention_mma(a, dtype, kernel == FST_KERNEL_AUTO ? FST_KERNEL_TMA : kernel, st));
    }

    int choice = kernel;
    const bool automatic = choice == FST_KERNEL_AUTO;
    if (automatic)
        choice = (mma_ok(dtype, head_dim, block_m) && rows_aligned) ? FST_KERNEL_TMA : FST_KERNEL_SIMT;
    if (choice == FST_KERNEL_SIMT) return cuda_status(launch_attention_simt(a, dtype, st));
    if (choice < FST_KERNEL_MMA || choice > FST_KERNEL_PERSIST) return FST_ERR_INVALID_ARG;
    if (!mma_ok(dtype, head_dim, block_m)) return FST_ERR_UNSUPPORTED;
    if (!rows_aligned) return FST_ERR_ALIGNMENT;

    // A shared prefix with a workspace: either the tcgen05 prefix kernel takes it in kv_splits runs
    // while the tree kernel does the tree part (head_dim 64 or 128; chosen automatically from 256
    // prefix rows on), or the tree kernel itself is launched kv_splits times over the prefix.
    const bool can_part = a.prefix > 0 && workspace != nullptr && choice != FST_KERNEL_MMA && choice != FST_KERNEL_PERSIST;
    // (the tcgen05 kernel takes Q from shared memory as it arrived, so it cannot flip Q's sign
    // for a negative factor; the tree kernel walks the prefix itself then)
    const bool want_umma = can_part && (head_dim == 128 || head_dim == 64) && sm_scale > 0.f &&
                           (choice == FST_KERNEL_TMA_UMMA || (automatic && a.prefix >= 256));
    if (choice == FST_KERNEL_TMA_UMMA && !want_umma) return FST_ERR_UNSUPPORTED;
    if (can_part && (want_umma || kv_splits > 1)) {
        const size_t need = fst_attention_split_workspace_bytes(Z, H, n_q, head_dim, kv_splits);
        if (workspace_bytes < need) return FST_ERR_WORKSPACE;
        if (!aligned16(workspace)) return FST_ERR_ALIGNMENT;
        a.part_slots = want_umma ? kv_splits + 1 : kv_splits;
        a.part_o = static_cast<float *>(workspace);
        a.part_lse = a.part_o + size_t(a.part_slots) * Z * H * n_q * head_dim;
        cudaError_t e;
        if (want_umma) {
            // The tree kernel (slot 0) and the prefix kernel (slots 1..) are independent: the tree
            // kernel runs on a second stream, forked from and joined back into the caller's.  The
            // prefix kernel is launched first: its CTAs need a whole SM's shared memory each and
            // would otherwise queue behind the tree kernel's, which fit beside one another.
            a.skip_prefix = 1;
            SideStream *side = side_stream(st);
            cudaStream_t tree_st = st;
            if (side != nullptr && cudaEventRecord(side->fork, st) == cudaSuccess &&
                cudaStreamWaitEvent(side->stream, side->fork, 0) == cudaSuccess)
                tree_st = side->stream;
            else
                (void)cudaGetLastError();                 // no fork: same stream, and no stale error for the launches below
            e = launch_prefix_umma(a, dtype, kv_splits, 1, st);
            const cudaError_t et = launch_attention_mma(a, dtype, FST_KERNEL_TMA, tree_st);
            if (tree_st != st) {                          // always join what was forked
                cudaError_t ej = cudaEventRecord(side->join, tree_st);
                if (ej == cudaSuccess) ej = cudaStreamWaitEvent(st, side->join, 0);
                if (e == cudaSuccess) e = ej;
            }
            if (e == cudaSuccess) e = et;
        } else {
            a.n_splits = kv_splits;
            e = launch_attention_mma(a, dtype, choice, st);
        }
        if (e == cudaSuccess) e = launch_combine(a, dtype, st);
        if (e != cudaErrorNotSupported || !automatic) return cuda_status(e);
        a.n_splits = 1;                                   // a tensor map could not be built: fall through
        a.skip_prefix = 0;
        a.part_slots = 1;
    }
    cudaError_t e = launch_attention_mma(a, dtype, choice == FST_KERNEL_TMA_UMMA ? FST_KERNEL_TMA : choice, st);
    // shapes or strides the TMA variant cannot describe fall back to the cp.async variant
    if (e == cudaErrorNotSupported && automatic) e = launch_attention_mma(a, dtype, FST_KERNEL_MMA, st);
    return cuda_status(e);
}

int fst_attention_fwd(const void *q, const void *k, const void *v, void *o, float *lse,
                      const void *packed, size_t meta_tree_stride, int Z, int H, int n_q, int n_kv,
                      int head_dim, int64_t q_stride_z, int64_t q_stride_h, int64_t q_stride_n,
                      int64_t k_stride_z, int64_t k_stride_h, int64_t k_stride_n,
                      int64_t v_stride_z, int64_t v_stride_h, int64_t v_stride_n,
                      int64_t o_stride_z, int64_t o_stride_h, int64_t o_stride_n, int block_m,
                      int max_ancestors, float sm_scale, int dtype, int kernel, int32_t *status,
                      void *stream) {
    return attention_fwd_impl(q, k, v, o, lse, packed, meta_tree_stride, Z, H, H, n_q, n_kv, head_dim,
                              q_stride_z, q_stride_h, q_stride_n, k_stride_z, k_stride_h, k_stride_n,
                              v_stride_z, v_stride_h, v_stride_n, o_stride_z, o_stride_h, o_stride_n,
                              block_m, max_ancestors, sm_scale, dtype, kernel, 1, nullptr, 0, status,
                              stream);
}

int fst_attention_fwd_scatter(const void *q, const void *k, const void *v, void *const *o_ranks, int n_ranks,
                              int my_rank, int shard_z0, int shard_h0, int Z_total, int H_total, float *lse,
                              const void *packed, size_t meta_tree_stride, int Z, int H, int n_q, int n_kv,
                              int head_dim, int64_t q_stride_z, int64_t q_stride_h, int64_t q_stride_n,
                              int64_t k_stride_z, int64_t k_stride_h, int64_t k_stride_n,
                              int64_t v_stride_z, int64_t v_stride_h, int64_t v_stride_n,
                              int64_t o_stride_z, int64_t o_stride_h, int64_t o_stride_n, int block_m,
                              int max_ancestors, float sm_scale, int dtype, int kernel, int32_t *status,
                              void *stream) {
    if (!o_ranks || n_ranks < 1 || n_ranks > kMaxRanks) return FST_ERR_INVALID_ARG;
    const ScatterTo sc{o_ranks, n_ranks, my_rank, shard_z0, shard_h0, Z_total, H_total};
    return attention_fwd_impl(q, k, v, o_ranks[0], lse, packed, meta_tree_stride, Z, H, H, n_q, n_kv, head_dim,
                              q_stride_z, q_stride_h, q_stride_n, k_stride_z, k_stride_h, k_stride_n,
                              v_stride_z, v_stride_h, v_stride_n, o_stride_z, o_stride_h, o_stride_n,
                              block_m, max_ancestors, sm_scale, dtype, kernel, 1, nullptr, 0, status,
                              stream, &sc);
}

int fst_attention_fwd_splitkv(const void *q, const void *k, const void *v, void *o, float *lse,
                              const void *packed, size_t meta_tree_stride, int Z, int H, int n_q,
                              int n_kv, int head_dim, int64_t q_stride_z, int64_t q_stride_h,
                              int64_t q_stride_n, int64_t k_stride_z, int64_t k_stride_h,
                              int64_t k_stride_n, int64_t v_stride_z, int64_t v_stride_h,
                              int64_t v_stride_n, int64_t o_stride_z, int64_t o_stride_h,
                              int64_t o_stride_n, int block_m, int max_ancestors, float sm_scale,
                              int dtype, int kernel, int kv_splits, void *workspace,
                              size_t workspace_bytes, int32_t *status, void *stream) {
    if (kv_splits < 1) return FST_ERR_INVALID_ARG;
    if (kv_splits > 1 && (long long)Z * kv_splits > 65535) return FST_ERR_TOO_LARGE;
    return attention_fwd_impl(q, k, v, o, lse, packed, meta_tree_stride, Z, H, H, n_q, n_kv, head_dim,
                              q_stride_z, q_stride_h, q_stride_n, k_stride_z, k_stride_h, k_stride_n,
                              v_stride_z, v_stride_h, v_stride_n, o_stride_z, o_stride_h, o_stride_n,
                              block_m, max_ancestors, sm_scale, dtype, kernel, kv_splits, workspace,
                              workspace_bytes, status, stream);
}

int fst_attention_fwd_gqa(const void *q, const void *k, const void *v, void *o, float *lse,
                          const void *packed, size_t meta_tree_stride, int Z, int H, int H_kv, int n_q,
                          int n_kv, int head_dim, int64_t q_stride_z, int64_t q_stride_h,
                          int64_t q_stride_n, int64_t k_stride_z, int64_t k_stride_h,
                          int64_t k_stride_n, int64_t v_stride_z, int64_t v_stride_h,
                          int64_t v_stride_n, int64_t o_stride_z, int64_t o_stride_h,
                          int64_t o_stride_n, int block_m, int max_ancestors, float sm_scale,
                          int dtype, int kernel, int kv_splits, void *workspace,
                          size_t workspace_bytes, int32_t *status, void *stream) {
    if (kv_splits < 1) return FST_ERR_INVALID_ARG;
    if (kv_splits > 1 && (long long)Z * kv_splits > 65535) return FST_ERR_TOO_LARGE;
    return attention_fwd_impl(q, k, v, o, lse, packed, meta_tree_stride, Z, H, H_kv, n_q, n_kv, head_dim,
                              q_stride_z, q_stride_h, q_stride_n, k_stride_z, k_stride_h, k_stride_n,
                              v_stride_z, v_stride_h, v_stride_n, o_stride_z, o_stride_h, o_stride_n,
                              block_m, max_ancestors, sm_scale, dtype, kernel, kv_splits, workspace,
                              workspace_bytes, status, stream);
}

int fst_attention_fwd_paged(const void *q, const void *k_tree, const void *v_tree, void *o, float *lse,
                            const void *packed, size_t meta_tree_stride, const void *k_pool,
                            const void *v_pool, const int32_t *block_table, int table_stride,
                            const int32_t *prefix_lens, int max_prefix, int page_size, int n_pages,
                            int64_t pool_stride_page, int64_t pool_stride_row, int64_t pool_stride_head,
                            int Z, int H, int H_kv, int n_q, int head_dim, int64_t q_stride_z,
                            int64_t q_stride_h, int64_t q_stride_n, int64_t k_stride_z, int64_t k_stride_h,
                            int64_t k_stride_n, int64_t v_stride_z, int64_t v_stride_h, int64_t v_stride_n,
                            int64_t o_stride_z, int64_t o_stride_h, int64_t o_stride_n, int block_m,
                            int max_ancestors, float sm_scale, int dtype, int kv_splits, void *workspace,
                            size_t workspace_bytes, int32_t *status, void *stream) {
    if (!q || !k_tree || !v_tree || !o || !packed || !k_pool || !v_pool || !block_table || !prefix_lens ||
        !workspace || Z <= 0 || H <= 0 || H_kv <= 0 || H % H_kv != 0 || n_q <= 0 || block_m <= 0 ||
        max_ancestors <= 0 || max_prefix <= 0 || n_pages <= 0 || kv_splits < 1 || table_stride <= 0)
        return FST_ERR_INVALID_ARG;
    if ((head_dim != 128 && head_dim != 64) || !mma_ok(dtype, head_dim, block_m)) return FST_ERR_UNSUPPORTED;
    if (!(sm_scale > 0.f) || !std::isfinite(sm_scale)) return FST_ERR_INVALID_ARG;   // the tcgen05 prefix kernel wants a positive factor
    if (page_size != 16 && page_size != 32 && page_size != 64 && page_size != 128) return FST_ERR_UNSUPPORTED;
    if (H > 65535 || Z > 65535 || (long long)Z * kv_splits > 65535) return FST_ERR_TOO_LARGE;
    if ((long long)table_stride * page_size < max_prefix) return FST_ERR_INVALID_ARG;
    const int64_t strides[] = {q_stride_z, q_stride_h, q_stride_n, k_stride_z, k_stride_h, k_stride_n,
                               v_stride_z, v_stride_h, v_stride_n, o_stride_z, o_stride_h, o_stride_n,
                               pool_stride_page, pool_stride_row, pool_stride_head};
    bool ok = aligned16(q) && aligned16(k_tree) && aligned16(v_tree) && aligned16(o) && aligned16(k_pool) &&
              aligned16(v_pool) && aligned16(packed) && aligned16(workspace) && !(meta_tree_stride & 15);
    for (int64_t s : strides)
        if ((s * 2) & 15) ok = false;
    if (!ok) return FST_ERR_ALIGNMENT;
    if (workspace_bytes < fst_attention_split_workspace_bytes(Z, H, n_q, head_dim, kv_splits))
        return FST_ERR_WORKSPACE;

    AttnArgs a = {};                                      // the tree part: K/V rows of the tree nodes only
    a.q = q; a.k = k_tree; a.v = v_tree; a.o = o; a.lse = lse;
    a.packed = static_cast<const unsigned char *>(packed);
    a.meta_stride = meta_tree_stride;
    a.Z = Z; a.H = H; a.n_q = n_q; a.n_kv = n_q; a.D = head_dim; a.prefix = 0;
    a.kv_group = H / H_kv;
    a.qs_z = q_stride_z; a.qs_h = q_stride_h; a.qs_n = q_stride_n;
    a.ks_z = k_stride_z; a.ks_h = k_stride_h; a.ks_n = k_stride_n;
    a.vs_z = v_stride_z; a.vs_h = v_stride_h; a.vs_n = v_stride_n;
    a.os_z = o_stride_z; a.os_h = o_stride_h; a.os_n = o_stride_n;
    a.bm = block_m; a.ma = max_ancestors; a.nb = (n_q + block_m - 1) / block_m;
    a.scale_log2 = sm_scale * 1.4426950408889634f;
    a.status = status;
    a.n_splits = 1;
    a.skip_prefix = 1;
    a.part_slots = kv_splits + 1;
    a.meta_stable = 0;
    a.part_o = static_cast<float *>(workspace);
    a.part_lse = a.part_o + size_t(a.part_slots) * Z * H * n_q * head_dim;
    AttnArgs ap = a;                                      // the prefix part: rows come from the page pool
    ap.prefix = max_prefix;
    PagedArgs pg{k_pool, v_pool, block_table, prefix_lens, table_stride, page_size, n_pages,
                 pool_stride_page, pool_stride_row, pool_stride_head};

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    SideStream *side = side_stream(st);                   // as in the contiguous prefix path
    cudaStream_t tree_st = st;
    if (side != nullptr && cudaEventRecord(side->fork, st) == cudaSuccess &&
        cudaStreamWaitEvent(side->stream, side->fork, 0) == cudaSuccess)
        tree_st = side->stream;
    else
        (void)cudaGetLastError();
    cudaError_t e = launch_prefix_umma_paged(ap, pg, dtype, kv_splits, 1, st);
    const cudaError_t et = launch_attention_mma(a, dtype, FST_KERNEL_TMA, tree_st);
    if (tree_st != st) {
        cudaError_t ej = cudaEventRecord(side->join, tree_st);
        if (ej == cudaSuccess) ej = cudaStreamWaitEvent(st, side->join, 0);
        if (e == cudaSuccess) e = ej;
    }
    if (e == cudaSuccess) e = et;
    if (e == cudaSuccess) e = launch_combine(a, dtype, st);
    return cuda_status(e);
}

size_t fst_attention_ref_workspace_bytes(int n_meta_trees, int n_q, int block_m, int max_ancestors) {
    if (n_meta_trees <= 0 || n_q <= 0 || block_m <= 0 || max_ancestors <= 0) return 0;
    const int nb = (n_q + block_m - 1) / block_m;
    return size_t(n_meta_trees) * packed_layout(nb, block_m, max_ancestors).total;
}

int fst_attention_fwd_ref(const void *q, const void *k, const void *v, void *o, float *lse,
                          const int64_t *ancestor_idx, const uint8_t *ancestor_mask,
                          const int64_t *leaf_idx, int n_meta_trees, int Z, int H, int n_q, int n_kv,
                          int head_dim, int64_t q_stride_z, int64_t q_stride_h, int64_t q_stride_n,
                          int64_t k_stride_z, int64_t k_stride_h, int64_t k_stride_n,
                          int64_t v_stride_z, int64_t v_stride_h, int64_t v_stride_n,
                          int64_t o_stride_z, int64_t o_stride_h, int64_t o_stride_n, int block_m,
                          int max_ancestors, float sm_scale, int dtype, int kernel, void *workspace,
                          size_t workspace_bytes, int32_t *status, void *stream) {
    if (!workspace) return FST_ERR_INVALID_ARG;
    if (n_meta_trees != 1 && n_meta_trees != Z) return FST_ERR_INVALID_ARG;
    if (n_q <= 0 || n_kv < n_q || block_m <= 0 || max_ancestors <= 0) return FST_ERR_INVALID_ARG;
    const size_t need = fst_attention_ref_workspace_bytes(n_meta_trees, n_q, block_m, max_ancestors);
    if (workspace_bytes < need) return FST_ERR_WORKSPACE;
    const int nb = (n_q + block_m - 1) / block_m;
    const size_t tree_bytes = packed_layout(nb, block_m, max_ancestors).total;
    int rc = fst_pack_metadata(ancestor_idx, ancestor_mask, leaf_idx, n_meta_trees, nb, block_m,
                               max_ancestors, int64_t(n_kv - n_q), workspace, tree_bytes, status,
                               stream);
    if (rc != FST_OK) return rc;
    return fst_attention_fwd(q, k, v, o, lse, workspace, n_meta_trees == 1 ? 0 : tree_bytes, Z, H,
                             n_q, n_kv, head_dim, q_stride_z, q_stride_h, q_stride_n, k_stride_z,
                             k_stride_h, k_stride_n, v_stride_z, v_stride_h, v_stride_n, o_stride_z,
                             o_stride_h, o_stride_n, block_m, max_ancestors, sm_scale, dtype,
                             kernel & FST_KERNEL_MASK,    // the metadata was written a launch ago: never "stable"
                             status, stream);
}

int fst_attention_fwd_ref_static(const void *q, const void *k, const void *v, void *o, float *lse,
                                 const int64_t *ancestor_idx, const uint8_t *ancestor_mask,
                                 const int64_t *leaf_idx, int n_meta_trees, int Z, int H, int n_q,
                                 int n_kv, int head_dim, int64_t q_stride_z, int64_t q_stride_h,
                                 int64_t q_stride_n, int64_t k_stride_z, int64_t k_stride_h,
                                 int64_t k_stride_n, int64_t v_stride_z, int64_t v_stride_h,
                                 int64_t v_stride_n, int64_t o_stride_z, int64_t o_stride_h,
                                 int64_t o_stride_n, int block_m, int max_ancestors, float sm_scale,
                                 int dtype, int kernel, int32_t *status, void *stream) {
    if (n_meta_trees <= 0 || n_q <= 0 || block_m <= 0 || max_ancestors <= 0) return FST_ERR_INVALID_ARG;
    const size_t need = fst_attention_ref_workspace_bytes(n_meta_trees, n_q, block_m, max_ancestors);
    if (need == 0) return FST_ERR_INVALID_ARG;
    if (need > FST_STATIC_SCRATCH_BYTES) return FST_ERR_TOO_LARGE;   // metadata does not fit the built-in scratch
    void *scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != FST_OK) return rc;
    return fst_attention_fwd_ref(q, k, v, o, lse, ancestor_idx, ancestor_mask, leaf_idx, n_meta_trees,
                                 Z, H, n_q, n_kv, head_dim, q_stride_z, q_stride_h, q_stride_n,
                                 k_stride_z, k_stride_h, k_stride_n, v_stride_z, v_stride_h, v_stride_n,
                                 o_stride_z, o_stride_h, o_stride_n, block_m, max_ancestors, sm_scale,
                                 dtype, kernel, scratch, FST_STATIC_SCRATCH_BYTES, status, stream);
}

}  // extern "C"
