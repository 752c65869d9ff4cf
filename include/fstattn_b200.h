/*
 * fstattn_b200 - fused sparse tree attention for NVIDIA B200 (sm_100a), C ABI.
 *
 * Everything here is plain C: device pointers, sizes and a CUDA stream handle passed as
 * void*.  No function allocates or frees device memory or synchronises; each one enqueues its
 * kernels on the given stream and returns a status code (0 = FST_OK) describing host-side
 * argument checks.  Host-side state the library keeps: per host thread a table of the tensor
 * maps it has built (about 200 KB of host memory, filled as calls come), and - only for calls
 * that hand a shared prefix to the tcgen05 kernel (fst_attention_fwd_splitkv / _gqa / _paged with
 * a workspace) - one extra CUDA stream and two events per host thread and device, created at the
 * first such call outside stream capture and kept until the process ends.  The first call of a
 * kernel variant on a device also sets that kernel's shared-memory attribute; make one call per
 * shape and dtype before capturing a stream into a graph.
 * Problems that only the GPU can see (a malformed tree, too many ancestors in a block, an
 * index out of range) are recorded in a caller-provided device status record
 * (int32_t status[FST_STATUS_WORDS]) and never fault the device; the kernels keep going with
 * the offending element ignored.  Clear the record once (cudaMemsetAsync) and read it back
 * whenever a check is wanted.
 *
 * "Reference" below means the project this library is a drop-in for; paths are inside it.
 */
#ifndef FSTATTN_B200_H
#define FSTATTN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FST_VERSION 100
#define FST_STATUS_WORDS 4   /* status[0]=code, [1]=tree*65536+block or row, [2]=detail, [3]=spare */

enum fst_status {
    FST_OK = 0,
    FST_ERR_INVALID_ARG = 1,       /* null pointer, non-positive size, unknown enum            */
    FST_ERR_UNSUPPORTED = 2,       /* head_dim / dtype / block_m combination has no kernel      */
    FST_ERR_ALIGNMENT = 3,         /* pointer or stride not 16-byte aligned                     */
    FST_ERR_WORKSPACE = 4,         /* workspace too small                                       */
    FST_ERR_CUDA = 5,              /* a CUDA runtime call failed (launch configuration)         */
    FST_ERR_TOO_LARGE = 6,         /* size beyond a documented limit                            */
    /* device-side codes, written to status[0] */
    FST_DEV_MALFORMED_TREE = 16,   /* parent[i] >= i or < -1; status[1] = node                  */
    FST_DEV_ANCESTOR_OVERFLOW = 17,/* a block has more unique ancestors than max_ancestors;     */
                                   /* status[1] = tree*65536+block, status[2] = the count        */
    FST_DEV_INDEX_RANGE = 18,      /* a metadata index points outside the K/V rows              */
    FST_DEV_TIMEOUT = 19           /* a bounded wait on an asynchronous copy ran out            */
};

enum fst_dtype { FST_F16 = 0, FST_BF16 = 1, FST_F32 = 2 };

/* Kernel choice for fst_attention_fwd*; FST_KERNEL_AUTO is what callers want. */
enum fst_kernel {
    FST_KERNEL_AUTO = 0,
    FST_KERNEL_SIMT = 1,           /* fp32 arithmetic, any dtype / head_dim in {16,32,64,128}   */
    FST_KERNEL_MMA = 2,            /* tensor-core kernel, cp.async gathers: fp16/bf16, D 64/128  */
    FST_KERNEL_TMA = 3,            /* same arithmetic, TMA tile loads + mbarriers, swizzled smem; */
                                   /* 32- or 64-column tiles chosen by grid size                 */
    FST_KERNEL_TMA_T32 = 4,        /* ... forced 32-column tiles (three CTAs per SM)             */
    FST_KERNEL_TMA_T64 = 5,        /* ... forced 64-column tiles (fewest softmax rounds)         */
    FST_KERNEL_TMA_UMMA = 6,       /* tree part as FST_KERNEL_TMA, shared prefix by the tcgen05  */
                                   /* kernel (head_dim 64 / 128, fst_attention_fwd_splitkv only) */
    FST_KERNEL_PERSIST = 7         /* persistent CTAs, a producer warp streaming tiles through a */
                                   /* shared-memory ring ahead of the arithmetic: block_m 64 or  */
                                   /* 128, no prefix.  Slower than FST_KERNEL_TMA on every shape */
                                   /* measured, so never the automatic choice                    */
};

/*
 * Flags that may be OR-ed into the `kernel` argument.
 * FST_KERNEL_FLAG_META_STABLE: the packed metadata was completely written before the launch that
 * precedes this call on the stream began (one precompute per decode step, then one attention call
 * per layer: true for every call but the first after the precompute).  The tree kernel is
 * launched so that it may become resident while the kernel ahead of it drains; with this flag it
 * fetches its index list and mask words during that time instead of afterwards.  Q, K, V and O
 * are never touched early.  Leaving the flag out is always correct.
 */
#define FST_KERNEL_MASK 0xff
#define FST_KERNEL_FLAG_META_STABLE 0x100

int fst_version(void);
const char *fst_status_string(int status);

/*
 * Packed block metadata, the form the attention kernels read.  For one tree with
 * n_blocks = ceil(n_nodes / block_m) query blocks it is one blob of
 * fst_packed_meta_bytes() bytes holding four arrays, each starting on a 16-byte boundary:
 *   int32  count[n_blocks]                 ancestors of the block that lie outside its own rows
 *   int32  idx  [n_blocks][max_ancestors]  their node indices, in list order, -1 padded
 *   uint32 emask[n_blocks][block_m][W]     W = ceil(max_ancestors/32); bit a of row j set when
 *                                          row j attends to idx[a]
 *   uint32 bmask[n_blocks][block_m][ceil(block_m/32)]
 *                                          bit c of row j set when row j attends to row c of
 *                                          its own block: itself (always) and the ancestors
 *                                          that live inside the block
 * The reference's ancestor list is the external list followed by the in-block ancestors; its
 * leaf path (utils.py:121-122) is the diagonal of bmask.
 * Indices are relative to the first tree row (the shared prefix is not counted).
 * A batch of trees is an array of such blobs, meta_tree_stride bytes apart.
 */
size_t fst_packed_meta_bytes(int n_blocks, int block_m, int max_ancestors);

/*
 * Tree precompute on the GPU.  Replaces utils.py:104-129
 * (create_fst_attention_kernel_inputs) of the reference, taking the tree as a parent array
 * instead of lineage/level_lookup (utils.py:42-44): parent[t][i] in [-1, i), -1 for roots.
 *
 * For each of n_trees trees (parent arrays n_nodes apart) writes, when the pointer is not
 * NULL:
 *   ancestor_idx  int64 [n_trees][n_blocks][max_ancestors]           (-1 padded)
 *   ancestor_mask uint8 [n_trees][n_blocks][block_m][max_ancestors]  (0/1, torch.bool layout)
 *   leaf_idx      int64 [n_trees][n_blocks][block_m]                 (-1 where not a leaf)
 *   packed        blobs as described above, packed_tree_stride bytes apart
 * bit-identical to the reference, including leaf entries past the last node in a partial
 * last block (utils.py:121-122).  Where the reference raises on more than max_ancestors
 * ancestors (utils.py:120) this records FST_DEV_ANCESTOR_OVERFLOW and keeps the first
 * max_ancestors.  Limits: 1 <= block_m <= 1024, n_nodes <= 262144.
 */
int fst_precompute(const int32_t *parent, int n_trees, int n_nodes, int block_m,
                   int max_ancestors, int64_t *ancestor_idx, uint8_t *ancestor_mask,
                   int64_t *leaf_idx, void *packed, size_t packed_tree_stride,
                   int32_t *status, void *stream);

/*
 * Self-test of the bounded waits (no counterpart in the reference).  Every wait on an
 * asynchronous copy or tensor-core product in these kernels gives up after about 50 ms, records
 * FST_DEV_TIMEOUT and lets the kernel run to its end, so that a lost completion cannot hang the
 * GPU.  This launches one thread that waits on a barrier nobody arrives at: afterwards
 * status[0] == FST_DEV_TIMEOUT, status[1] == 12345 and *done == 2 (1 would mean the wait
 * returned as if somebody had arrived).  Takes about 50 ms of one SM.  Device pointers.
 */
int fst_selftest_wait_timeout(int32_t *status, int32_t *done, void *stream);

/*
 * Depth-first renumbering of n_trees trees of n_nodes nodes each (parent as for fst_precompute),
 * the node ordering the reference leaves open (README.md:19-20; utils.py:104-129 takes the
 * caller's numbering).  order[t][i] = old index of the node that becomes node i of tree t
 * (pre-order, children in their old relative order); new_parent[t][i] = its parent in the new
 * numbering (< i, or -1), ready for fst_precompute.  The caller permutes the tree rows of
 * q/k/v with `order` and scatters the output rows back.  n_nodes <= 8192 (FST_ERR_TOO_LARGE
 * beyond); a malformed parent sets FST_DEV_MALFORMED_TREE in `status` and leaves the outputs
 * untouched.  All pointers are device pointers.
 */
int fst_dfs_order(const int32_t *parent, int n_trees, int n_nodes, int32_t *order,
                  int32_t *new_parent, int32_t *status, void *stream);

/*
 * Tree construction on the device from top-k candidate scores.  The reference builds its forest
 * on the CPU and only as a fixed synthetic shape (create_tree, utils.py:27-77: topk roots, level
 * sizes size[l] = topk * int(size[l-1] * left_weight_factor), node r of a level under node
 * r / topk of the level above); its README.md:17 names the use, Medusa-style trees over every
 * head's top-k candidates.  Here the same recurrence is driven by scores so that a decode step
 * never leaves the GPU (this call, then fst_dfs_order and/or fst_precompute):
 *   scores     float [n_trees][depth + 1][topk]  candidate scores (log-probabilities) of head l
 *   parent     int32 [n_trees][max_nodes]        out: parent[i] < i, -1 for the topk roots
 *   choice     int32 [n_trees][max_nodes]        out, optional: l * topk + k, the candidate
 *                                                 (head l, k-th entry of its scores) node i stands for
 *   node_score float [n_trees][max_nodes]        out, optional: sum of the scores along the path
 * A node's score is the sum along its path.  Of every level the int(size * left_weight_factor)
 * best nodes are expanded, best first (ties: the earlier node), each into the topk candidates of
 * the next head in the order given; nodes are numbered level by level.  With equal scores
 * the parent array is exactly that of create_tree(depth, topk, left_weight_factor).  The node
 * count depends on the three shape arguments only: fst_tree_topk_nodes() (-1: a level outgrows
 * the kernel's 4096 nodes, or more than 32 levels).  Nodes at and beyond max_nodes are dropped;
 * entries between the node count and max_nodes become isolated roots (parent -1, choice -1).
 * Device pointers.
 */
long long fst_tree_topk_nodes(int depth, int topk, double left_weight_factor);
int fst_build_tree_topk(const float *scores, int n_trees, int depth, int topk,
                        double left_weight_factor, int max_nodes, int32_t *parent, int32_t *choice,
                        float *node_score, void *stream);

/*
 * Convert reference-format metadata (the three tensors of utils.py:104-129, already on the
 * device) into packed blobs.  index_base is subtracted from every index; entries below it
 * are padding.  The reference's test shifts the index tensors by the prefix length,
 * sentinels included (fstattention.py:211-212); with index_base = prefix length both the
 * shifted sentinels and plain -1 read as padding here.
 */
int fst_pack_metadata(const int64_t *ancestor_idx, const uint8_t *ancestor_mask,
                      const int64_t *leaf_idx, int n_trees, int n_blocks, int block_m,
                      int max_ancestors, int64_t index_base, void *packed,
                      size_t packed_tree_stride, int32_t *status, void *stream);

/*
 * Fused sparse tree attention, forward.  Replaces the kernel and launch of
 * fstattention.py:21-181 (_fwd_kernel / fst_attention).
 *
 *   q, o : [Z][H][n_q][head_dim]      strides in elements, innermost dimension contiguous
 *   k, v : [Z][H][n_kv][head_dim]     rows [0, prefix_len) are a prefix every query attends
 *                                      to; tree node i lives in row prefix_len + i
 *   lse  : optional float [Z][H][n_q], base-2 log-sum-exp of the scaled scores
 *          (fstattention.py:140-141); NULL to skip
 *   packed, meta_tree_stride : packed metadata; stride 0 shares one tree between all Z
 *          (the reference's behaviour, fstattention.py:62-67), otherwise tree z is used for
 *          batch element z
 * The prefix length is n_kv - n_q, as in fstattention.py:163.  Block rows >= n_q are neither
 * read nor written, so n_q need not be a multiple of block_m.
 * dtype: FST_F16 / FST_BF16 (tensor cores: head_dim 64 or 128 and block_m 16, 32, 64 or 128;
 * other block sizes run on the SIMT kernel) or any of the three with head_dim in {16,32,64,128}
 * on the fp32 SIMT kernel.  sm_scale: any finite value of either sign, applied before the row
 * maximum as in fstattention.py:78-97 (NaN or infinity: FST_ERR_INVALID_ARG).
 */
int fst_attention_fwd(const void *q, const void *k, const void *v, void *o, float *lse,
                      const void *packed, size_t meta_tree_stride,
                      int Z, int H, int n_q, int n_kv, int head_dim,
                      int64_t q_stride_z, int64_t q_stride_h, int64_t q_stride_n,
                      int64_t k_stride_z, int64_t k_stride_h, int64_t k_stride_n,
                      int64_t v_stride_z, int64_t v_stride_h, int64_t v_stride_n,
                      int64_t o_stride_z, int64_t o_stride_h, int64_t o_stride_n,
                      int block_m, int max_ancestors, float sm_scale, int dtype, int kernel,
                      int32_t *status, void *stream);

/*
 * fst_attention_fwd on one GPU's shard of a problem split over several GPUs of a node, with the
 * all-gather of the output done by the attention kernel itself.  (No counterpart in the
 * reference, which is single-GPU; its programs are independent, fstattention.py:42-45, grid
 * :159, so a batch of trees splits by tree and a single tree by head.)
 *
 * Every rank holds the full output tensor [Z_total][H_total][n_q][head_dim] (strides
 * o_stride_*, the same on all ranks) and has the other ranks' copies mapped into its address
 * space (CUDA IPC or virtual-memory export; peer access enabled): o_ranks[r] is rank r's copy as
 * THIS process addresses it, this rank's own (o_ranks[my_rank]) included, n_ranks <= 8, a HOST
 * array.  q, k, v are
 * this rank's shard, [Z][H][..][head_dim]; its (z, h) is element (shard_z0 + z, shard_h0 + h) of
 * the full tensor.  Each CTA stores its finished tile once per rank (plain TMA stores, one per rank),
 * so rows cross NVLink while other CTAs still compute.  When the kernel has finished on the
 * stream this rank's rows are in place everywhere; before anyone reads a full tensor, and before
 * a buffer is written again, the ranks must meet (a barrier on the streams: the caller's job).
 * Tensor-core TMA kernel only: fp16 / bf16, head_dim 64 or 128, block_m 32, 64 or 128, no shared
 * prefix (n_kv == n_q), kernel = FST_KERNEL_AUTO or one of FST_KERNEL_TMA*; FST_ERR_UNSUPPORTED
 * otherwise.  lse, when given, is this shard's [Z][H][n_q] and stays local.
 */
int fst_attention_fwd_scatter(const void *q, const void *k, const void *v, void *const *o_ranks, int n_ranks,
                              int my_rank, int shard_z0, int shard_h0, int Z_total, int H_total, float *lse,
                              const void *packed, size_t meta_tree_stride,
                              int Z, int H, int n_q, int n_kv, int head_dim,
                              int64_t q_stride_z, int64_t q_stride_h, int64_t q_stride_n,
                              int64_t k_stride_z, int64_t k_stride_h, int64_t k_stride_n,
                              int64_t v_stride_z, int64_t v_stride_h, int64_t v_stride_n,
                              int64_t o_stride_z, int64_t o_stride_h, int64_t o_stride_n,
                              int block_m, int max_ancestors, float sm_scale, int dtype, int kernel,
                              int32_t *status, void *stream);

/*
 * fst_attention_fwd with the shared prefix cut into kv_splits runs of rows, each handled by its
 * own CTA per (block, head, batch) - the decode case, where a long prompt meets a tree too small
 * to fill the GPU (the reference walks the prefix in one program, fstattention.py:113-136).
 * Partial results (fp32) and their log-sum-exps pass through `workspace`
 * (fst_attention_split_workspace_bytes bytes, 16-byte aligned, scratch) and a second kernel merges
 * them.  With head_dim 64 or 128 and at least 256 prefix rows FST_KERNEL_AUTO hands the prefix to a
 * tcgen05/TMEM kernel (128 x 128 tiles, dense) in kv_splits runs and keeps the tree part in the
 * tree kernel; FST_KERNEL_TMA_UMMA forces that, FST_KERNEL_TMA* forces the tree kernel to walk
 * the prefix itself in kv_splits runs.  Without a prefix this is fst_attention_fwd.
 */
size_t fst_attention_split_workspace_bytes(int Z, int H, int n_q, int head_dim, int kv_splits);
int fst_attention_fwd_splitkv(const void *q, const void *k, const void *v, void *o, float *lse,
                              const void *packed, size_t meta_tree_stride,
                              int Z, int H, int n_q, int n_kv, int head_dim,
                              int64_t q_stride_z, int64_t q_stride_h, int64_t q_stride_n,
                              int64_t k_stride_z, int64_t k_stride_h, int64_t k_stride_n,
                              int64_t v_stride_z, int64_t v_stride_h, int64_t v_stride_n,
                              int64_t o_stride_z, int64_t o_stride_h, int64_t o_stride_n,
                              int block_m, int max_ancestors, float sm_scale, int dtype, int kernel,
                              int kv_splits, void *workspace, size_t workspace_bytes,
                              int32_t *status, void *stream);

/*
 * fst_attention_fwd_splitkv for grouped-query attention: q and o have H heads, k and v have H_kv
 * heads, H a multiple of H_kv; query head h reads K/V head h / (H / H_kv).  The reference assumes
 * H_kv == H (fstattention.py:44-45 index K and V with the query's head offset); this is the
 * layout of the KV caches the kernel meets in a decoder.  Query heads of one group sit in
 * neighbouring CTAs, so their shared K/V rows are fetched from HBM once and from L2 afterwards.
 * workspace as for fst_attention_fwd_splitkv (sized by H); kv_splits = 1 and workspace = NULL
 * give the plain single-kernel call.
 */
int fst_attention_fwd_gqa(const void *q, const void *k, const void *v, void *o, float *lse,
                          const void *packed, size_t meta_tree_stride,
                          int Z, int H, int H_kv, int n_q, int n_kv, int head_dim,
                          int64_t q_stride_z, int64_t q_stride_h, int64_t q_stride_n,
                          int64_t k_stride_z, int64_t k_stride_h, int64_t k_stride_n,
                          int64_t v_stride_z, int64_t v_stride_h, int64_t v_stride_n,
                          int64_t o_stride_z, int64_t o_stride_h, int64_t o_stride_n,
                          int block_m, int max_ancestors, float sm_scale, int dtype, int kernel,
                          int kv_splits, void *workspace, size_t workspace_bytes,
                          int32_t *status, void *stream);

/*
 * Tree attention behind a prefix that lives in a paged KV cache.  The reference keeps prefix and
 * tree rows in one contiguous K/V tensor (fstattention.py:163, 207-212); a serving engine keeps
 * the prompt in pages.  Here the tree nodes' K/V rows come as tensors of their own
 * (k_tree, v_tree: [Z, H_kv, n_q, head_dim] by the given strides) and the prefix rows of batch
 * element z are rows [0, prefix_lens[z]) of the sequence whose pages block_table[z][0..] lists:
 * row r sits in page block_table[z * table_stride + r / page_size] at row r % page_size.
 * k_pool / v_pool: element (page, row, head, d) at page * pool_stride_page + row * pool_stride_row
 * + head * pool_stride_head + d (element strides, multiples of 8).  page_size 16, 32, 64 or 128;
 * head_dim 64 or 128; fp16 / bf16.  max_prefix >= every prefix_lens[z] (it sizes the grid; lengths
 * above it are cut).  The prefix goes to the tcgen05 kernel in kv_splits runs, the tree part to
 * the tree kernel, partial results through `workspace`
 * (fst_attention_split_workspace_bytes(Z, H, n_q, head_dim, kv_splits) bytes).  A page number
 * outside [0, n_pages) reads as zeros and sets FST_DEV_INDEX_RANGE.  block_table and prefix_lens
 * are device pointers.  sm_scale must be positive here (the tcgen05 prefix kernel takes Q as it
 * lies in shared memory and cannot fold a sign into it): FST_ERR_INVALID_ARG otherwise.
 */
int fst_attention_fwd_paged(const void *q, const void *k_tree, const void *v_tree, void *o, float *lse,
                            const void *packed, size_t meta_tree_stride,
                            const void *k_pool, const void *v_pool,
                            const int32_t *block_table, int table_stride,
                            const int32_t *prefix_lens, int max_prefix, int page_size, int n_pages,
                            int64_t pool_stride_page, int64_t pool_stride_row, int64_t pool_stride_head,
                            int Z, int H, int H_kv, int n_q, int head_dim,
                            int64_t q_stride_z, int64_t q_stride_h, int64_t q_stride_n,
                            int64_t k_stride_z, int64_t k_stride_h, int64_t k_stride_n,
                            int64_t v_stride_z, int64_t v_stride_h, int64_t v_stride_n,
                            int64_t o_stride_z, int64_t o_stride_h, int64_t o_stride_n,
                            int block_m, int max_ancestors, float sm_scale, int dtype, int kv_splits,
                            void *workspace, size_t workspace_bytes, int32_t *status, void *stream);

/*
 * The same with reference-format metadata, i.e. exactly the arguments of the reference's
 * fst_attention(q, k, v, ancestor_idx, ancestor_mask, leaf_idx, sm_scale, BLOCK_M,
 * MAX_ANCESTORS) (fstattention.py:153).  Index tensors hold absolute K/V rows
 * (tree index + prefix length); n_meta_trees is 1 (shared) or Z.  workspace is scratch
 * device memory of at least fst_attention_ref_workspace_bytes() bytes, 16-byte aligned, that
 * the call fills with the packed form and the attention kernel then reads; it must stay
 * untouched until the call has finished on the stream.
 */
size_t fst_attention_ref_workspace_bytes(int n_meta_trees, int n_q, int block_m,
                                         int max_ancestors);
int fst_attention_fwd_ref(const void *q, const void *k, const void *v, void *o, float *lse,
                          const int64_t *ancestor_idx, const uint8_t *ancestor_mask,
                          const int64_t *leaf_idx, int n_meta_trees,
                          int Z, int H, int n_q, int n_kv, int head_dim,
                          int64_t q_stride_z, int64_t q_stride_h, int64_t q_stride_n,
                          int64_t k_stride_z, int64_t k_stride_h, int64_t k_stride_n,
                          int64_t v_stride_z, int64_t v_stride_h, int64_t v_stride_n,
                          int64_t o_stride_z, int64_t o_stride_h, int64_t o_stride_n,
                          int block_m, int max_ancestors, float sm_scale, int dtype, int kernel,
                          void *workspace, size_t workspace_bytes,
                          int32_t *status, void *stream);

/*
 * fst_attention_fwd_ref for hosts that must not allocate.  (No counterpart in the reference,
 * whose wrapper allocates freely through torch, fstattention.py:158-160.)
 *
 * Some callers cannot provide the workspace above because they cannot call cudaMalloc or a
 * framework allocator where this function runs: an inference engine's per-layer plugin hook
 * that is only handed its input and output buffers, or a serving loop that gave all device
 * memory to its own pool at start-up and forbids (or cannot afford, since cudaMalloc
 * synchronises the device) allocation on the decode path.  For them the packed metadata is
 * written into a fixed array of FST_STATIC_SCRATCH_BYTES bytes that is part of the library's
 * device image; inputs and outputs are still the caller's.
 *
 *   - Metadata whose packed form (fst_attention_ref_workspace_bytes) exceeds
 *     FST_STATIC_SCRATCH_BYTES is refused with FST_ERR_TOO_LARGE and nothing is launched.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress) with that device current, and the first call with a new
 *     combination of dtype, head_dim and block_m sets the shared-memory attribute of the kernel
 *     it picks and builds its tensor maps (host memory only): make one call per such combination
 *     before any stream capture begins.  Calls after that only launch kernels.  No call
 *     allocates or frees device memory.
 *   - All calls on a device share the one array and it keeps whatever the last call wrote;
 *     every call rewrites all of it that it reads, so nothing has to be cleared.  Two calls
 *     whose kernels can overlap on the GPU (different streams without ordering) race on it:
 *     keep calls on one stream or order them with events.
 */
#define FST_STATIC_SCRATCH_BYTES (512 * 1024)
int fst_attention_fwd_ref_static(const void *q, const void *k, const void *v, void *o, float *lse,
                                 const int64_t *ancestor_idx, const uint8_t *ancestor_mask,
                                 const int64_t *leaf_idx, int n_meta_trees,
                                 int Z, int H, int n_q, int n_kv, int head_dim,
                                 int64_t q_stride_z, int64_t q_stride_h, int64_t q_stride_n,
                                 int64_t k_stride_z, int64_t k_stride_h, int64_t k_stride_n,
                                 int64_t v_stride_z, int64_t v_stride_h, int64_t v_stride_n,
                                 int64_t o_stride_z, int64_t o_stride_h, int64_t o_stride_n,
                                 int block_m, int max_ancestors, float sm_scale, int dtype,
                                 int kernel, int32_t *status, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* FSTATTN_B200_H */
