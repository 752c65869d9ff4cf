// Tree construction on the device: from the top-k candidate scores of the speculation heads to
// a parent array, without a host round trip.
//
// The reference only builds a fixed synthetic forest on the CPU (create_tree, utils.py:27-77):
// topk roots, level sizes size[l] = topk * int(size[l-1] * left_weight_factor), node r of a level
// hanging under node r / topk of the level above - a "left-weighted" tree in which only the
// first part of every level is expanded.  Its README (README.md:17) names the use: Medusa-style
// trees, the cartesian products of every head's top-k candidates.  This kernel is that
// construction driven by scores: head l gives topk candidate scores (log-probabilities, any
// order), a node's score is the sum along its path, and of every level the
// int(size * left_weight_factor) best nodes are expanded, best first, each into the topk
// candidates of the next head.  With equal scores "best" falls back to position and the result
// is exactly create_tree's forest.  Node numbering is level by level, so parents precede their
// children and fst_dfs_order / fst_precompute can take the array as it is.
//
// One CTA per tree.  A level is at most LEVEL_CAP nodes; ranking them is a count of the nodes
// that beat each one (ties broken by position, which makes the order total and the kept set
// the one a stable sort would give), quadratic in the level size, all in shared memory.

#include "fst_common.cuh"

namespace fst {

constexpr int BUILD_THREADS = 512;
constexpr int LEVEL_CAP = 4096;

struct LevelPlan {
    int n_levels;                       // depth + 1
    int size[kMaxTreeLevels];           // nodes of level l
    int start[kMaxTreeLevels + 1];      // first node of level l; start[n_levels] = node count
};

__global__ void __launch_bounds__(BUILD_THREADS)
build_tree_topk_kernel(const float *__restrict__ scores_all, int topk, LevelPlan plan, int max_nodes,
                       int32_t *__restrict__ parent_all, int32_t *__restrict__ choice_all,
                       float *__restrict__ node_score_all) {
    __shared__ float cum[2][LEVEL_CAP];                   // path scores of the previous / the new level
    __shared__ int slot[LEVEL_CAP];                       // slot[r] = position (in its level) of the r-th best node
    const int tree = blockIdx.x, tid = threadIdx.x;
    const float *scores = scores_all + size_t(tree) * plan.n_levels * topk;
    int32_t *parent = parent_all + size_t(tree) * max_nodes;
    int32_t *choice = choice_all ? choice_all + size_t(tree) * max_nodes : nullptr;
    float *node_score = node_score_all ? node_score_all + size_t(tree) * max_nodes : nullptr;

    for (int i = tid; i < plan.size[0]; i += BUILD_THREADS) {
        const float s = scores[i];
        cum[0][i] = s;
        if (i < max_nodes) {
            parent[i] = -1;
            if (choice) choice[i] = i;
            if (node_score) node_score[i] = s;
        }
    }
    // rows past the last node of the forest (a caller with fixed-size tensors): isolated roots
    for (int i = plan.start[plan.n_levels] + tid; i < max_nodes; i += BUILD_THREADS) {
        parent[i] = -1;
        if (choice) choice[i] = -1;
        if (node_score) node_score[i] = -INFINITY;
    }
    __syncthreads();
    int cur = 0;
    for (int l = 1; l < plan.n_levels; ++l) {
        const int prev = plan.size[l - 1], here = plan.size[l], keep = here / topk;
        const float *c = cum[cur];
        // the r-th best node of the previous level, r < keep, will be expanded
        for (int i = tid; i < prev; i += BUILD_THREADS) {
            const float mine = c[i];
            int better = 0;
            for (int j = 0; j < prev; ++j) {
                const float other = c[j];
                better += (other > mine) || (other == mine && j < i);
            }
            if (better < keep) slot[better] = i;
        }
        __syncthreads();
        float *nxt = cum[cur ^ 1];
        const float *head = scores + size_t(l) * topk;
        for (int r = tid; r < here; r += BUILD_THREADS) {
            const int p = slot[r / topk], k = r - (r / topk) * topk;
            const float s = c[p] + head[k];
            nxt[r] = s;
            const int node = plan.start[l] + r;
            if (node < max_nodes) {
                parent[node] = plan.start[l - 1] + p;
                if (choice) choice[node] = l * topk + k;
                if (node_score) node_score[node] = s;
            }
        }
        __syncthreads();
        cur ^= 1;
    }
}

// Level sizes of the forest (the reference's recurrence, utils.py:46-52, in the same double
// arithmetic Python uses).  Returns the node count, or -1 when a level outgrows the kernel.
static long long plan_levels(int depth, int topk, double left_weight_factor, LevelPlan *plan) {
    if (depth < 0 || depth + 1 > kMaxTreeLevels || topk < 1) return -1;
    long long total = 0;
    long long sz = topk;
    for (int l = 0; l <= depth; ++l) {
        if (l > 0) sz = (long long)topk * (long long)(double(sz) * left_weight_factor);
        if (sz < 0 || sz > LEVEL_CAP) return -1;
        if (plan) {
            plan->size[l] = int(sz);
            plan->start[l] = int(total);
        }
        total += sz;
    }
    if (plan) {
        plan->n_levels = depth + 1;
        plan->start[depth + 1] = int(total);
    }
    return total;
}

long long tree_topk_nodes(int depth, int topk, double left_weight_factor) {
    return plan_levels(depth, topk, left_weight_factor, nullptr);
}

cudaError_t launch_build_tree_topk(const float *scores, int n_trees, int depth, int topk,
                                   double left_weight_factor, int max_nodes, int32_t *parent, int32_t *choice,
                                   float *node_score, cudaStream_t stream) {
    LevelPlan plan;
    const long long total = plan_levels(depth, topk, left_weight_factor, &plan);
    if (total < 0) return cudaErrorInvalidConfiguration;
    build_tree_topk_kernel<<<n_trees, BUILD_THREADS, 0, stream>>>(scores, topk, plan, max_nodes, parent, choice,
                                                                  node_score);
    return cudaGetLastError();
}

}  // namespace fst
