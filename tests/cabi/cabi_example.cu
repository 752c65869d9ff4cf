// A caller of the C ABI with no Python and no torch: builds the block metadata of a small tree,
// runs tree attention in fp32, and checks the result against a plain loop on the host.
// Build: nvcc -I include tests/cabi/cabi_example.cu -L fstattention_b200 -lfstattn_b200 -o cabi_example
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include <cuda_runtime.h>

#include "fstattn_b200.h"

#define CHECK_CUDA(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); return 2; } } while (0)
#define CHECK_FST(x) do { int s_ = (x); if (s_ != FST_OK) { std::printf("fst error %d (%s) at %s:%d\n", s_, fst_status_string(s_), __FILE__, __LINE__); return 3; } } while (0)

int main() {
    const int N = 45, H = 3, D = 32, BM = 16, MA = 48, P = 5;      // 45 nodes, 5 prefix rows, ragged last block
    const int NKV = P + N, NB = (N + BM - 1) / BM;
    std::vector<int32_t> parent(N);
    parent[0] = -1;
    for (int i = 1; i < N; ++i) parent[i] = (i * 7 + 3) % i;        // some tree with parent[i] < i
    const float scale = 1.0f / std::sqrt(float(D));

    std::vector<float> q(size_t(H) * N * D), k(size_t(H) * NKV * D), v(k.size());
    unsigned seed = 12345u;
    auto rnd = [&]() { seed = seed * 1664525u + 1013904223u; return float(int(seed >> 9) % 2001 - 1000) / 1000.f; };
    for (auto &x : q) x = rnd();
    for (auto &x : k) x = rnd();
    for (auto &x : v) x = rnd();

    int32_t *d_parent, *d_status;
    void *d_packed;
    float *d_q, *d_k, *d_v, *d_o, *d_lse;
    const size_t packed_bytes = fst_packed_meta_bytes(NB, BM, MA);
    CHECK_CUDA(cudaMalloc(&d_parent, N * sizeof(int32_t)));
    CHECK_CUDA(cudaMalloc(&d_status, 4 * sizeof(int32_t)));
    CHECK_CUDA(cudaMemset(d_status, 0, 4 * sizeof(int32_t)));
    CHECK_CUDA(cudaMalloc(&d_packed, packed_bytes));
    CHECK_CUDA(cudaMalloc(&d_q, q.size() * 4));
    CHECK_CUDA(cudaMalloc(&d_k, k.size() * 4));
    CHECK_CUDA(cudaMalloc(&d_v, v.size() * 4));
    CHECK_CUDA(cudaMalloc(&d_o, q.size() * 4));
    CHECK_CUDA(cudaMalloc(&d_lse, size_t(H) * N * 4));
    CHECK_CUDA(cudaMemcpy(d_parent, parent.data(), N * sizeof(int32_t), cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(d_q, q.data(), q.size() * 4, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(d_k, k.data(), k.size() * 4, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(d_v, v.data(), v.size() * 4, cudaMemcpyHostToDevice));

    cudaStream_t stream;
    CHECK_CUDA(cudaStreamCreate(&stream));
    CHECK_FST(fst_precompute(d_parent, 1, N, BM, MA, nullptr, nullptr, nullptr, d_packed, packed_bytes, d_status, stream));
    CHECK_FST(fst_attention_fwd(d_q, d_k, d_v, d_o, d_lse, d_packed, 0, 1, H, N, NKV, D,
                                int64_t(H) * N * D, int64_t(N) * D, D, int64_t(H) * NKV * D, int64_t(NKV) * D, D,
                                int64_t(H) * NKV * D, int64_t(NKV) * D, D, int64_t(H) * N * D, int64_t(N) * D, D,
                                BM, MA, scale, FST_F32, FST_KERNEL_AUTO, d_status, stream));
    CHECK_CUDA(cudaStreamSynchronize(stream));
    int32_t status[4];
    CHECK_CUDA(cudaMemcpy(status, d_status, sizeof(status), cudaMemcpyDeviceToHost));
    if (status[0] != 0) { std::printf("device status %d (%s)\n", status[0], fst_status_string(status[0])); return 4; }
    std::vector<float> o(q.size());
    CHECK_CUDA(cudaMemcpy(o.data(), d_o, o.size() * 4, cudaMemcpyDeviceToHost));

    // host check: row i attends to the prefix rows, its ancestors and itself
    double worst = 0.0;
    for (int h = 0; h < H; ++h)
        for (int i = 0; i < N; ++i) {
            std::vector<int> rows;
            for (int p = 0; p < P; ++p) rows.push_back(p);
            for (int a = i; a >= 0; a = parent[a]) rows.push_back(P + a);
            std::vector<double> w(rows.size());
            double mx = -1e300, sum = 0.0;
            for (size_t j = 0; j < rows.size(); ++j) {
                double s = 0.0;
                for (int d = 0; d < D; ++d) s += double(q[(size_t(h) * N + i) * D + d]) * k[(size_t(h) * NKV + rows[j]) * D + d];
                w[j] = s * scale;
                mx = std::max(mx, w[j]);
            }
            for (auto &x : w) { x = std::exp(x - mx); sum += x; }
            for (int d = 0; d < D; ++d) {
                double acc = 0.0;
                for (size_t j = 0; j < rows.size(); ++j) acc += w[j] * v[(size_t(h) * NKV + rows[j]) * D + d];
                worst = std::max(worst, std::fabs(acc / sum - double(o[(size_t(h) * N + i) * D + d])));
            }
        }
    std::printf("fst_version %d, max-abs difference from the host loop %.3e\n", fst_version(), worst);
    return worst <= 2e-5 ? 0 : 1;
}
