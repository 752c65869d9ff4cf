// A caller of the C ABI with no Python and no torch: builds the block metadata of a small tree,
// runs tree attention in fp32, and checks the result against a plain loop on the host.
// Build: nvcc -I include tests/cabi/cabi_example.cu -L fstattention_b200 -lfstattn_b200 -o cabi_example
#include <chrono>
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
    if (worst > 2e-5) return 1;

    // Host cost of the entry point at a decoder's shapes (fp16, 32 heads x 256 nodes x 128, 64-row
    // blocks): how long fst_attention_fwd takes to return, on sixteen rotating layer buffers, with
    // the flag that lets the kernel fetch its index lists early.  After the first round the
    // library encodes no tensor map any more (they are kept per thread), so a call is argument
    // checks plus one launch.
    {
        const int N2 = 256, H2 = 32, D2 = 128, BM2 = 64, MA2 = 256, LAYERS = 16, NB2 = N2 / BM2;
        std::vector<int32_t> par2(N2);
        par2[0] = -1;
        for (int i = 1; i < N2; ++i) par2[i] = (i * 7 + 3) % i;
        int32_t *d_par2;
        void *d_packed2, *d_buf;
        const size_t pk2 = fst_packed_meta_bytes(NB2, BM2, MA2), tensor = size_t(H2) * N2 * D2 * 2;
        CHECK_CUDA(cudaMalloc(&d_par2, N2 * sizeof(int32_t)));
        CHECK_CUDA(cudaMalloc(&d_packed2, pk2));
        CHECK_CUDA(cudaMalloc(&d_buf, tensor * 4 * LAYERS));
        CHECK_CUDA(cudaMemset(d_buf, 0, tensor * 4 * LAYERS));
        CHECK_CUDA(cudaMemcpy(d_par2, par2.data(), N2 * sizeof(int32_t), cudaMemcpyHostToDevice));
        CHECK_FST(fst_precompute(d_par2, 1, N2, BM2, MA2, nullptr, nullptr, nullptr, d_packed2, pk2, d_status, stream));
        auto layer_call = [&](int l, int flags) {
            char *base = static_cast<char *>(d_buf) + size_t(l) * 4 * tensor;
            return fst_attention_fwd(base, base + tensor, base + 2 * tensor, base + 3 * tensor, nullptr, d_packed2, 0, 1, H2,
                                     N2, N2, D2, int64_t(H2) * N2 * D2, int64_t(N2) * D2, D2, int64_t(H2) * N2 * D2,
                                     int64_t(N2) * D2, D2, int64_t(H2) * N2 * D2, int64_t(N2) * D2, D2,
                                     int64_t(H2) * N2 * D2, int64_t(N2) * D2, D2, BM2, MA2, 0.088f, FST_F16,
                                     FST_KERNEL_AUTO | flags, d_status, stream);
        };
        for (int l = 0; l < LAYERS; ++l) CHECK_FST(layer_call(l, l ? FST_KERNEL_FLAG_META_STABLE : 0));
        CHECK_CUDA(cudaStreamSynchronize(stream));
        const int rounds = 200;
        const auto t0 = std::chrono::steady_clock::now();
        for (int r = 0; r < rounds; ++r)
            for (int l = 0; l < LAYERS; ++l) CHECK_FST(layer_call(l, FST_KERNEL_FLAG_META_STABLE));
        const auto t1 = std::chrono::steady_clock::now();
        CHECK_CUDA(cudaStreamSynchronize(stream));
        const auto t2 = std::chrono::steady_clock::now();
        const double calls = double(rounds) * LAYERS;
        std::printf("host time per fst_attention_fwd call: %.2f us to return, %.2f us per call until the stream is idle\n",
                    std::chrono::duration<double, std::micro>(t1 - t0).count() / calls,
                    std::chrono::duration<double, std::micro>(t2 - t0).count() / calls);
        CHECK_CUDA(cudaMemcpy(status, d_status, sizeof(status), cudaMemcpyDeviceToHost));
        if (status[0] != 0) { std::printf("device status %d (%s)\n", status[0], fst_status_string(status[0])); return 4; }
    }
    return 0;
}
