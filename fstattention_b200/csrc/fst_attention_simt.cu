// Tree attention, fp32-arithmetic kernel for every dtype and head_dim in {16,32,64,128}.
//
// Computes what the reference's _fwd_kernel computes (fstattention.py:21-151): for each query
// row of a block, softmax over {its ancestors outside the block, from the block's gathered
// list} + {itself and its ancestors inside the block} + {every shared-prefix row}, times V.  One warp owns one
// query row at a time; keys are taken 32 at a time, one per lane, with an online softmax in
// base 2 (scores are scaled by sm_scale*log2(e) like fstattention.py:59).  All arithmetic is
// fp32, so fp32 inputs keep fp32 accuracy; this is the kernel for fp32 tensors, small head
// dimensions and odd block sizes.  The tensor-core kernel covers fp16/bf16 at D=64/128.

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fst_common.cuh"

namespace fst {

constexpr int SIMT_WARPS = 4;

template <typename T> __device__ inline float to_float(T x);
template <> __device__ inline float to_float<float>(float x) { return x; }
template <> __device__ inline float to_float<__half>(__half x) { return __half2float(x); }
template <> __device__ inline float to_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ inline T from_float(float x);
template <> __device__ inline float from_float<float>(float x) { return x; }
template <> __device__ inline __half from_float<__half>(float x) { return __float2half_rn(x); }
template <> __device__ inline __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

template <typename T, int D>
__global__ void __launch_bounds__(SIMT_WARPS * 32)
attn_simt_kernel(const AttnArgs a) {
    constexpr int NV = (D + 31) / 32;                 // output columns per lane
    __shared__ float s_q[SIMT_WARPS][D];
    const int b = blockIdx.x, h = blockIdx.y, z = blockIdx.z;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;

    const PackedLayout L = packed_layout(a.nb, a.bm, a.ma);
    const unsigned char *blob = a.packed + size_t(z) * a.meta_stride;
    const int count = min(max(reinterpret_cast<const int32_t *>(blob + L.off_count)[b], 0), a.ma);
    const int32_t *idx = reinterpret_cast<const int32_t *>(blob + L.off_idx) + size_t(b) * a.ma;
    const uint32_t *emask = reinterpret_cast<const uint32_t *>(blob + L.off_emask) + size_t(b) * a.bm * L.maw;
    const uint32_t *bmask = reinterpret_cast<const uint32_t *>(blob + L.off_bmask) + size_t(b) * a.bm * L.bw;

    const T *qp = static_cast<const T *>(a.q) + z * a.qs_z + h * a.qs_h;
    const int hk = h / a.kv_group;                        // my K/V head
    const T *kp = static_cast<const T *>(a.k) + z * a.ks_z + hk * a.ks_h;
    const T *vp = static_cast<const T *>(a.v) + z * a.vs_z + hk * a.vs_h;
    T *op = static_cast<T *>(a.o) + z * a.os_z + h * a.os_h;

    for (int j = wid; j < a.bm; j += SIMT_WARPS) {
        const int row = b * a.bm + j;
        if (row >= a.n_q) break;                      // rows only grow with j
        __syncwarp();
        for (int d = lane; d < D; d += 32) s_q[wid][d] = to_float(qp[row * a.qs_n + d]);
        __syncwarp();

        float m = -INFINITY, l = 0.f, acc[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) acc[i] = 0.f;

        // one step of the online softmax over up to 32 keys (lane's key row, or -1)
        auto absorb = [&](long long key) {
            float s = -INFINITY;
            if (key >= 0) {
                const T *kr = kp + key * a.ks_n;
                float dot = 0.f;
#pragma unroll 8
                for (int d = 0; d < D; ++d) dot = fmaf(s_q[wid][d], to_float(kr[d]), dot);
                s = dot * a.scale_log2;
            }
            float cm = s;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
            if (cm == -INFINITY) return;              // no key in this chunk (uniform)
            const float m_new = fmaxf(m, cm);
            const float alpha = exp2f(m - m_new);
            const float p = key >= 0 ? exp2f(s - m_new) : 0.f;
            float ps = p;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
            l = l * alpha + ps;
#pragma unroll
            for (int i = 0; i < NV; ++i) acc[i] *= alpha;
            for (int jj = 0; jj < 32; ++jj) {
                const long long kj = __shfl_sync(0xffffffffu, key, jj);
                const float pj = __shfl_sync(0xffffffffu, p, jj);
                if (kj >= 0) {
                    const T *vr = vp + kj * a.vs_n;
#pragma unroll
                    for (int i = 0; i < NV; ++i) {
                        const int d = lane + 32 * i;
                        if (d < D) acc[i] = fmaf(pj, to_float(vr[d]), acc[i]);
                    }
                }
            }
            m = m_new;
        };

        for (int a0 = 0; a0 < count; a0 += 32) {      // external ancestors, gated by mask bits
            const int s = a0 + lane;
            long long key = -1;
            if (s < count && ((emask[j * L.maw + (s >> 5)] >> (s & 31)) & 1u)) {
                const int node = idx[s];
                if (node >= 0 && node < a.n_q) key = a.prefix + node;
                else report(a.status, FST_DEV_INDEX_RANGE, b, s);
            }
            absorb(key);
        }
        for (int c0 = 0; c0 < a.bm; c0 += 32) {       // the row itself and ancestors in the block
            const int c = c0 + lane, node = b * a.bm + c;
            const bool on = c < a.bm && ((bmask[j * L.bw + (c >> 5)] >> (c & 31)) & 1u) && node < a.n_q;
            absorb(on ? (long long)(a.prefix + node) : -1LL);
        }
        for (int p0 = 0; p0 < a.prefix; p0 += 32)     // shared prefix, dense
            absorb(p0 + lane < a.prefix ? (long long)(p0 + lane) : -1LL);

        const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int d = lane + 32 * i;
            if (d < D) op[row * a.os_n + d] = from_float<T>(acc[i] * inv);
        }
        if (a.lse && lane == 0)
            a.lse[(size_t(z) * a.H + h) * a.n_q + row] = m + log2f(l);
    }
}

template <typename T>
static cudaError_t launch_simt_t(const AttnArgs &a, cudaStream_t stream) {
    dim3 grid(a.nb, a.H, a.Z), block(SIMT_WARPS * 32);
    switch (a.D) {
        case 16: attn_simt_kernel<T, 16><<<grid, block, 0, stream>>>(a); break;
        case 32: attn_simt_kernel<T, 32><<<grid, block, 0, stream>>>(a); break;
        case 64: attn_simt_kernel<T, 64><<<grid, block, 0, stream>>>(a); break;
        case 128: attn_simt_kernel<T, 128><<<grid, block, 0, stream>>>(a); break;
        default: return cudaErrorNotSupported;
    }
    return cudaGetLastError();
}

cudaError_t launch_attention_simt(const AttnArgs &a, int dtype, cudaStream_t stream) {
    switch (dtype) {
        case FST_F16: return launch_simt_t<__half>(a, stream);
        case FST_BF16: return launch_simt_t<__nv_bfloat16>(a, stream);
        case FST_F32: return launch_simt_t<float>(a, stream);
        default: return cudaErrorNotSupported;
    }
}

}  // namespace fst
