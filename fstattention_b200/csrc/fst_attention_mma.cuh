// Tree attention on tensor cores for fp16 / bf16, head_dim 64 or 128 (sm_100a).
//
// One CTA per (query block, head, batch element); warp w owns query rows 16w..16w+15.
// What is computed follows the reference's _fwd_kernel (fstattention.py:21-151) with two
// structural differences: ancestors are taken in tiles of TN rows with a real online softmax
// (the reference has a single tile of MAX_ANCESTORS columns, fstattention.py:75-84), and the
// shared prefix is walked with the same tile loop (fstattention.py:113-136).
//
// Data movement.  Every K/V row this block needs is brought into shared memory with 16-byte
// cp.async.cg copies (L1 bypassed): 16 consecutive threads fetch one 256-byte row, so a warp
// instruction covers two whole rows.  The block's own rows (needed by the leaf path, the
// diagonal term of fstattention.py:86-91 and :104-107) are contiguous and do not depend on the
// metadata, so they and Q are requested before the ancestor indices have even arrived; the
// gathered ancestor tiles are double buffered.  Rows are padded by 16 bytes in shared memory
// so ldmatrix and the 4-byte fragment accesses are bank-conflict free.
//
// Arithmetic.  S = Q K^T and O += P V use mma.sync m16n8k16 with fp32 accumulation; P is rounded
// to the input type for the second product, as in fstattention.py:102.  Q is not pre-scaled:
// scores are scaled by sm_scale*log2(e) in fp32 (the reference rounds the scaled Q to fp16,
// fstattention.py:78) and the leaf term stays in fp32 throughout.  The tree mask is read as
// packed bits.  Column tiles that hold no ancestor are skipped.

#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fst_common.cuh"

namespace fst {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte global->shared copy; bytes beyond src_bytes (0 or 16) are zero filled
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

template <typename T> struct MmaTraits;
template <> struct MmaTraits<__half> {
    __device__ static __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    __device__ static __forceinline__ uint32_t pack(float x, float y) {
        __half2 h = __floats2half2_rn(x, y);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    __device__ static __forceinline__ float2 unpack(uint32_t u) {
        return __half22float2(*reinterpret_cast<__half2 *>(&u));
    }
};
template <> struct MmaTraits<__nv_bfloat16> {
    __device__ static __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    __device__ static __forceinline__ uint32_t pack(float x, float y) {
        __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    __device__ static __forceinline__ float2 unpack(uint32_t u) {
        return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&u));
    }
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

template <int D, int BM, int TN>
struct MmaSmem {
    static constexpr int RS = D * 2 + 16;                 // padded row, bytes
    static constexpr int Q = 0;
    static constexpr int KB = Q + BM * RS;
    static constexpr int VB = KB + BM * RS;
    static constexpr int KA = VB + BM * RS;               // [2][TN] rows
    static constexpr int VA = KA + 2 * TN * RS;           // [2][TN] rows
    static constexpr int MASK = VA + 2 * TN * RS;         // [BM][maw] words
    static size_t bytes(int maw) { return size_t(MASK) + size_t(BM) * maw * 4; }
};

template <typename T, int D, int BM, int TN>
__global__ void __launch_bounds__(BM * 2)
attn_mma_kernel(const AttnArgs a) {
    using MT = MmaTraits<T>;
    using SM = MmaSmem<D, BM, TN>;
    constexpr int RS = SM::RS;
    constexpr int NT = BM * 2;            // threads
    constexpr int CH = D * 2 / 16;        // 16-byte chunks per row
    constexpr int KS = D / 16;            // k-steps of Q K^T
    constexpr int ND = D / 8;             // 8-wide output column tiles
    constexpr int NS = TN / 8;            // 8-wide score column tiles

    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t s_base = smem_u32(smem);
    const int b = blockIdx.x, h = blockIdx.y, z = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = b * BM;

    const PackedLayout L = packed_layout(a.nb, BM, a.ma);
    const int maw = L.maw;
    const unsigned char *blob = a.packed + size_t(z) * a.meta_stride;
    const int32_t *g_idx = reinterpret_cast<const int32_t *>(blob + L.off_idx) + size_t(b) * a.ma;
    const unsigned char *g_mask = blob + L.off_mask + size_t(b) * BM * maw * 4;
    const uint32_t *g_leaf = reinterpret_cast<const uint32_t *>(blob + L.off_leaf) + size_t(b) * L.lw;
    int count = reinterpret_cast<const int32_t *>(blob + L.off_count)[b];

    const T *qp = static_cast<const T *>(a.q) + z * a.qs_z + h * a.qs_h;
    const T *kp = static_cast<const T *>(a.k) + z * a.ks_z + h * a.ks_h;
    const T *vp = static_cast<const T *>(a.v) + z * a.vs_z + h * a.vs_h;
    T *op = static_cast<T *>(a.o) + z * a.os_z + h * a.os_h;
    const int prefix = a.prefix, n_q = a.n_q;

    // my two rows inside the block, and whether each takes the leaf path
    const int r0 = warp * 16 + g, r1 = r0 + 8;
    const uint32_t leaf_w0 = g_leaf[r0 >> 5], leaf_w1 = g_leaf[r1 >> 5];

    // ---- loads that do not depend on the metadata: Q, this block's K rows, mask words
    for (int i = tid; i < BM * CH; i += NT) {
        const int r = i / CH, c = i - r * CH, row = row0 + r;
        const bool ok = row < n_q;
        const long long rr = ok ? row : 0;
        cp_async16(s_base + SM::Q + r * RS + c * 16, qp + rr * a.qs_n + c * 8, ok);
        cp_async16(s_base + SM::KB + r * RS + c * 16, kp + (prefix + rr) * a.ks_n + c * 8, ok);
    }
    for (int i = tid; i < BM * maw / 4; i += NT)
        cp_async16(s_base + SM::MASK + i * 16, g_mask + i * 16, true);

    // tile `tile` of K or V into stage `st`: ancestor tiles first, then prefix tiles
    count = min(max(count, 0), a.ma);
    const int nt_anc = max(1, (count + TN - 1) / TN);
    const int nt = nt_anc + (prefix + TN - 1) / TN;
    auto load_tile = [&](int tile, int st, const T *base, int64_t stride_n, int smem_off) {
        const uint32_t dst0 = s_base + smem_off + st * TN * RS;
        if (tile < nt_anc) {
            for (int i = tid; i < TN * CH; i += NT) {
                const int s = i / CH, c = i - s * CH, slot = tile * TN + s;
                const int node = slot < a.ma ? __ldg(g_idx + slot) : -1;
                const bool ok = node >= 0 && node < n_q;
                if (node >= n_q) report(a.status, FST_DEV_INDEX_RANGE, b, slot);
                const long long rr = ok ? prefix + node : 0;
                cp_async16(dst0 + s * RS + c * 16, base + rr * stride_n + c * 8, ok);
            }
        } else {
            const int p0 = (tile - nt_anc) * TN;
            for (int i = tid; i < TN * CH; i += NT) {
                const int s = i / CH, c = i - s * CH;
                const bool ok = p0 + s < prefix;
                const long long rr = ok ? p0 + s : 0;
                cp_async16(dst0 + s * RS + c * 16, base + rr * stride_n + c * 8, ok);
            }
        }
    };

    load_tile(0, 0, kp, a.ks_n, SM::KA);
    cp_async_commit();                                    // group 0: Q, block K, mask, K tile 0
    for (int i = tid; i < BM * CH; i += NT) {
        const int r = i / CH, c = i - r * CH, row = row0 + r;
        const bool ok = row < n_q;
        const long long rr = ok ? row : 0;
        cp_async16(s_base + SM::VB + r * RS + c * 16, vp + (prefix + rr) * a.vs_n + c * 8, ok);
    }
    load_tile(0, 0, vp, a.vs_n, SM::VA);
    cp_async_commit();                                    // group 1: block V, V tile 0

    uint32_t qf[KS][4];
    float acc[ND][4];
#pragma unroll
    for (int i = 0; i < ND; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // l is this thread's share

    for (int it = 0; it < nt; ++it) {
        const int st = it & 1;
        if (it + 1 < nt) {
            load_tile(it + 1, st ^ 1, kp, a.ks_n, SM::KA);
            load_tile(it + 1, st ^ 1, vp, a.vs_n, SM::VA);
        }
        cp_async_commit();
        if (it == 0) cp_async_wait<2>(); else cp_async_wait<1>();
        __syncthreads();

        if (it == 0) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
                ldmatrix_x4(qf[ks], s_base + SM::Q + (warp * 16 + (lane & 15)) * RS +
                                        (ks * 16 + (lane >> 4) * 8) * 2);
        }

        // columns of this tile that can hold anything
        const bool anc_tile = it < nt_anc;
        const int cols = anc_tile ? min(TN, count - it * TN) : min(TN, prefix - (it - nt_anc) * TN);
        const int n16 = (max(cols, 0) + 15) >> 4;

        // ---- S = Q K^T
        float s[NS][4];
#pragma unroll
        for (int n = 0; n < NS; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
        const uint32_t ka = s_base + SM::KA + st * TN * RS;
#pragma unroll
        for (int np = 0; np < NS / 2; ++np) {
            if (np < n16) {
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    uint32_t kb[4];
                    ldmatrix_x4(kb, ka + (np * 16 + ((lane >> 4) << 3) + (lane & 7)) * RS +
                                        (ks * 16 + ((lane >> 3) & 1) * 8) * 2);
                    MT::mma(s[2 * np], qf[ks], kb[0], kb[1]);
                    MT::mma(s[2 * np + 1], qf[ks], kb[2], kb[3]);
                }
            }
        }

        // ---- scale and mask
        float mx0 = -INFINITY, mx1 = -INFINITY;
        if (anc_tile) {
            const uint32_t *sm = reinterpret_cast<const uint32_t *>(smem + SM::MASK);
            uint32_t w0[TN / 32], w1[TN / 32];
#pragma unroll
            for (int w = 0; w < TN / 32; ++w) {
                const int wi = it * (TN / 32) + w;
                w0[w] = wi < maw ? sm[r0 * maw + wi] : 0u;
                w1[w] = wi < maw ? sm[r1 * maw + wi] : 0u;
            }
#pragma unroll
            for (int n = 0; n < NS; ++n) {
                if (n / 2 < n16) {
                    const int c = n * 8 + 2 * t;
                    const uint32_t b0 = w0[c >> 5] >> (c & 31), b1 = w1[c >> 5] >> (c & 31);
                    s[n][0] = (b0 & 1u) ? s[n][0] * a.scale_log2 : -INFINITY;
                    s[n][1] = (b0 & 2u) ? s[n][1] * a.scale_log2 : -INFINITY;
                    s[n][2] = (b1 & 1u) ? s[n][2] * a.scale_log2 : -INFINITY;
                    s[n][3] = (b1 & 2u) ? s[n][3] * a.scale_log2 : -INFINITY;
                    mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
                    mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
                }
            }
        } else {
#pragma unroll
            for (int n = 0; n < NS; ++n) {
                if (n / 2 < n16) {
                    const int c = n * 8 + 2 * t;
                    s[n][0] = c < cols ? s[n][0] * a.scale_log2 : -INFINITY;
                    s[n][1] = c + 1 < cols ? s[n][1] * a.scale_log2 : -INFINITY;
                    s[n][2] = c < cols ? s[n][2] * a.scale_log2 : -INFINITY;
                    s[n][3] = c + 1 < cols ? s[n][3] * a.scale_log2 : -INFINITY;
                    mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
                    mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
                }
            }
        }

        // ---- leaf score: the row against its own K row (first tile only)
        float lq0 = -INFINITY, lq1 = -INFINITY;
        if (it == 0) {
            float d0 = 0.f, d1 = 0.f;
            const unsigned char *kb0 = smem + SM::KB + r0 * RS + t * 4;
            const unsigned char *kb1 = smem + SM::KB + r1 * RS + t * 4;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const float2 q00 = MT::unpack(qf[ks][0]), q10 = MT::unpack(qf[ks][1]);
                const float2 q01 = MT::unpack(qf[ks][2]), q11 = MT::unpack(qf[ks][3]);
                const float2 k00 = MT::unpack(*reinterpret_cast<const uint32_t *>(kb0 + ks * 32));
                const float2 k01 = MT::unpack(*reinterpret_cast<const uint32_t *>(kb0 + ks * 32 + 16));
                const float2 k10 = MT::unpack(*reinterpret_cast<const uint32_t *>(kb1 + ks * 32));
                const float2 k11 = MT::unpack(*reinterpret_cast<const uint32_t *>(kb1 + ks * 32 + 16));
                d0 = fmaf(q00.x, k00.x, fmaf(q00.y, k00.y, fmaf(q01.x, k01.x, fmaf(q01.y, k01.y, d0))));
                d1 = fmaf(q10.x, k10.x, fmaf(q10.y, k10.y, fmaf(q11.x, k11.x, fmaf(q11.y, k11.y, d1))));
            }
            d0 += __shfl_xor_sync(0xffffffffu, d0, 1);
            d0 += __shfl_xor_sync(0xffffffffu, d0, 2);
            d1 += __shfl_xor_sync(0xffffffffu, d1, 1);
            d1 += __shfl_xor_sync(0xffffffffu, d1, 2);
            if (((leaf_w0 >> (r0 & 31)) & 1u) && row0 + r0 < n_q) lq0 = d0 * a.scale_log2;
            if (((leaf_w1 >> (r1 & 31)) & 1u) && row0 + r1 < n_q) lq1 = d1 * a.scale_log2;
            mx0 = fmaxf(mx0, lq0);
            mx1 = fmaxf(mx1, lq1);
        }

        // ---- online softmax (base 2)
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
        const float al0 = fast_exp2(m0 - mu0), al1 = fast_exp2(m1 - mu1);
        m0 = mn0; m1 = mn1;
        float ps0 = 0.f, ps1 = 0.f;
        uint32_t pf[NS / 2][4];
#pragma unroll
        for (int n = 0; n < NS; ++n) {
            if (n / 2 < n16) {
                const float p0 = fast_exp2(s[n][0] - mu0), p1 = fast_exp2(s[n][1] - mu0);
                const float p2 = fast_exp2(s[n][2] - mu1), p3 = fast_exp2(s[n][3] - mu1);
                ps0 += p0 + p1;
                ps1 += p2 + p3;
                pf[n / 2][(n & 1) * 2 + 0] = MT::pack(p0, p1);
                pf[n / 2][(n & 1) * 2 + 1] = MT::pack(p2, p3);
            }
        }
        const float lp0 = fast_exp2(lq0 - mu0), lp1 = fast_exp2(lq1 - mu1);   // 0 unless it == 0
        l0 = l0 * al0 + ps0 + (t == 0 ? lp0 : 0.f);
        l1 = l1 * al1 + ps1 + (t == 0 ? lp1 : 0.f);
#pragma unroll
        for (int i = 0; i < ND; ++i) {
            acc[i][0] *= al0; acc[i][1] *= al0;
            acc[i][2] *= al1; acc[i][3] *= al1;
        }

        if (it == 0) {                                    // V of the first tile and of the block
            cp_async_wait<1>();
            __syncthreads();
        }

        // ---- O += P V
        const uint32_t va = s_base + SM::VA + st * TN * RS;
#pragma unroll
        for (int kk = 0; kk < NS / 2; ++kk) {
            if (kk < n16) {
#pragma unroll
                for (int dp = 0; dp < ND / 2; ++dp) {
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, va + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * RS +
                                              (dp * 16 + (lane >> 4) * 8) * 2);
                    MT::mma(acc[2 * dp], pf[kk], vb[0], vb[1]);
                    MT::mma(acc[2 * dp + 1], pf[kk], vb[2], vb[3]);
                }
            }
        }
        if (it == 0) {                                    // leaf value: the row's own V row
            const unsigned char *vb0 = smem + SM::VB + r0 * RS + t * 4;
            const unsigned char *vb1 = smem + SM::VB + r1 * RS + t * 4;
#pragma unroll
            for (int i = 0; i < ND; ++i) {
                const float2 v0 = MT::unpack(*reinterpret_cast<const uint32_t *>(vb0 + i * 16));
                const float2 v1 = MT::unpack(*reinterpret_cast<const uint32_t *>(vb1 + i * 16));
                acc[i][0] = fmaf(lp0, v0.x, acc[i][0]);
                acc[i][1] = fmaf(lp0, v0.y, acc[i][1]);
                acc[i][2] = fmaf(lp1, v1.x, acc[i][2]);
                acc[i][3] = fmaf(lp1, v1.y, acc[i][3]);
            }
        }
        __syncthreads();                                  // stage st is free for tile it+2
    }

    // ---- epilogue: normalise, stage through this warp's rows of the Q area, store 16 bytes wide
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
    unsigned char *o0 = smem + SM::Q + r0 * RS + t * 4, *o1 = smem + SM::Q + r1 * RS + t * 4;
#pragma unroll
    for (int i = 0; i < ND; ++i) {
        *reinterpret_cast<uint32_t *>(o0 + i * 16) = MT::pack(acc[i][0] * inv0, acc[i][1] * inv0);
        *reinterpret_cast<uint32_t *>(o1 + i * 16) = MT::pack(acc[i][2] * inv1, acc[i][3] * inv1);
    }
    __syncwarp();
    for (int i = lane; i < 16 * CH; i += 32) {
        const int r = i / CH, c = i - r * CH, row = row0 + warp * 16 + r;
        if (row < n_q) {
            const uint4 val = *reinterpret_cast<const uint4 *>(smem + SM::Q + (warp * 16 + r) * RS + c * 16);
            *reinterpret_cast<uint4 *>(op + (long long)row * a.os_n + c * 8) = val;
        }
    }
    if (a.lse != nullptr && t == 0) {
        float *lse = a.lse + (size_t(z) * a.H + h) * n_q;
        if (row0 + r0 < n_q) lse[row0 + r0] = m0 + log2f(l0);
        if (row0 + r1 < n_q) lse[row0 + r1] = m1 + log2f(l1);
    }
}

template <typename T, int D, int BM, int TN>
cudaError_t launch_mma_inst(const AttnArgs &a, cudaStream_t stream) {
    using SM = MmaSmem<D, BM, TN>;
    const size_t smem = SM::bytes((a.ma + 31) / 32);
    if (smem > 227 * 1024) return cudaErrorNotSupported;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_mma_kernel<T, D, BM, TN>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        configured = smem;
    }
    dim3 grid(a.nb, a.H, a.Z), block(BM * 2);
    attn_mma_kernel<T, D, BM, TN><<<grid, block, smem, stream>>>(a);
    return cudaGetLastError();
}

template <typename T, int D>
cudaError_t launch_mma_d(const AttnArgs &a, int tile_rows, cudaStream_t stream) {
    if (tile_rows == 64) {
        switch (a.bm) {
            case 16: return launch_mma_inst<T, D, 16, 64>(a, stream);
            case 32: return launch_mma_inst<T, D, 32, 64>(a, stream);
            case 64: return launch_mma_inst<T, D, 64, 64>(a, stream);
            case 128: return launch_mma_inst<T, D, 128, 64>(a, stream);
        }
    } else if (tile_rows == 32) {
        switch (a.bm) {
            case 16: return launch_mma_inst<T, D, 16, 32>(a, stream);
            case 32: return launch_mma_inst<T, D, 32, 32>(a, stream);
            case 64: return launch_mma_inst<T, D, 64, 32>(a, stream);
            case 128: return launch_mma_inst<T, D, 128, 32>(a, stream);
        }
    }
    return cudaErrorNotSupported;
}

}  // namespace fst
