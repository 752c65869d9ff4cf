// Tree attention on tensor cores for fp16 / bf16, head_dim 64 or 128 (sm_100a).
//
// One CTA per (query block, head, batch element); warp w owns query rows 16w..16w+15.
// What is computed follows the reference's _fwd_kernel (fstattention.py:21-151).  The work of a
// block is cut into column tiles of 32 K/V rows, all handled by one piece of code:
//   * the block's own rows (contiguous in memory; they carry the self term - the reference's
//     leaf path, fstattention.py:86-91 and :104-107 - and the ancestors that live inside the
//     block), masked by the per-row in-block bit mask;
//   * the gathered external ancestors, masked by the per-row ancestor bit mask (the reference
//     takes one tile of MAX_ANCESTORS columns, fstattention.py:75-84; here any number);
//   * the shared prefix, dense (fstattention.py:113-136).
// A warp skips a tile, or a 16-column half of it, when none of its 16 rows has a mask bit
// there, so the tensor-core work tracks the tree, not the padded tile shape.
//
// Data movement.  K/V rows go to shared memory with 16-byte cp.async.cg copies (L1 bypassed):
// 16 consecutive threads fetch one 256-byte row, so one warp instruction covers two whole
// rows.  The block's own rows do not depend on the metadata and are requested first; the
// first two gathered tiles are requested right behind them, later ones are double buffered.
// Shared-memory rows are padded by 16 bytes so ldmatrix is bank-conflict free.  Q goes from
// global memory straight into mma A fragments and O straight from the accumulators to global
// memory: each quad reads or writes a 16-byte piece of a row, neighbouring instructions
// complete the 32-byte sectors.
//
// Arithmetic.  S = Q K^T and O += P V use mma.sync m16n8k16 with fp32 accumulation; P is rounded
// to the input type for the second product, as in fstattention.py:102.  Q is not pre-scaled:
// scores are scaled by sm_scale*log2(e) in fp32 inside the exponent (the reference rounds the
// scaled Q to fp16, fstattention.py:78).  The running maximum is tracked in raw score units, so a
// negative sm_scale is applied as a sign flip of Q and |sm_scale| in the exponent.

#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fst_common.cuh"

namespace fst {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte global->shared copy; with valid == false nothing is read and zeros are written
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
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

constexpr int MMA_TN = 32;                                // K/V rows per column tile

template <int TN = MMA_TN>
__device__ __forceinline__ int nt_ext_of(int count, int ma) {   // external-ancestor tiles
    return (min(max(count, 0), ma) + TN - 1) / TN;
}

template <int D, int BM>
struct MmaSmem {
    static constexpr int RS = D * 2 + 16;                 // padded row, bytes
    static constexpr int KB = 0;                          // the block's own K rows
    static constexpr int VB = KB + BM * RS;
    static constexpr int KE = VB + BM * RS;               // [2][MMA_TN] gathered / prefix K rows
    static constexpr int VE = KE + 2 * MMA_TN * RS;
    static constexpr int BYTES = VE + 2 * MMA_TN * RS;
};

template <typename T, int D, int BM>
__global__ void __launch_bounds__(BM * 2, (BM <= 64 ? 3 : 1))
attn_mma_kernel(const AttnArgs a) {
    using MT = MmaTraits<T>;
    using SM = MmaSmem<D, BM>;
    constexpr int RS = SM::RS;
    constexpr int TN = MMA_TN;
    constexpr int NT = BM * 2;            // threads
    constexpr int CH = D / 8;             // 16-byte chunks per row
    constexpr int KS = D / 16;            // k-steps of Q K^T
    constexpr int ND = D / 8;             // 8-wide output column tiles
    constexpr int RPP = NT / CH;          // rows covered by one pass of all threads
    constexpr int NBLK = (BM + TN - 1) / TN;   // column tiles holding the block's own rows
    constexpr int BW = (BM + 31) / 32;
    static_assert(NT % CH == 0, "thread count must cover whole rows");

    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t s_base = smem_u32(smem);
    const int b = blockIdx.x, h = blockIdx.y, z = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = b * BM;
    const int prefix = a.prefix, n_q = a.n_q;

    const PackedLayout L = packed_layout(a.nb, BM, a.ma);
    const int maw = L.maw;
    const unsigned char *blob = a.packed + size_t(z) * a.meta_stride;
    const int32_t *g_idx = reinterpret_cast<const int32_t *>(blob + L.off_idx) + size_t(b) * a.ma;
    const uint32_t *g_emask = reinterpret_cast<const uint32_t *>(blob + L.off_emask) + size_t(b) * BM * maw;
    const uint32_t *g_bmask = reinterpret_cast<const uint32_t *>(blob + L.off_bmask) + size_t(b) * BM * BW;
    int count = __ldg(reinterpret_cast<const int32_t *>(blob + L.off_count) + b);

    const T *qp = static_cast<const T *>(a.q) + z * a.qs_z + h * a.qs_h;
    const int hk = h / a.kv_group;                        // my K/V head
    const T *kp = static_cast<const T *>(a.k) + z * a.ks_z + hk * a.ks_h;
    const T *vp = static_cast<const T *>(a.v) + z * a.vs_z + hk * a.vs_h;
    T *op = static_cast<T *>(a.o) + z * a.os_z + h * a.os_h;

    const int lr = tid / CH, lc = tid % CH;               // my row-in-pass and 16-byte chunk
    constexpr int SPT = TN / RPP;                         // gathered rows per thread and tile
    static_assert(TN % RPP == 0, "a gathered tile must be whole passes");

    // A warp issues in order, so a load result must not be touched before everything that does
    // not depend on it has been requested.  Order: index list and count (plain loads), Q
    // fragments, the block's own rows (cp.async), and only then the gathered rows, whose
    // addresses need the indices.
    const int r0 = warp * 16 + g, r1 = r0 + 8;            // my two rows inside the block
    const bool ok0 = row0 + r0 < n_q, ok1 = row0 + r1 < n_q;

    int nodeA[SPT], nodeB[SPT];                           // my slots of the next two external tiles
    auto fetch_idx = [&](int e, int (&node)[SPT]) {       // the index list is -1 padded
#pragma unroll
        for (int j = 0; j < SPT; ++j) {
            const int slot = e * TN + lr + j * RPP;
            node[j] = slot < a.ma ? __ldg(g_idx + slot) : -1;
        }
    };
    fetch_idx(0, nodeA);
    fetch_idx(1, nodeB);

    uint32_t qf[KS][4];
    {
        const uint32_t *q0 = reinterpret_cast<const uint32_t *>(qp + (long long)(ok0 ? row0 + r0 : 0) * a.qs_n) + t;
        const uint32_t *q1 = reinterpret_cast<const uint32_t *>(qp + (long long)(ok1 ? row0 + r1 : 0) * a.qs_n) + t;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qf[ks][0] = ok0 ? __ldg(q0 + ks * 8) : 0u;
            qf[ks][1] = ok1 ? __ldg(q1 + ks * 8) : 0u;
            qf[ks][2] = ok0 ? __ldg(q0 + ks * 8 + 4) : 0u;
            qf[ks][3] = ok1 ? __ldg(q1 + ks * 8 + 4) : 0u;
        }
        // a negative scale moves into Q as a sign flip (the running maximum below is kept in raw
        // score units, which orders scores correctly only for a positive factor)
        if (a.scale_log2 < 0.f) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
#pragma unroll
                for (int i = 0; i < 4; ++i) qf[ks][i] ^= 0x80008000u;
        }
    }

    // ---- the block's own K and V rows: contiguous, no metadata needed
    auto load_block = [&](const T *base, int64_t stride_n, int smem_off) {
#pragma unroll 1
        for (int r = lr; r < BM; r += RPP) {
            const bool ok = row0 + r < n_q;
            const long long rr = ok ? prefix + row0 + r : 0;
            cp_async16(s_base + smem_off + r * RS + lc * 16, base + rr * stride_n + lc * 8, ok);
        }
    };
    load_block(kp, a.ks_n, SM::KB);
    cp_async_commit();                                    // group 0
    load_block(vp, a.vs_n, SM::VB);
    cp_async_commit();                                    // group 1

    // ---- gathered tiles: external ancestors first, then the prefix
    auto load_gathered = [&](int e, int st, bool ext, const int (&node)[SPT]) {
        const uint32_t kd = s_base + SM::KE + st * TN * RS + lc * 16;
        const uint32_t vd = s_base + SM::VE + st * TN * RS + lc * 16;
#pragma unroll
        for (int j = 0; j < SPT; ++j) {
            const int s = lr + j * RPP;
            long long rr = 0;
            bool ok;
            if (ext) {
                ok = node[j] >= 0 && node[j] < n_q;
                if (node[j] >= n_q) report(a.status, FST_DEV_INDEX_RANGE, b, e * TN + s);
                if (ok) rr = prefix + node[j];
            } else {
                const int p = (e - nt_ext_of(count, a.ma)) * TN + s;
                ok = p < prefix;
                if (ok) rr = p;
            }
            cp_async16(kd + s * RS, kp + rr * a.ks_n + lc * 8, ok);
            cp_async16(vd + s * RS, vp + rr * a.vs_n + lc * 8, ok);
        }
    };
    // without a prefix the first gathered tile is requested before the count has arrived
    if (prefix == 0) {
        load_gathered(0, 0, true, nodeA);
        cp_async_commit();                                // group 2
    }
    const int nt_ext = nt_ext_of(count, a.ma);
    const int nt_gat = nt_ext + (prefix + TN - 1) / TN;
    if (prefix != 0) {
        if (nt_gat > 0) load_gathered(0, 0, nt_ext > 0, nodeA);
        cp_async_commit();                                // group 2
    }
    if (nt_gat > 1) load_gathered(1, 1, nt_ext > 1, nodeB);
    cp_async_commit();                                    // group 3
    fetch_idx(2, nodeA);
    fetch_idx(3, nodeB);

    float acc[ND][4];
#pragma unroll
    for (int i = 0; i < ND; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // m in raw score units; l is my share
    const float c2 = fabsf(a.scale_log2);

    const int n_tiles = NBLK + nt_gat;
    // mask words of my two rows for column tile i (fetched one tile ahead of their use)
    auto mask_words = [&](int i, uint32_t &w0, uint32_t &w1) {
        w0 = w1 = 0u;
        if (i < NBLK) {
            if (ok0) w0 = __ldg(g_bmask + r0 * BW + i);
            if (ok1) w1 = __ldg(g_bmask + r1 * BW + i);
        } else if (i - NBLK < nt_ext) {
            const int e = i - NBLK;
            if (ok0 && e < maw) w0 = __ldg(g_emask + r0 * maw + e);
            if (ok1 && e < maw) w1 = __ldg(g_emask + r1 * maw + e);
        } else if (i < n_tiles) {
            const int rem = prefix - (i - NBLK - nt_ext) * TN;
            w0 = w1 = rem >= 32 ? 0xffffffffu : ((1u << rem) - 1u);
        }
    };
    uint32_t w0n, w1n;
    mask_words(0, w0n, w1n);
#pragma unroll 1
    for (int i = 0; i < n_tiles; ++i) {
        const bool blk = i < NBLK;
        const int e = i - NBLK;                           // gathered tile number
        const uint32_t w0 = w0n, w1 = w1n;
        mask_words(i + 1, w0n, w1n);
        uint32_t kbase, vbase;
        if (blk) {
            kbase = s_base + SM::KB + i * TN * RS;
            vbase = s_base + SM::VB + i * TN * RS;
            if (i == 0) { cp_async_wait<3>(); __syncthreads(); }
        } else {
            kbase = s_base + SM::KE + (e & 1) * TN * RS;
            vbase = s_base + SM::VE + (e & 1) * TN * RS;
            cp_async_wait<1>();
            __syncthreads();
        }
        const uint32_t occ = __reduce_or_sync(0xffffffffu, w0 | w1);   // columns any of my 16 rows use
        const bool lo = (occ & 0xffffu) != 0u, hi = (occ >> 16) != 0u;

        uint32_t pf[2][4];
        if (occ) {
            // ---- S = Q K^T on the occupied 16-column halves
            float s[4][4];
#pragma unroll
            for (int n = 0; n < 4; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
            const uint32_t kaddr = kbase + (((lane >> 4) << 3) + (lane & 7)) * RS + ((lane >> 3) & 1) * 16;
#pragma unroll
            for (int cg = 0; cg < 2; ++cg) {
                if (cg == 0 ? lo : hi) {
#pragma unroll
                    for (int ks = 0; ks < KS; ++ks) {
                        uint32_t kb[4];
                        ldmatrix_x4(kb, kaddr + cg * 16 * RS + ks * 32);
                        MT::mma(s[2 * cg], qf[ks], kb[0], kb[1]);
                        MT::mma(s[2 * cg + 1], qf[ks], kb[2], kb[3]);
                    }
                }
            }
            // ---- mask, running max (raw units), probabilities
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                if (n < 2 ? lo : hi) {
                    const int c = n * 8 + 2 * t;
                    s[n][0] = ((w0 >> c) & 1u) ? s[n][0] : -INFINITY;
                    s[n][1] = ((w0 >> c) & 2u) ? s[n][1] : -INFINITY;
                    s[n][2] = ((w1 >> c) & 1u) ? s[n][2] : -INFINITY;
                    s[n][3] = ((w1 >> c) & 2u) ? s[n][3] : -INFINITY;
                    mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
                    mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
                }
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            const float mu0 = mn0 == -INFINITY ? 0.f : mn0 * c2, mu1 = mn1 == -INFINITY ? 0.f : mn1 * c2;
            const float al0 = fast_exp2(m0 * c2 - mu0), al1 = fast_exp2(m1 * c2 - mu1);
            m0 = mn0; m1 = mn1;
            float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                if (n < 2 ? lo : hi) {
                    const float p0 = fast_exp2(fmaf(s[n][0], c2, -mu0)), p1 = fast_exp2(fmaf(s[n][1], c2, -mu0));
                    const float p2 = fast_exp2(fmaf(s[n][2], c2, -mu1)), p3 = fast_exp2(fmaf(s[n][3], c2, -mu1));
                    ps0 += p0 + p1;
                    ps1 += p2 + p3;
                    pf[n >> 1][(n & 1) * 2 + 0] = MT::pack(p0, p1);
                    pf[n >> 1][(n & 1) * 2 + 1] = MT::pack(p2, p3);
                }
            }
            l0 = l0 * al0 + ps0;
            l1 = l1 * al1 + ps1;
            if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {
#pragma unroll
                for (int d = 0; d < ND; ++d) {
                    acc[d][0] *= al0; acc[d][1] *= al0;
                    acc[d][2] *= al1; acc[d][3] *= al1;
                }
            }
        }

        if (blk && i == 0) { cp_async_wait<2>(); __syncthreads(); }   // the block's V rows

        if (occ) {
            // ---- O += P V
            const uint32_t vaddr = vbase + ((((lane >> 3) & 1) << 3) + (lane & 7)) * RS + (lane >> 4) * 16;
#pragma unroll
            for (int cg = 0; cg < 2; ++cg) {
                if (cg == 0 ? lo : hi) {
#pragma unroll
                    for (int dp = 0; dp < ND / 2; ++dp) {
                        uint32_t vb[4];
                        ldmatrix_x4_trans(vb, vaddr + cg * 16 * RS + dp * 32);
                        MT::mma(acc[2 * dp], pf[cg], vb[0], vb[1]);
                        MT::mma(acc[2 * dp + 1], pf[cg], vb[2], vb[3]);
                    }
                }
            }
        }

        if (!blk) {                                       // recycle this stage for tile e + 2
            if (e + 2 < nt_gat) {
                __syncthreads();
                if (e & 1) {
                    load_gathered(e + 2, 1, e + 2 < nt_ext, nodeB);
                    fetch_idx(e + 4, nodeB);
                } else {
                    load_gathered(e + 2, 0, e + 2 < nt_ext, nodeA);
                    fetch_idx(e + 4, nodeA);
                }
            }
            cp_async_commit();
        }
    }

    // ---- epilogue: normalise and store each quad's 16-byte pieces directly
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
    if (ok0) {
        uint32_t *o0 = reinterpret_cast<uint32_t *>(op + (long long)(row0 + r0) * a.os_n) + t;
#pragma unroll
        for (int d = 0; d < ND; ++d) o0[d * 4] = MT::pack(acc[d][0] * inv0, acc[d][1] * inv0);
    }
    if (ok1) {
        uint32_t *o1 = reinterpret_cast<uint32_t *>(op + (long long)(row0 + r1) * a.os_n) + t;
#pragma unroll
        for (int d = 0; d < ND; ++d) o1[d * 4] = MT::pack(acc[d][2] * inv1, acc[d][3] * inv1);
    }
    if (a.lse != nullptr && t == 0) {
        float *lse = a.lse + (size_t(z) * a.H + h) * n_q;
        if (ok0) lse[row0 + r0] = m0 * c2 + log2f(l0);
        if (ok1) lse[row0 + r1] = m1 * c2 + log2f(l1);
    }
}

template <typename T, int D, int BM>
cudaError_t launch_mma_inst(const AttnArgs &a, cudaStream_t stream) {
    using SM = MmaSmem<D, BM>;
    constexpr size_t smem = SM::BYTES;
    static DeviceOnce configured;                          // the attribute is per device
    const cudaError_t ce = configured.run([&] {
        return cudaFuncSetAttribute(attn_mma_kernel<T, D, BM>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    });
    if (ce != cudaSuccess) return ce;
    dim3 grid(a.nb, a.H, a.Z), block(BM * 2);
    attn_mma_kernel<T, D, BM><<<grid, block, smem, stream>>>(a);
    return cudaGetLastError();
}

template <typename T, int D>
cudaError_t launch_mma_d(const AttnArgs &a, int variant, cudaStream_t stream) {
    (void)variant;
    switch (a.bm) {
        case 16: return launch_mma_inst<T, D, 16>(a, stream);
        case 32: return launch_mma_inst<T, D, 32>(a, stream);
        case 64: return launch_mma_inst<T, D, 64>(a, stream);
        case 128: return launch_mma_inst<T, D, 128>(a, stream);
    }
    return cudaErrorNotSupported;
}

}  // namespace fst
