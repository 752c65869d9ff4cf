// Tree attention for large grids: attn_tma_kernel's arithmetic (reference fstattention.py:21-151)
// in a CTA small enough that four of them share an SM.
//
// Why: with thousands of (block, head, tree) items the tree kernel is not bound by memory or by
// the tensor pipe but by how many warps, each a long chain of dependent instructions, an SM can
// interleave; a persistent producer/consumer variant with its operands always ready in shared
// memory took exactly as long per item and warp.  attn_tma_kernel holds 168 registers per thread
// and 66 KB of shared memory, i.e. three CTAs (twelve warps) per SM.  This kernel fits four:
//   * Q is not kept in 32 registers per thread: its fragments are re-read from the Q tiles by
//     ldmatrix for every column tile (the tiles stay until they are rewritten as the O staging
//     area), which brings the kernel to 128 registers;
//   * the block's own K/V rows are not held for the whole item either: like the gathered
//     ancestors they pass, one 32-row K tile and V tile at a time, through two stages of
//     16 KB, so a CTA needs 48 KB (head_dim 128) instead of 66 KB.
// Contiguous rows arrive as cp.async.bulk.tensor boxes on per-stage mbarriers, gathered rows by
// 16-byte cp.async copies, everything in the 128-byte-swizzled layout; O leaves by a TMA store.
// No shared prefix, no split (those calls keep attn_tma_kernel).  Every mbarrier wait is bounded.

#pragma once

#include "fst_attention_tma.cuh"

namespace fst {

template <int D, int BM>
struct LeanSmem {
    static constexpr int TILE = SwzTile<D>::BYTES;        // one 32-row tile
    static constexpr int NB32 = BM / 32;
    static constexpr int QO = 0;                          // Q tiles, later the O staging tiles
    static constexpr int ST0 = QO + NB32 * TILE;          // stage 0: K tile, V tile
    static constexpr int ST1 = ST0 + 2 * TILE;
    static constexpr int BAR = ST1 + 2 * TILE;            // bar_q, bar_s[2]
    static constexpr int BYTES = BAR + 32 + 1024;         // + slack to align the base to 1 KB
    static constexpr int CTAS = 512 / (BM * 2);           // sixteen warps per SM
    static_assert(BM == 64 || BM == 128, "64- or 128-row blocks");
};

template <typename T, int D, int BM>
__global__ void __launch_bounds__(BM * 2, LeanSmem<D, BM>::CTAS)
attn_lean_kernel(const AttnArgs a, const __grid_constant__ CUtensorMap tm_q,
                 const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                 const __grid_constant__ CUtensorMap tm_o) {
    using MT = MmaTraits<T>;
    using SM = LeanSmem<D, BM>;
    using TL = SwzTile<D>;
    constexpr int NT = BM * 2;
    constexpr int CH = D / 8;
    constexpr int KS = D / 16;
    constexpr int ND = D / 8;
    constexpr int RPP = NT / CH;          // rows covered by one pass of all threads
    constexpr int SPT = 32 / RPP;         // gathered rows per thread and tile
    constexpr int NB32 = SM::NB32;
    constexpr int BW = BM / 32;
    static_assert(NT % CH == 0 && 32 % RPP == 0, "thread count must cover whole rows and tiles");

    extern __shared__ unsigned char smem_raw[];
    const uint32_t s_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int b = blockIdx.x, h = blockIdx.y, z = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const int row0 = b * BM, n_q = a.n_q;
    const uint32_t bar_q = s_base + SM::BAR, bar_s = bar_q + 8;      // bar_s + 8 * stage

    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const bool early_meta = a.meta_stable != 0;
    if (!early_meta) asm volatile("griddepcontrol.wait;\n" ::: "memory");

    const PackedLayout L = packed_layout(a.nb, BM, a.ma);
    const int maw = L.maw;
    const unsigned char *blob = a.packed + size_t(z) * a.meta_stride;
    const int32_t *g_idx = reinterpret_cast<const int32_t *>(blob + L.off_idx) + size_t(b) * a.ma;
    const uint32_t *g_emask = reinterpret_cast<const uint32_t *>(blob + L.off_emask) + size_t(b) * BM * maw;
    const uint32_t *g_bmask = reinterpret_cast<const uint32_t *>(blob + L.off_bmask) + size_t(b) * BM * BW;
    const int count = __ldg(reinterpret_cast<const int32_t *>(blob + L.off_count) + b);

    const int hk = h / a.kv_group;
    const T *kp = static_cast<const T *>(a.k) + z * a.ks_z + hk * a.ks_h;
    const T *vp = static_cast<const T *>(a.v) + z * a.vs_z + hk * a.vs_h;
    const int lr = tid / CH, lc = tid % CH;
    const int r0 = warp * 16 + g, r1 = r0 + 8;
    const bool ok0 = row0 + r0 < n_q, ok1 = row0 + r1 < n_q;

    int node[SPT];                                        // my slots of the next gathered tile
    auto fetch_idx = [&](int e) {
#pragma unroll
        for (int j = 0; j < SPT; ++j) {
            const int slot = e * 32 + lr + j * RPP;
            node[j] = slot < a.ma ? __ldg(g_idx + slot) : -1;
        }
    };
    fetch_idx(0);
    uint32_t wb0[BW], wb1[BW];
#pragma unroll
    for (int p = 0; p < BW; ++p) {
        wb0[p] = ok0 ? __ldg(g_bmask + r0 * BW + p) : 0u;
        wb1[p] = ok1 ? __ldg(g_bmask + r1 * BW + p) : 0u;
    }
    uint32_t en0 = ok0 ? __ldg(g_emask + r0 * maw) : 0u, en1 = ok1 ? __ldg(g_emask + r1 * maw) : 0u;
    if (tid == 0) {
        mbar_init(bar_q, 1);
        mbar_init(bar_s, 1);
        mbar_init(bar_s + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (early_meta) asm volatile("griddepcontrol.wait;\n" ::: "memory");

    // tile i of the item: the block's own rows first (NB32 tiles, TMA), then the gathered ancestors
    auto load_own = [&](int i, int st) {                  // one thread: K tile and V tile of block rows 32 i ..
        const uint32_t kd = s_base + (st ? SM::ST1 : SM::ST0), vd = kd + SM::TILE, bar = bar_s + st * 8;
        mbar_arrive_expect_tx(bar, 2 * SM::TILE);
#pragma unroll
        for (int hf = 0; hf < TL::HALVES; ++hf) {
            tma_load_4d(kd + hf * 4096, &tm_k, hf * 64, row0 + i * 32, hk, z, bar);
            tma_load_4d(vd + hf * 4096, &tm_v, hf * 64, row0 + i * 32, hk, z, bar);
        }
    };
    auto load_ext = [&](int e, int st) {                  // all threads: gathered tile e from node[]
        const uint32_t kd = s_base + (st ? SM::ST1 : SM::ST0), vd = kd + SM::TILE;
#pragma unroll
        for (int j = 0; j < SPT; ++j) {
            const int s = lr + j * RPP;
            const bool ok = node[j] >= 0 && node[j] < n_q;
            if (node[j] >= n_q) report(a.status, FST_DEV_INDEX_RANGE, b, e * 32 + s);
            const long long rr = ok ? node[j] : 0;
            const uint32_t o = TL::off(s, lc);
            cp_async16(kd + o, kp + rr * a.ks_n + lc * 8, ok);
            cp_async16(vd + o, vp + rr * a.vs_n + lc * 8, ok);
        }
    };
    if (tid == 0) {
        mbar_arrive_expect_tx(bar_q, NB32 * SM::TILE);
#pragma unroll
        for (int j = 0; j < NB32; ++j)
#pragma unroll
            for (int hf = 0; hf < TL::HALVES; ++hf)
                tma_load_4d(s_base + SM::QO + j * SM::TILE + hf * 4096, &tm_q, hf * 64, row0 + j * 32, h, z, bar_q);
        load_own(0, 0);
        load_own(1, 1);                                   // NB32 >= 2
    }
    const int nt_ext = nt_ext_of<32>(count, a.ma);
    const int n_tiles = NB32 + nt_ext;

    float acc[ND][4];
#pragma unroll
    for (int i = 0; i < ND; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const bool neg = a.scale_log2 < 0.f;
    const float c2 = fabsf(a.scale_log2);

    __syncthreads();                                      // barrier initialisation is visible
    bool alive = mbar_wait(bar_q, 0, a.status, b);
    const int qr = warp * 16 + (lane & 15);
    const uint32_t q_addr = s_base + SM::QO + (qr >> 5) * SM::TILE;

#pragma unroll 1
    for (int i = 0; i < n_tiles; ++i) {
        const bool own = i < NB32;
        const int st = i & 1;
        uint32_t w0 = 0u, w1 = 0u;
        if (own) {
#pragma unroll
            for (int q = 0; q < BW; ++q)
                if (q == i) { w0 = wb0[q]; w1 = wb1[q]; }
        } else {
            w0 = en0;
            w1 = en1;
            const int e1 = i - NB32 + 1;                  // the words of the tile after this one
            en0 = en1 = 0u;
            if (e1 < nt_ext && e1 < maw) {
                if (ok0) en0 = __ldg(g_emask + r0 * maw + e1);
                if (ok1) en1 = __ldg(g_emask + r1 * maw + e1);
            }
        }
        const uint32_t kbase = s_base + (st ? SM::ST1 : SM::ST0), vbase = kbase + SM::TILE;
        if (own) {
            alive = mbar_wait(bar_s + st * 8, uint32_t(i >> 1) & 1u, a.status, b) && alive;   // fill i / 2 of this stage
        } else {
            cp_async_wait<1>();
            __syncthreads();
        }
        const uint32_t occ = __reduce_or_sync(0xffffffffu, w0 | w1);
        const bool act0 = (occ & 0xffffu) != 0u, act1 = (occ >> 16) != 0u;
        if (occ != 0u) {
            float s[4][4];
#pragma unroll
            for (int n = 0; n < 4; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
            const int krow = ((lane >> 4) << 3) + (lane & 7), kch = (lane >> 3) & 1;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t qf[4];
                ldmatrix_x4(qf, q_addr + TL::off(qr & 31, ks * 2 + (lane >> 4)));
                if (neg) {
#pragma unroll
                    for (int x = 0; x < 4; ++x) qf[x] ^= 0x80008000u;
                }
#pragma unroll
                for (int cg = 0; cg < 2; ++cg) {
                    if (cg == 0 ? act0 : act1) {
                        uint32_t kb[4];
                        ldmatrix_x4(kb, kbase + TL::off(cg * 16 + krow, ks * 2 + kch));
                        MT::mma(s[2 * cg], qf, kb[0], kb[1]);
                        MT::mma(s[2 * cg + 1], qf, kb[2], kb[3]);
                    }
                }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                if ((n >> 1) == 0 ? act0 : act1) {
                    const int c = n * 8 + 2 * tq;
                    const uint32_t b0 = w0 >> c, b1 = w1 >> c;
                    s[n][0] = (b0 & 1u) ? s[n][0] : -INFINITY;
                    s[n][1] = (b0 & 2u) ? s[n][1] : -INFINITY;
                    s[n][2] = (b1 & 1u) ? s[n][2] : -INFINITY;
                    s[n][3] = (b1 & 2u) ? s[n][3] : -INFINITY;
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
            uint32_t pf[2][4];
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                if ((n >> 1) == 0 ? act0 : act1) {
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
            const int vrow = (((lane >> 3) & 1) << 3) + (lane & 7), vch = lane >> 4;
#pragma unroll
            for (int cg = 0; cg < 2; ++cg) {
                if (cg == 0 ? act0 : act1) {
#pragma unroll
                    for (int dp = 0; dp < ND / 2; ++dp) {
                        uint32_t vb[4];
                        ldmatrix_x4_trans(vb, vbase + TL::off(cg * 16 + vrow, dp * 2 + vch));
                        MT::mma(acc[2 * dp], pf[cg], vb[0], vb[1]);
                        MT::mma(acc[2 * dp + 1], pf[cg], vb[2], vb[3]);
                    }
                }
            }
        }
        // recycle this stage for tile i + 2
        if (i + 2 < n_tiles) {
            __syncthreads();                              // everybody has read the stage
            if (i + 2 < NB32) {
                if (tid == 0) load_own(i + 2, st);
            } else {
                load_ext(i + 2 - NB32, st);
                fetch_idx(i + 3 - NB32);
            }
        }
        cp_async_commit();                                // one group per tile, empty or not
    }

    // ---- epilogue: normalise, stage O in the Q tiles, hand them to TMA
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = (l0 > 0.f && alive) ? 1.f / l0 : 0.f, inv1 = (l1 > 0.f && alive) ? 1.f / l1 : 0.f;
    __syncthreads();                                      // every warp has read its last Q fragments
    {
        const uint32_t ob0 = s_base + SM::QO + (r0 >> 5) * SM::TILE + tq * 4;
        const uint32_t ob1 = s_base + SM::QO + (r1 >> 5) * SM::TILE + tq * 4;
#pragma unroll
        for (int d = 0; d < ND; ++d) {
            const uint32_t v0 = MT::pack(acc[d][0] * inv0, acc[d][1] * inv0);
            const uint32_t v1 = MT::pack(acc[d][2] * inv1, acc[d][3] * inv1);
            asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(ob0 + TL::off(r0 & 31, d)), "r"(v0) : "memory");
            asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(ob1 + TL::off(r1 & 31, d)), "r"(v1) : "memory");
        }
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    __syncthreads();
    if (tid == 0) {
#pragma unroll
        for (int j = 0; j < NB32; ++j)
#pragma unroll
            for (int hf = 0; hf < TL::HALVES; ++hf)
                tma_store_4d(&tm_o, s_base + SM::QO + j * SM::TILE + hf * 4096, hf * 64, row0 + j * 32, h, z);
        asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
    }
    if (a.lse != nullptr && tq == 0) {
        float *lse = a.lse + (size_t(z) * a.H + h) * n_q;
        if (ok0) lse[row0 + r0] = m0 * c2 + log2f(l0);
        if (ok1) lse[row0 + r1] = m1 * c2 + log2f(l1);
    }
    if (tid == 0) asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
}

template <typename T, int D, int BM>
cudaError_t launch_lean_inst(const AttnArgs &a, cudaStream_t stream) {
    using SM = LeanSmem<D, BM>;
    constexpr size_t smem = SM::BYTES;
    constexpr bool bf16 = sizeof(T) == 2 && !std::is_same<T, __half>::value;
    if (a.prefix != 0 || a.n_splits != 1 || a.skip_prefix || a.n_out > 0) return cudaErrorNotSupported;
    alignas(64) CUtensorMap tq, tk, tv, to;
    if (!make_map(&tq, a.q, bf16, D, a.n_q, a.H, a.Z, a.qs_n, a.qs_h, a.qs_z) ||
        !make_map(&tk, a.k, bf16, D, a.n_kv, a.H / a.kv_group, a.Z, a.ks_n, a.ks_h, a.ks_z) ||
        !make_map(&tv, a.v, bf16, D, a.n_kv, a.H / a.kv_group, a.Z, a.vs_n, a.vs_h, a.vs_z) ||
        !make_map(&to, a.o, bf16, D, a.n_q, a.H, a.Z, a.os_n, a.os_h, a.os_z))
        return cudaErrorNotSupported;
    static DeviceOnce configured;
    const cudaError_t ce = configured.run([&] {
        return cudaFuncSetAttribute(attn_lean_kernel<T, D, BM>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    });
    if (ce != cudaSuccess) return ce;
    if (a.Z > 65535) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.nb, a.H, a.Z);
    cfg.blockDim = dim3(BM * 2);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, attn_lean_kernel<T, D, BM>, a, tq, tk, tv, to);
}

template <typename T, int D>
cudaError_t launch_lean_d(const AttnArgs &a, cudaStream_t stream) {
    switch (a.bm) {
        case 64: return launch_lean_inst<T, D, 64>(a, stream);
        case 128: return launch_lean_inst<T, D, 128>(a, stream);
    }
    return cudaErrorNotSupported;
}

}  // namespace fst
