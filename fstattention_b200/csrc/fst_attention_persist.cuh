// Tree attention for large grids: a persistent, warp-specialised variant of attn_tma_kernel
// (the same arithmetic; reference fstattention.py:21-151, the work of one program is :62-110).
//
// Why: with one CTA per (block, head, tree) every CTA pays its own start-up serially with its
// arithmetic - index list, then addresses, then a DRAM round trip before the first product -
// and while it computes it has no loads in flight.  With thousands of such CTAs the memory
// system idles half the time although the kernel is memory bound.  Here a CTA stays on its SM
// and walks a list of (block, head, tree) items:
//   * one PRODUCER warp runs ahead of the arithmetic.  It streams every item's operands, as
//     32-row tiles in the order the arithmetic needs them (Q tiles; per 32 block rows a K tile and
//     a V tile; per 32 gathered ancestors a K tile and a V tile), into a ring of shared-memory
//     tiles: contiguous rows as cp.async.bulk.tensor boxes through local tensor maps, gathered
//     ancestor rows as 16-byte cp.async copies whose completion is tied to the tile's mbarrier
//     (cp.async.mbarrier.arrive.noinc).  A ring slot is refilled as soon as every consumer warp
//     has released it, so the next item's rows are on their way while this item is computed.
//   * BM / 16 CONSUMER warps (16 query rows each) wait for a tile's "full" barrier, use it
//     (ldmatrix, mma.sync, online softmax in base 2 as in attn_tma_kernel), and release it on
//     its "empty" barrier.  O is staged in shared memory and leaves by a TMA store that
//     overlaps the next item.
// Two such CTAs share an SM for 64-row blocks (one for 128-row blocks), so that two warps per
// scheduler interleave their dependent instruction chains.
//
// No shared prefix here (a call with a prefix keeps the other kernels).  Every mbarrier wait is
// bounded in time; a warp whose wait ran out records FST_DEV_TIMEOUT and goes on through the
// item list without waiting, computing or copying, so that the barriers the other warps meet it
// at are still reached and the kernel ends.

#pragma once

#include "fst_attention_tma.cuh"

namespace fst {

template <int D, int BM>
struct PersistCfg {
    static constexpr int TILE = SwzTile<D>::BYTES;        // one 32-row tile
    static constexpr int NB32 = BM / 32;                  // 32-row tiles per block
    static constexpr int CW = BM / 16;                    // consumer warps
    static constexpr int THREADS = (CW + 1) * 32;
    static constexpr int CTAS = BM <= 64 ? 2 : 1;         // per SM
    static constexpr int R = (CTAS == 2 ? 88 : 176) * 1024 / TILE;   // ring slots
    static constexpr int RING = 0;
    static constexpr int OST = RING + R * TILE;           // O staging: the block's rows, swizzled like Q
    static constexpr int BAR = OST + NB32 * TILE;         // full[R], empty[R]
    static constexpr int BYTES = BAR + 2 * R * 8 + 1024;  // + slack to align the base to 1 KB
    static_assert(BM == 64 || BM == 128, "64- or 128-row blocks");
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
// arrive once every cp.async this thread has issued so far has landed (counts against the
// barrier's expected arrivals)
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
}

template <typename T, int D, int BM>
__global__ void __launch_bounds__(PersistCfg<D, BM>::THREADS, PersistCfg<D, BM>::CTAS)
attn_persist_kernel(const AttnArgs a, const __grid_constant__ CUtensorMap tm_q,
                    const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                    const __grid_constant__ CUtensorMap tm_o, const int n_items) {
    using MT = MmaTraits<T>;
    using CF = PersistCfg<D, BM>;
    using TL = SwzTile<D>;
    constexpr int R = CF::R, CW = CF::CW, NB32 = CF::NB32;
    constexpr int CH = D / 8;             // 16-byte chunks per row
    constexpr int KS = D / 16;
    constexpr int ND = D / 8;
    constexpr int BW = BM / 32;           // mask words per row over the block's own rows
    constexpr int RPP = 32 / CH;          // rows one pass of the producer warp covers
    constexpr int PASSES = 32 / RPP;

    extern __shared__ unsigned char smem_raw[];
    const uint32_t s_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t full0 = s_base + CF::BAR, empty0 = full0 + R * 8;
    auto slot_addr = [&](uint32_t t) { return s_base + CF::RING + (t % R) * CF::TILE; };
    auto full_bar = [&](uint32_t t) { return full0 + (t % R) * 8; };
    auto empty_bar = [&](uint32_t t) { return empty0 + (t % R) * 8; };

    if (tid == 0) {
        for (int i = 0; i < R; ++i) {
            mbar_init(full0 + i * 8, 32);                 // every producer lane arrives once per fill
            mbar_init(empty0 + i * 8, CW);                // one arrival per consumer warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    __syncthreads();

    const PackedLayout L = packed_layout(a.nb, BM, a.ma);
    const int maw = L.maw, n_q = a.n_q, nb = a.nb, H = a.H;
    const int step = gridDim.x;

    if (warp == CW) {
        // =============================== producer ===============================
        bool alive = true;
        uint32_t t = 0;                                   // tiles issued so far
        // wait until slot t % R is free again (the first R fills find it free: parity trick)
        auto acquire = [&](uint32_t tt) {
            if (alive) alive = __all_sync(0xffffffffu, mbar_wait(empty_bar(tt), ((tt / R) & 1u) ^ 1u, a.status, int(tt)));
        };
        auto tma_tile = [&](uint32_t tt, const CUtensorMap *map, int row, int head, int z) {
            acquire(tt);
            if (!alive) return;
            if (lane == 0) {
                mbar_arrive_expect_tx(full_bar(tt), CF::TILE);
#pragma unroll
                for (int hf = 0; hf < TL::HALVES; ++hf)
                    tma_load_4d(slot_addr(tt) + hf * 4096, map, hf * 64, row, head, z, full_bar(tt));
            } else {
                mbar_arrive(full_bar(tt));
            }
        };
        const int prow = lane / CH, pch = lane % CH;      // my row within a pass and my 16-byte chunk
        auto gather_tile = [&](uint32_t tt, const T *base, int64_t stride_n, int node) {
            acquire(tt);
            if (!alive) return;
            const uint32_t dst = slot_addr(tt);
#pragma unroll
            for (int p = 0; p < PASSES; ++p) {
                const int r = p * RPP + prow;
                const int nd = __shfl_sync(0xffffffffu, node, r);
                const bool ok = nd >= 0;
                cp_async16(dst + TL::off(r, pch), base + (long long)(ok ? nd : 0) * stride_n + pch * 8, ok);
            }
            cp_async_arrive_noinc(full_bar(tt));
        };
        int item = blockIdx.x;
        int count = 0;
        if (item < n_items) {
            const int b = item % nb, z = item / (nb * H);
            count = __ldg(reinterpret_cast<const int32_t *>(a.packed + size_t(z) * a.meta_stride + L.off_count) + b);
        }
#pragma unroll 1
        for (; item < n_items; item += step) {
            const int b = item % nb, zh = item / nb, h = zh % H, z = zh / H;
            const int hk = h / a.kv_group, row0 = b * BM;
            const unsigned char *blob = a.packed + size_t(z) * a.meta_stride;
            const int32_t *g_idx = reinterpret_cast<const int32_t *>(blob + L.off_idx) + size_t(b) * a.ma;
            const int nt_ext = nt_ext_of<32>(count, a.ma);
            // my slot of the first two gathered tiles, asked for before the contiguous tiles go out
            int node0 = (nt_ext > 0 && lane < a.ma) ? __ldg(g_idx + lane) : -1;
            int node1 = (nt_ext > 1 && 32 + lane < a.ma) ? __ldg(g_idx + 32 + lane) : -1;
            // the next item's count, a global-memory latency ahead of its use
            int count_next = 0;
            if (item + step < n_items) {
                const int b2 = (item + step) % nb, z2 = (item + step) / (nb * H);
                count_next = __ldg(reinterpret_cast<const int32_t *>(a.packed + size_t(z2) * a.meta_stride + L.off_count) + b2);
            }
#pragma unroll
            for (int j = 0; j < NB32; ++j) tma_tile(t++, &tm_q, row0 + j * 32, h, z);
#pragma unroll
            for (int j = 0; j < NB32; ++j) {
                tma_tile(t++, &tm_k, row0 + j * 32, hk, z);
                tma_tile(t++, &tm_v, row0 + j * 32, hk, z);
            }
            const T *kp = static_cast<const T *>(a.k) + z * a.ks_z + hk * a.ks_h;
            const T *vp = static_cast<const T *>(a.v) + z * a.vs_z + hk * a.vs_h;
#pragma unroll 1
            for (int e = 0; e < nt_ext; ++e) {
                int node = e == 0 ? node0 : (e == 1 ? node1 : ((e * 32 + lane < a.ma) ? __ldg(g_idx + e * 32 + lane) : -1));
                if (node >= n_q) {
                    report(a.status, FST_DEV_INDEX_RANGE, b, e * 32 + lane);
                    node = -1;
                }
                gather_tile(t++, kp, a.ks_n, node);
                gather_tile(t++, vp, a.vs_n, node);
            }
            count = count_next;
        }
        asm volatile("cp.async.wait_all;\n" ::: "memory");
    } else {
        // =============================== consumers ===============================
        const int g = lane >> 2, tq = lane & 3;
        const int r0 = warp * 16 + g, r1 = r0 + 8;        // my two rows inside the block
        const bool neg = a.scale_log2 < 0.f;
        const float c2 = fabsf(a.scale_log2);
        bool alive = true;
        uint32_t t = 0;                                   // tiles consumed so far
        auto wait_full = [&](uint32_t tt) {
            if (alive) alive = __all_sync(0xffffffffu, mbar_wait(full_bar(tt), (tt / R) & 1u, a.status, int(tt)));
        };
        auto release = [&](uint32_t tt) {
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(tt));
        };
        // metadata of one item, fetched an item ahead: count, the mask words of my two rows over
        // the block's own rows, and over the first gathered tile
        struct ItemMeta {
            int count;
            uint32_t wb0[BW], wb1[BW], e0, e1;
        };
        auto fetch_meta = [&](int item, ItemMeta &m) {
            const int b = item % nb, z = item / (nb * H);
            const unsigned char *blob = a.packed + size_t(z) * a.meta_stride;
            const uint32_t *g_emask = reinterpret_cast<const uint32_t *>(blob + L.off_emask) + size_t(b) * BM * maw;
            const uint32_t *g_bmask = reinterpret_cast<const uint32_t *>(blob + L.off_bmask) + size_t(b) * BM * BW;
            const bool ok0 = b * BM + r0 < n_q, ok1 = b * BM + r1 < n_q;
            m.count = __ldg(reinterpret_cast<const int32_t *>(blob + L.off_count) + b);
#pragma unroll
            for (int p = 0; p < BW; ++p) {
                m.wb0[p] = ok0 ? __ldg(g_bmask + r0 * BW + p) : 0u;
                m.wb1[p] = ok1 ? __ldg(g_bmask + r1 * BW + p) : 0u;
            }
            m.e0 = ok0 ? __ldg(g_emask + r0 * maw) : 0u;
            m.e1 = ok1 ? __ldg(g_emask + r1 * maw) : 0u;
        };
        ItemMeta cur, nxt;
        int item = blockIdx.x;
        if (item < n_items) fetch_meta(item, cur);
        bool stored = false;                              // a TMA store of mine may still be reading the staging tiles
#pragma unroll 1
        for (; item < n_items; item += step) {
            const int b = item % nb, zh = item / nb, h = zh % H, z = zh / H;
            const int row0 = b * BM;
            const bool ok0 = row0 + r0 < n_q, ok1 = row0 + r1 < n_q;
            const unsigned char *blob = a.packed + size_t(z) * a.meta_stride;
            const uint32_t *g_emask = reinterpret_cast<const uint32_t *>(blob + L.off_emask) + size_t(b) * BM * maw;
            if (item + step < n_items) fetch_meta(item + step, nxt);
            const int nt_ext = nt_ext_of<32>(cur.count, a.ma);

            // ---- Q fragments, then the Q tiles go back to the producer
            uint32_t qf[KS][4];
#pragma unroll
            for (int j = 0; j < NB32; ++j) wait_full(t + j);
            if (alive) {
                const int qr = warp * 16 + (lane & 15);
                const uint32_t qb = slot_addr(t + (qr >> 5));
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) ldmatrix_x4(qf[ks], qb + TL::off(qr & 31, ks * 2 + (lane >> 4)));
                if (neg) {
#pragma unroll
                    for (int ks = 0; ks < KS; ++ks)
#pragma unroll
                        for (int i = 0; i < 4; ++i) qf[ks][i] ^= 0x80008000u;
                }
            }
#pragma unroll
            for (int j = 0; j < NB32; ++j) release(t + j);
            t += NB32;

            float acc[ND][4];
#pragma unroll
            for (int i = 0; i < ND; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
            float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

            uint32_t en0 = cur.e0, en1 = cur.e1;          // mask words of the next gathered tile
            const int n_tiles = NB32 + nt_ext;
#pragma unroll 1
            for (int i = 0; i < n_tiles; ++i, t += 2) {
                const bool blk = i < NB32;
                uint32_t w0 = 0u, w1 = 0u;
                if (blk) {
#pragma unroll
                    for (int q = 0; q < BW; ++q)
                        if (q == i) { w0 = cur.wb0[q]; w1 = cur.wb1[q]; }
                } else {
                    w0 = en0;
                    w1 = en1;
                    const int e1i = i - NB32 + 1;         // fetch the words of the tile after this one
                    en0 = en1 = 0u;
                    if (e1i < nt_ext && e1i < maw) {
                        if (ok0) en0 = __ldg(g_emask + r0 * maw + e1i);
                        if (ok1) en1 = __ldg(g_emask + r1 * maw + e1i);
                    }
                }
                const uint32_t occ = __reduce_or_sync(0xffffffffu, w0 | w1);
                const bool act0 = (occ & 0xffffu) != 0u, act1 = (occ >> 16) != 0u;
                const bool any = (occ != 0u) && alive;

                wait_full(t);                             // K tile (waited for even when skipped: see release)
                uint32_t pf[2][4];
                if (any && alive) {
                    const uint32_t kbase = slot_addr(t);
                    float s[4][4];
#pragma unroll
                    for (int n = 0; n < 4; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
                    const int krow = ((lane >> 4) << 3) + (lane & 7), kch = (lane >> 3) & 1;
#pragma unroll
                    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
                        for (int cg = 0; cg < 2; ++cg) {
                            if (cg == 0 ? act0 : act1) {
                                uint32_t kb[4];
                                ldmatrix_x4(kb, kbase + TL::off(cg * 16 + krow, ks * 2 + kch));
                                MT::mma(s[2 * cg], qf[ks], kb[0], kb[1]);
                                MT::mma(s[2 * cg + 1], qf[ks], kb[2], kb[3]);
                            }
                        }
                    }
                    release(t);
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
                } else {
                    release(t);
                }

                wait_full(t + 1);                         // V tile
                if (any && alive) {
                    const uint32_t vbase = slot_addr(t + 1);
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
                release(t + 1);
            }

            // ---- epilogue: normalise, stage O (swizzled like the Q tiles), hand it to TMA
            l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
            l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
            l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
            l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
            const float inv0 = (l0 > 0.f && alive) ? 1.f / l0 : 0.f, inv1 = (l1 > 0.f && alive) ? 1.f / l1 : 0.f;
            // the previous item's store must have read the staging tiles before they are rewritten
            if (tid == 0 && stored) asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
            asm volatile("bar.sync 1, %0;\n" ::"n"(CW * 32) : "memory");
            {
                const uint32_t ob0 = s_base + CF::OST + (r0 >> 5) * CF::TILE + tq * 4;
                const uint32_t ob1 = s_base + CF::OST + (r1 >> 5) * CF::TILE + tq * 4;
#pragma unroll
                for (int d = 0; d < ND; ++d) {
                    const uint32_t v0 = MT::pack(acc[d][0] * inv0, acc[d][1] * inv0);
                    const uint32_t v1 = MT::pack(acc[d][2] * inv1, acc[d][3] * inv1);
                    asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(ob0 + TL::off(r0 & 31, d)), "r"(v0) : "memory");
                    asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(ob1 + TL::off(r1 & 31, d)), "r"(v1) : "memory");
                }
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            asm volatile("bar.sync 1, %0;\n" ::"n"(CW * 32) : "memory");
            if (tid == 0) {
#pragma unroll
                for (int j = 0; j < NB32; ++j)
#pragma unroll
                    for (int hf = 0; hf < TL::HALVES; ++hf)
                        tma_store_4d(&tm_o, s_base + CF::OST + j * CF::TILE + hf * 4096, hf * 64, row0 + j * 32, h, z);
                asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
                stored = true;
            }
            if (a.lse != nullptr && tq == 0) {
                float *lse = a.lse + (size_t(z) * H + h) * n_q;
                if (ok0) lse[row0 + r0] = m0 * c2 + log2f(l0);
                if (ok1) lse[row0 + r1] = m1 * c2 + log2f(l1);
            }
            cur = nxt;
        }
        if (tid == 0 && stored) asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();                                      // nobody leaves while copies into this CTA's memory may be under way
}

template <typename T, int D, int BM>
cudaError_t launch_persist_inst(const AttnArgs &a, cudaStream_t stream) {
    using CF = PersistCfg<D, BM>;
    constexpr size_t smem = CF::BYTES;
    constexpr bool bf16 = sizeof(T) == 2 && !std::is_same<T, __half>::value;
    if (a.prefix != 0 || a.n_splits != 1 || a.skip_prefix) return cudaErrorNotSupported;
    alignas(64) CUtensorMap tq, tk, tv, to;
    if (!make_map(&tq, a.q, bf16, D, a.n_q, a.H, a.Z, a.qs_n, a.qs_h, a.qs_z) ||
        !make_map(&tk, a.k, bf16, D, a.n_kv, a.H / a.kv_group, a.Z, a.ks_n, a.ks_h, a.ks_z) ||
        !make_map(&tv, a.v, bf16, D, a.n_kv, a.H / a.kv_group, a.Z, a.vs_n, a.vs_h, a.vs_z) ||
        !make_map(&to, a.o, bf16, D, a.n_q, a.H, a.Z, a.os_n, a.os_h, a.os_z))
        return cudaErrorNotSupported;
    static DeviceOnce configured;
    const cudaError_t ce = configured.run([&] {
        return cudaFuncSetAttribute(attn_persist_kernel<T, D, BM>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    });
    if (ce != cudaSuccess) return ce;
    const long long items = (long long)a.nb * a.H * a.Z;
    if (items > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    const long long slots = (long long)sm_count() * CF::CTAS;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(items < slots ? items : slots));
    cfg.blockDim = dim3(CF::THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, attn_persist_kernel<T, D, BM>, a, tq, tk, tv, to, int(items));
}

template <typename T, int D>
cudaError_t launch_persist_d(const AttnArgs &a, cudaStream_t stream) {
    switch (a.bm) {
        case 64: return launch_persist_inst<T, D, 64>(a, stream);
        case 128: return launch_persist_inst<T, D, 128>(a, stream);
    }
    return cudaErrorNotSupported;
}

// Whether the automatic choice should take this kernel.  Measured on B200 (D 128, 64-row
// blocks, fp16): 64 batched 256-node trees 171 us against 113 us for attn_tma_kernel, the deep
// 4096-node tree 105 against 85 us - it loses.  The tree kernel is bound by how many warps with
// dependent instruction chains an SM can interleave, and that is bound by registers: twelve
// compute warps of 168 registers fill the register file, and this design spends two of its ten
// warps per SM (and a third of the shared memory a third CTA would need) on staging.  So it is
// never picked automatically; FST_KERNEL_PERSIST selects it by hand.
inline bool persist_pays(const AttnArgs &) { return false; }

}  // namespace fst
