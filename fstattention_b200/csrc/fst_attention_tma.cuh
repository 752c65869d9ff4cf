// Tree attention, TMA variant: the same mathematics and tile structure as attn_mma_kernel
// (fst_attention_mma.cuh; reference fstattention.py:21-151), with the contiguous operands moved
// by the tensor memory accelerator instead of the load/store unit.
//
// Why: with 16-byte cp.async copies and 4-byte Q accesses the LSU data pipe is the busiest
// unit of the SM (about 3000 wavefronts per 64-row block, 58 % busy at 3 CTAs/SM, a third of
// them Q fragment loads) and sits on the critical path of the prologue.  Here
//   * Q and the block's own K and V rows are 32-row x 64-column boxes fetched with
//     cp.async.bulk.tensor (one thread issues them; rows past the end of the tensor arrive as
//     zeros) and complete on mbarriers;
//   * every tile lives in shared memory in the 128-byte-swizzled layout TMA writes (16-byte
//     chunk c of row r sits at chunk c ^ (r & 7)), which makes ldmatrix conflict free without
//     padding; the gathered ancestor rows are placed into the same layout by cp.async;
//   * Q is read with ldmatrix; its buffer doubles as the second gathered stage and, at the end,
//     as the staging tile from which O leaves through a TMA store.
//
// Every mbarrier wait is bounded in time: when it runs out the kernel records FST_DEV_TIMEOUT in
// the status record and carries on to its exit instead of spinning.

#pragma once

#include <cuda.h>

#include <atomic>
#include <memory>
#include <new>
#include <type_traits>

#include "fst_attention_mma.cuh"

namespace fst {

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}\n" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}
// Wait for a phase, but never longer than ~50 ms: on giving up the status record gets
// FST_DEV_TIMEOUT and the caller carries on to its exit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int32_t *status, int where) {
    if (mbar_test(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
#pragma unroll 1
    for (int it = 0; it < (1 << 24); ++it) {
        if (mbar_test(bar, parity)) return true;
        if ((it & 15) == 15 && global_ns() - t0 > 50000000ull) break;
    }
    report(status, FST_DEV_TIMEOUT, where, int(parity));
    return false;
}
// one box of a rank-4 tensor (columns, rows, head, batch) into shared memory
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2,
                                            int c3, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%2, %3, %4, %5}], [%6];\n"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar) : "memory");
}

// ask for one box of a rank-4 tensor to be brought into L2 (nothing is returned to the SM)
__device__ __forceinline__ void tma_prefetch_4d(const CUtensorMap *map, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];\n"
                 ::"l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

// one box from shared memory back to a rank-4 tensor; rows past the end of the tensor are dropped
__device__ __forceinline__ void tma_store_4d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];\n"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

// A tile is 32 rows; with D = 128 it is two 4 KB halves (columns 0-63, 64-127), each 32 rows of
// 128 bytes in the swizzled layout.
template <int D>
struct SwzTile {
    static constexpr int HALVES = D / 64;
    static constexpr int BYTES = 32 * D * 2;
    // byte offset of 16-byte chunk `c` (0 .. D/8-1) of row `r` (0..31)
    __device__ static __forceinline__ uint32_t off(int r, int c) {
        return uint32_t((c >> 3) * 4096 + r * 128 + (((c & 7) ^ (r & 7)) << 4));
    }
};

// Column tiles are TN = 32 or 64 K/V rows: 32 keeps three CTAs on an SM (the choice for large
// grids), 64 halves the number of softmax rounds a warp runs one after the other (the choice when
// the grid is too small to fill the machine and the latency of one CTA is what counts).
template <int D, int BM, int TN>
struct TmaSmem {
    static constexpr int TILE = SwzTile<D>::BYTES;        // one 32-row physical tile
    static constexpr int NB32 = (BM + 31) / 32;           // physical tiles per block
    static constexpr int TP = TN / 32;                    // physical tiles per column tile
    static constexpr int NBT = (BM + TN - 1) / TN;        // column tiles holding the block's own rows
    static constexpr int KB = 0;                          // the block's own K rows
    static constexpr int VB = KB + NBT * TP * TILE;
    static constexpr int ST0 = VB + NBT * TP * TILE;      // stage 0: one K column tile then one V
    static constexpr int ST1 = ST0 + 2 * TP * TILE;       // stage 1, shared with the Q tiles
    static constexpr int QO = ST1;
    static constexpr int QO_TILES = NB32 > 2 * TP ? NB32 : 2 * TP;
    static constexpr int BAR = QO + QO_TILES * TILE;      // two mbarriers
    static constexpr int BYTES = BAR + 64 + 1024;         // + slack to align the base to 1 KB
};

// Tensor maps of the output: one, or - when the call also delivers its rows to the other GPUs of
// a sharded problem - one per rank, each over that rank's copy of the full output tensor.
template <int NOUT>
struct OutMaps {
    CUtensorMap m[NOUT];
};

// PFX = false compiles the shared-prefix machinery (dense tiles, split over CTAs) out: the
// no-prefix kernel is smaller, and for a latency-bound kernel fewer instruction bytes is time.
// NOUT > 1: the attention and the all-gather of its output in one kernel.  Every CTA hands its
// staged O tile to TMA once per rank, with the coordinates of this rank's shard inside the full
// tensor (a.out_z0, a.out_h0); stores to the other GPUs' buffers travel over NVLink while other
// CTAs still compute, so the exchange overlaps the arithmetic tile by tile.
template <typename T, int D, int BM, int TN, bool PFX, int NOUT>
__global__ void __launch_bounds__(BM * 2, (BM <= 64 && TN == 32 ? 3 : (BM == 128 && D == 64 && TN == 32 ? 2 : 1)))
attn_tma_kernel(const AttnArgs a, const __grid_constant__ CUtensorMap tm_q,
                const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                const __grid_constant__ OutMaps<NOUT> tm_o) {
    using MT = MmaTraits<T>;
    using SM = TmaSmem<D, BM, TN>;
    using TL = SwzTile<D>;
    constexpr int NT = BM * 2;            // threads
    constexpr int CH = D / 8;             // 16-byte chunks per row
    constexpr int KS = D / 16;
    constexpr int ND = D / 8;
    constexpr int RPP = NT / CH;          // rows covered by one pass of all threads
    constexpr int SPT = TN / RPP;         // gathered rows per thread and tile
    constexpr int NB32 = SM::NB32;
    constexpr int TP = SM::TP;            // 32-row physical tiles (= mask words) per column tile
    constexpr int NG = TN / 16;           // 16-column groups per column tile
    constexpr int BW = (BM + 31) / 32;
    static_assert(NT % CH == 0 && TN % RPP == 0, "thread count must cover whole rows and tiles");

    extern __shared__ unsigned char smem_raw[];
    const uint32_t s_base = (smem_u32(smem_raw) + 1023u) & ~1023u;    // swizzle atoms are 1 KB
    // Grid order.  Large grids: blocks fastest, so that CTAs running together share a head's K/V rows
    // in L2.  Grids of a few waves (a.heads_first): heads fastest and the blocks from the last one
    // down - blocks late in a tree have the most ancestors, so the long items start first and the
    // last wave is made of short ones.
    // (Only the 64-column-tile instantiations, the ones small grids get, can be launched that way:
    // the 32-column ones sit at their register limit and the choice would cost them spills.)
    const bool heads_first = TN == 64 && a.heads_first;
    const int b = heads_first ? int(gridDim.y) - 1 - int(blockIdx.y) : int(blockIdx.x);
    const int h = heads_first ? int(blockIdx.x) : int(blockIdx.y);
    const int n_splits = PFX ? a.n_splits : 1;
    const int z = blockIdx.z / n_splits, split = blockIdx.z - z * n_splits;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = b * BM;
    const int prefix = PFX ? a.prefix : 0, n_q = a.n_q;
    const uint32_t bar_qk = s_base + SM::BAR, bar_v = bar_qk + 8, bar_p = bar_qk + 16;   // bar_p: one per stage
    // With the prefix split over several CTAs, split 0 also owns the tree part (block rows and
    // external ancestors); every split takes a contiguous run of prefix tiles.
    const bool tree = split == 0;
    const int pt_total = (PFX && a.skip_prefix) ? 0 : (prefix + TN - 1) / TN, pt_per = (pt_total + n_splits - 1) / n_splits;
    const int pt_lo = min(split * pt_per, pt_total), pt_hi = min(pt_lo + pt_per, pt_total);
    const int p_lo = pt_lo * TN, p_end = min(prefix, pt_hi * TN);      // my prefix rows [p_lo, p_end)
    const int nblk = tree ? SM::NBT : 0;

    // Launched with programmatic stream serialisation: this grid may be resident before the grid
    // ahead of it in the stream has finished.  Let the one behind us in, then wait for the one
    // ahead (completion and memory flush) before the first access to memory it may have written.
    // Q, K, V and O always count as such.  The packed metadata does too, unless the caller says
    // (a.meta_stable) that it was complete before the launch ahead of this one - the usual case:
    // one precompute per decode step, then one attention call per layer - and then the index
    // list, the count and the mask words are requested while the grid ahead is still draining.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    // Small grids (the 64-column instantiations): a CTA that is resident before the launch ahead of
    // it has finished asks for its Q and its block's K/V rows to be brought into L2 meanwhile.  No
    // value reaches the SM before the dependency wait below, and L2 is where the other launch's
    // writes land too, so whatever it still writes to those rows is what the loads after the wait see.
    if (TN == 64 && tid == 0) {
        const int hk0 = h / a.kv_group;
#pragma unroll
        for (int j = 0; j < NB32; ++j)
#pragma unroll
            for (int hf = 0; hf < TL::HALVES; ++hf) {
                tma_prefetch_4d(&tm_q, hf * 64, row0 + j * 32, h, z);
                if (tree) {
                    tma_prefetch_4d(&tm_k, hf * 64, prefix + row0 + j * 32, hk0, z);
                    tma_prefetch_4d(&tm_v, hf * 64, prefix + row0 + j * 32, hk0, z);
                }
            }
    }
    const bool early_meta = a.meta_stable != 0;
    if (!early_meta) asm volatile("griddepcontrol.wait;\n" ::: "memory");

    const PackedLayout L = packed_layout(a.nb, BM, a.ma);
    const int maw = L.maw;
    const unsigned char *blob = a.packed + size_t(z) * a.meta_stride;
    const int32_t *g_idx = reinterpret_cast<const int32_t *>(blob + L.off_idx) + size_t(b) * a.ma;
    const uint32_t *g_emask = reinterpret_cast<const uint32_t *>(blob + L.off_emask) + size_t(b) * BM * maw;
    const uint32_t *g_bmask = reinterpret_cast<const uint32_t *>(blob + L.off_bmask) + size_t(b) * BM * BW;
    const int count = tree ? __ldg(reinterpret_cast<const int32_t *>(blob + L.off_count) + b) : 0;

    const int hk = h / a.kv_group;                        // my K/V head
    const T *kp = static_cast<const T *>(a.k) + z * a.ks_z + hk * a.ks_h;
    const T *vp = static_cast<const T *>(a.v) + z * a.vs_z + hk * a.vs_h;
    const int lr = tid / CH, lc = tid % CH;               // my row-in-pass and 16-byte chunk
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
    // All mask words of the block's own rows are asked for here, a global-memory latency before
    // the first product needs them (a block tile that turns out empty for this warp is skipped
    // in less time than a load takes); gathered tiles fetch theirs one tile ahead.
    uint32_t wb0[BW], wb1[BW];
#pragma unroll
    for (int p = 0; p < BW; ++p) {
        wb0[p] = (tree && ok0) ? __ldg(g_bmask + r0 * BW + p) : 0u;
        wb1[p] = (tree && ok1) ? __ldg(g_bmask + r1 * BW + p) : 0u;
    }
    // With at most 64 ancestor slots (two mask words per row: the reference's MAX_ANCESTORS) the
    // 32-column-tile instantiations fetch the words of the gathered tiles here too, with everything
    // else, instead of one tile ahead inside the loop, where a loaded L2 answers later than a tile
    // takes (2 % on 64 batched trees; the 64-column instantiations lose by the extra choice).
    constexpr int PRE = TN == 32 ? 2 : 0;
    const bool pre = PRE > 0 && maw <= PRE;
    uint32_t pe0[PRE + 1], pe1[PRE + 1];
#pragma unroll
    for (int p = 0; p < PRE; ++p) {
        pe0[p] = (pre && tree && ok0 && p < maw) ? __ldg(g_emask + r0 * maw + p) : 0u;
        pe1[p] = (pre && tree && ok1 && p < maw) ? __ldg(g_emask + r1 * maw + p) : 0u;
    }
    if (tid == 0) {                                       // shared memory only: needs no wait either
        mbar_init(bar_qk, 1);
        mbar_init(bar_v, 1);
        mbar_init(bar_p, 1);
        mbar_init(bar_p + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (early_meta) asm volatile("griddepcontrol.wait;\n" ::: "memory");

    // ---- one thread starts the TMA transfers: Q and block K on one barrier, block V on another
    if (tid == 0) {
        mbar_arrive_expect_tx(bar_qk, (tree ? 2 : 1) * NB32 * SM::TILE);
#pragma unroll
        for (int j = 0; j < NB32; ++j)
#pragma unroll
            for (int hf = 0; hf < TL::HALVES; ++hf) {
                if (tree)
                    tma_load_4d(s_base + SM::KB + j * SM::TILE + hf * 4096, &tm_k, hf * 64, prefix + row0 + j * 32, hk, z, bar_qk);
                tma_load_4d(s_base + SM::QO + j * SM::TILE + hf * 4096, &tm_q, hf * 64, row0 + j * 32, h, z, bar_qk);
            }
        if (tree) {
            mbar_arrive_expect_tx(bar_v, NB32 * SM::TILE);
#pragma unroll
            for (int j = 0; j < NB32; ++j)
#pragma unroll
                for (int hf = 0; hf < TL::HALVES; ++hf)
                    tma_load_4d(s_base + SM::VB + j * SM::TILE + hf * 4096, &tm_v, hf * 64, prefix + row0 + j * 32, hk, z, bar_v);
        }
    }

    // ---- gathered tiles.  External ancestors: cp.async row by row into the swizzled layout (all
    //      threads).  Prefix tiles are dense: thread 0 fetches them as TMA boxes onto the stage's
    //      mbarrier; rows past this CTA's share of the prefix arrive too and are masked off.
    auto load_gathered = [&](int e, int st, bool ext, const int (&node)[SPT]) {
        const uint32_t kd = s_base + (st ? SM::ST1 : SM::ST0);
        const uint32_t vd = kd + TP * SM::TILE;
        if (ext) {
#pragma unroll
            for (int j = 0; j < SPT; ++j) {
                const int s = lr + j * RPP;
                const bool ok = node[j] >= 0 && node[j] < n_q;
                if (node[j] >= n_q) report(a.status, FST_DEV_INDEX_RANGE, b, e * TN + s);
                const long long rr = ok ? prefix + node[j] : 0;
                const uint32_t o = (s >> 5) * SM::TILE + TL::off(s & 31, lc);
                cp_async16(kd + o, kp + rr * a.ks_n + lc * 8, ok);
                cp_async16(vd + o, vp + rr * a.vs_n + lc * 8, ok);
            }
        } else if (tid == 0) {
            const int p0 = p_lo + (e - nt_ext_of<TN>(count, a.ma)) * TN;
            const uint32_t bar = bar_p + st * 8;
            mbar_arrive_expect_tx(bar, 2 * TP * SM::TILE);
#pragma unroll
            for (int tp = 0; tp < TP; ++tp)
#pragma unroll
                for (int hf = 0; hf < TL::HALVES; ++hf) {
                    tma_load_4d(kd + tp * SM::TILE + hf * 4096, &tm_k, hf * 64, p0 + tp * 32, hk, z, bar);
                    tma_load_4d(vd + tp * SM::TILE + hf * 4096, &tm_v, hf * 64, p0 + tp * 32, hk, z, bar);
                }
        }
    };
    // without a prefix the first gathered tile is requested before the count has arrived
    if (prefix == 0) {
        load_gathered(0, 0, true, nodeA);
        cp_async_commit();                                // group 0
    }
    const int nt_ext = nt_ext_of<TN>(count, a.ma);
    const int nt_gat = nt_ext + (pt_hi - pt_lo);
    if (prefix != 0) {
        if (nt_gat > 0) load_gathered(0, 0, nt_ext > 0, nodeA);
        cp_async_commit();                                // group 0
    }
    fetch_idx(2, nodeA);

    // ---- Q fragments; afterwards stage 1, which shares Q's memory, may be filled
    __syncthreads();                                      // barrier initialisation is visible
    bool alive = mbar_wait(bar_qk, 0, a.status, b);
    uint32_t qf[KS][4];
    {
        const int qr = warp * 16 + (lane & 15);           // row of the block this lane addresses
        const uint32_t qb = s_base + SM::QO + (qr >> 5) * SM::TILE;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) ldmatrix_x4(qf[ks], qb + TL::off(qr & 31, ks * 2 + (lane >> 4)));
    }
    // A negative scale: the running maximum below is kept in raw score units and scaled inside
    // the exponent, which orders scores correctly only for a positive factor; so the sign moves
    // into Q (the sign bit of both halves of every fragment register) and the factor is |scale|.
    if (a.scale_log2 < 0.f) {
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
#pragma unroll
            for (int i = 0; i < 4; ++i) qf[ks][i] ^= 0x80008000u;
    }
    if (nt_gat > 1) {
        __syncthreads();
        load_gathered(1, 1, nt_ext > 1, nodeB);
    }
    cp_async_commit();                                    // group 1
    fetch_idx(3, nodeB);

    float acc[ND][4];
#pragma unroll
    for (int i = 0; i < ND; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // m in raw score units; l is my share
    const float c2 = fabsf(a.scale_log2);

    const int n_tiles = nblk + nt_gat;
    // mask words of my two rows for gathered tile e (external ancestors, then prefix tiles)
    auto gathered_words = [&](int e, uint32_t (&w0)[TP], uint32_t (&w1)[TP]) {
#pragma unroll
        for (int p = 0; p < TP; ++p) {
            w0[p] = w1[p] = 0u;
            if (e < nt_ext) {
                const int wi = e * TP + p;
                if (pre) {
#pragma unroll
                    for (int q = 0; q < PRE; ++q)
                        if (q == wi) { w0[p] = pe0[q]; w1[p] = pe1[q]; }
                } else {
                    if (ok0 && wi < maw) w0[p] = __ldg(g_emask + r0 * maw + wi);
                    if (ok1 && wi < maw) w1[p] = __ldg(g_emask + r1 * maw + wi);
                }
            } else if (e < nt_gat) {
                const int rem = p_end - p_lo - (e - nt_ext) * TN - p * 32;
                w0[p] = w1[p] = rem >= 32 ? 0xffffffffu : (rem > 0 ? (1u << rem) - 1u : 0u);
            }
        }
    };
    uint32_t w0n[TP], w1n[TP];                            // words of the next gathered tile
    // With several block tiles, those in which none of my warp's 16 rows has a column are passed
    // over outright (a block tile needs no CTA-wide step, so the warps need not agree); with
    // rows numbered breadth first that is every block tile but the one on the diagonal.  With a
    // single block tile there is nothing to pass over and the bookkeeping would only cost time.
    constexpr bool SKIP = SM::NBT > 1;
    uint32_t blk_live = 0xffffffffu;
    if (SKIP) {
        gathered_words(0, w0n, w1n);
        blk_live = 0u;
#pragma unroll
        for (int q = 0; q < BW; ++q)
            if (__reduce_or_sync(0xffffffffu, wb0[q] | wb1[q]) != 0u) blk_live |= 1u << (q / TP);
    } else if (nblk == 0) {
        gathered_words(0, w0n, w1n);
    }
    bool v_here = false;                                  // the block's V rows have been waited for
    bool have_acc = false;                                // some product has been added to acc
#pragma unroll 1
    for (int i = 0; i < n_tiles; ++i) {
        const bool blk = i < nblk;
        if (SKIP && blk && !((blk_live >> i) & 1u)) continue;
        const int e = i - nblk;                           // gathered tile number
        uint32_t w0[TP], w1[TP];                          // mask words of my two rows for this column tile
#pragma unroll
        for (int p = 0; p < TP; ++p) {
            if (blk) {
                const int wi = i * TP + p;
                w0[p] = w1[p] = 0u;
#pragma unroll
                for (int q = 0; q < BW; ++q)
                    if (q == wi) { w0[p] = wb0[q]; w1[p] = wb1[q]; }
            } else {
                w0[p] = w0n[p];
                w1[p] = w1n[p];
            }
        }
        if (SKIP ? !blk : e + 1 >= 0) gathered_words(e + 1, w0n, w1n);   // (single block tile: from that tile on)
        uint32_t kbase, vbase;
        if (blk) {
            kbase = s_base + SM::KB + i * TP * SM::TILE;
            vbase = s_base + SM::VB + i * TP * SM::TILE;
        } else {
            const int st = e & 1;
            kbase = s_base + (st ? SM::ST1 : SM::ST0);
            vbase = kbase + TP * SM::TILE;
            if (e < nt_ext) {
                cp_async_wait<1>();
                __syncthreads();
            } else {                                      // k-th TMA use of this stage: parity k & 1
                alive = mbar_wait(bar_p + st * 8, ((e - nt_ext) >> 1) & 1, a.status, b) && alive;
            }
        }
        // 16-column groups any of my warp's 16 rows use
        bool act[NG];
        bool any = false;
        uint32_t all_bits = 0xffffffffu;
#pragma unroll
        for (int p = 0; p < TP; ++p) all_bits &= w0[p] & w1[p];
        const bool dense = PFX && __reduce_and_sync(0xffffffffu, all_bits) == 0xffffffffu;   // every row, every column
#pragma unroll
        for (int p = 0; p < TP; ++p) {
            const uint32_t occ = __reduce_or_sync(0xffffffffu, w0[p] | w1[p]);
            act[2 * p] = (occ & 0xffffu) != 0u;
            act[2 * p + 1] = (occ >> 16) != 0u;
            any = any || occ != 0u;
        }

        uint32_t pf[NG][4];
        if (any) {
            // ---- S = Q K^T on the occupied groups (k-steps outermost: independent accumulators)
            float s[2 * NG][4];
#pragma unroll
            for (int n = 0; n < 2 * NG; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
            const int krow = ((lane >> 4) << 3) + (lane & 7), kch = (lane >> 3) & 1;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
                for (int cg = 0; cg < NG; ++cg) {
                    if (act[cg]) {
                        uint32_t kb[4];
                        ldmatrix_x4(kb, kbase + (cg >> 1) * SM::TILE + TL::off((cg & 1) * 16 + krow, ks * 2 + kch));
                        MT::mma(s[2 * cg], qf[ks], kb[0], kb[1]);
                        MT::mma(s[2 * cg + 1], qf[ks], kb[2], kb[3]);
                    }
                }
            }
            // ---- mask, running max (raw units), probabilities
            float mx0 = -INFINITY, mx1 = -INFINITY;
            if (dense) {                                  // a full prefix tile: nothing to mask
#pragma unroll
                for (int n = 0; n < 2 * NG; ++n) {
                    mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
                    mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
                }
            } else {
#pragma unroll
                for (int n = 0; n < 2 * NG; ++n) {
                    if (act[n >> 1]) {
                        const int c = (n & 3) * 8 + 2 * t;
                        const uint32_t b0 = w0[n >> 2] >> c, b1 = w1[n >> 2] >> c;
                        s[n][0] = (b0 & 1u) ? s[n][0] : -INFINITY;
                        s[n][1] = (b0 & 2u) ? s[n][1] : -INFINITY;
                        s[n][2] = (b1 & 1u) ? s[n][2] : -INFINITY;
                        s[n][3] = (b1 & 2u) ? s[n][3] : -INFINITY;
                        mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
                        mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
                    }
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
            for (int n = 0; n < 2 * NG; ++n) {
                if (act[n >> 1]) {
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
            // (nothing to rescale before the first product: the accumulators are still zero)
            if (have_acc && __any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {
#pragma unroll
                for (int d = 0; d < ND; ++d) {
                    acc[d][0] *= al0; acc[d][1] *= al0;
                    acc[d][2] *= al1; acc[d][3] *= al1;
                }
            }
        }

        if (blk && (SKIP ? !v_here : i == 0)) {           // the block's V rows, before their first use
            alive = mbar_wait(bar_v, 0, a.status, b) && alive;
            v_here = true;
        }

        if (any) {
            have_acc = true;
            // ---- O += P V
            const int vrow = (((lane >> 3) & 1) << 3) + (lane & 7), vch = lane >> 4;
#pragma unroll
            for (int cg = 0; cg < NG; ++cg) {
                if (act[cg]) {
#pragma unroll
                    for (int dp = 0; dp < ND / 2; ++dp) {
                        uint32_t vb[4];
                        ldmatrix_x4_trans(vb, vbase + (cg >> 1) * SM::TILE + TL::off((cg & 1) * 16 + vrow, dp * 2 + vch));
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

    // ---- epilogue: normalise, stage O in the Q tiles (same swizzled layout; each warp writes its
    //      own 16 rows, bank-conflict free), then one thread hands the tiles to TMA
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = (l0 > 0.f && alive) ? 1.f / l0 : 0.f, inv1 = (l1 > 0.f && alive) ? 1.f / l1 : 0.f;
    if (PFX && (n_splits > 1 || a.skip_prefix)) {
        // partial result of this split: normalised rows in fp32 plus their log-sum-exp; the
        // combine kernel weighs the splits against each other
        const size_t prow = ((size_t(split) * a.Z + z) * a.H + h) * n_q + row0;
        if (ok0) {
            float2 *o0 = reinterpret_cast<float2 *>(a.part_o + (prow + r0) * D) + t;
#pragma unroll
            for (int d = 0; d < ND; ++d) o0[d * 4] = make_float2(acc[d][0] * inv0, acc[d][1] * inv0);
            if (t == 0) a.part_lse[prow + r0] = l0 > 0.f ? m0 * c2 + log2f(l0) : -INFINITY;
        }
        if (ok1) {
            float2 *o1 = reinterpret_cast<float2 *>(a.part_o + (prow + r1) * D) + t;
#pragma unroll
            for (int d = 0; d < ND; ++d) o1[d * 4] = make_float2(acc[d][2] * inv1, acc[d][3] * inv1);
            if (t == 0) a.part_lse[prow + r1] = l1 > 0.f ? m1 * c2 + log2f(l1) : -INFINITY;
        }
        return;
    }
    if (nt_gat > 1) __syncthreads();                      // stage 1 shares this memory
    {
        // stmatrix.x4 stores four 8x8 tiles in the accumulators' own fragment layout: rows g and
        // g + 8 of two neighbouring 8-column blocks per instruction.  Lane l gives the address of
        // row (l & 7) + 8 * ((l >> 3) & 1) of my warp's sixteen rows in column block d + (l >> 4).
        const int sr = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const uint32_t ob = s_base + SM::QO + (sr >> 5) * SM::TILE;
#pragma unroll
        for (int d = 0; d < ND; d += 2) {
            const uint32_t v0 = MT::pack(acc[d][0] * inv0, acc[d][1] * inv0);
            const uint32_t v1 = MT::pack(acc[d][2] * inv1, acc[d][3] * inv1);
            const uint32_t v2 = MT::pack(acc[d + 1][0] * inv0, acc[d + 1][1] * inv0);
            const uint32_t v3 = MT::pack(acc[d + 1][2] * inv1, acc[d + 1][3] * inv1);
            asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1,%2,%3,%4};\n"
                         ::"r"(ob + TL::off(sr & 31, d + (lane >> 4))), "r"(v0), "r"(v1), "r"(v2), "r"(v3) : "memory");
        }
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    __syncthreads();
    if (tid == 0) {
        const int n_out = NOUT == 1 ? 1 : a.n_out;
        const int oh = NOUT == 1 ? h : h + a.out_h0, oz = NOUT == 1 ? z : z + a.out_z0;
        // Every rank starts with its own copy and then walks the others in ring order from its
        // right-hand neighbour on: at any moment the ranks' stores then head for different GPUs
        // (all starting at rank 0 would have seven senders share one receiver's links).
        int p = NOUT == 1 ? 0 : a.out_rank;
#pragma unroll 1
        for (int i = 0; i < n_out; ++i) {
#pragma unroll
            for (int j = 0; j < NB32; ++j)
#pragma unroll
                for (int hf = 0; hf < TL::HALVES; ++hf)
                    tma_store_4d(&tm_o.m[p], s_base + SM::QO + j * SM::TILE + hf * 4096, hf * 64, row0 + j * 32, oh, oz);
            p = p + 1 == n_out ? 0 : p + 1;
        }
        asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
    }
    if (a.lse != nullptr && t == 0) {
        float *lse = a.lse + (size_t(z) * a.H + h) * n_q;
        if (ok0) lse[row0 + r0] = m0 * c2 + log2f(l0);
        if (ok1) lse[row0 + r1] = m1 * c2 + log2f(l1);
    }
    if (tid == 0) {
        if (NOUT == 1) asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");   // smem stays valid until read
        else asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");   // rows bound for other GPUs: until written
    }
}

// Merge the partial results of a split prefix: O = sum_s 2^(L_s - L) O_s with L the log-sum-exp of
// the L_s.  One thread per (row, four output columns).
template <typename T, int D>
__global__ void __launch_bounds__(128)
combine_splits_kernel(const AttnArgs a) {
    constexpr int CPR = D / 4;                            // threads per row
    // launched with programmatic stream serialisation: resident while the kernels that write the
    // partial results drain, running once they have finished
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    const size_t rows = size_t(a.Z) * a.H * a.n_q;
    const size_t idx = size_t(blockIdx.x) * 128 + threadIdx.x;
    const size_t row = idx / CPR;
    const int c = int(idx - row * CPR) * 4;
    if (row >= rows) return;
    // Loads go out four slots at a time so that their latencies overlap.
    constexpr int U = 4;
    float big = -INFINITY;
    for (int s0 = 0; s0 < a.part_slots; s0 += U) {
        float ls[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            ls[u] = s0 + u < a.part_slots ? a.part_lse[size_t(s0 + u) * rows + row] : -INFINITY;
#pragma unroll
        for (int u = 0; u < U; ++u) big = fmaxf(big, ls[u]);
    }
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    float wsum = 0.f;
    for (int s0 = 0; s0 < a.part_slots; s0 += U) {
        float ls[U];
        float4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const bool in = s0 + u < a.part_slots;
            ls[u] = in ? a.part_lse[size_t(s0 + u) * rows + row] : -INFINITY;
            v[u] = in ? *reinterpret_cast<const float4 *>(a.part_o + (size_t(s0 + u) * rows + row) * D + c)
                      : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (ls[u] == -INFINITY) continue;            // an empty run: its O row is not meaningful
            const float w = exp2f(ls[u] - big);
            sum.x = fmaf(w, v[u].x, sum.x); sum.y = fmaf(w, v[u].y, sum.y);
            sum.z = fmaf(w, v[u].z, sum.z); sum.w = fmaf(w, v[u].w, sum.w);
            wsum += w;
        }
    }
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
    const size_t n = row % a.n_q, zh = row / a.n_q;
    const size_t hh = zh % a.H, zz = zh / a.H;
    T *op = static_cast<T *>(a.o) + zz * a.os_z + hh * a.os_h + n * a.os_n + c;
    uint2 packed;
    packed.x = MmaTraits<T>::pack(sum.x * inv, sum.y * inv);
    packed.y = MmaTraits<T>::pack(sum.z * inv, sum.w * inv);
    *reinterpret_cast<uint2 *>(op) = packed;
    if (a.lse != nullptr && c == 0) a.lse[row] = big + log2f(wsum);
}

template <typename T, int D>
cudaError_t launch_combine_t(const AttnArgs &a, cudaStream_t stream) {
    const size_t items = size_t(a.Z) * a.H * a.n_q * (D / 4);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned((items + 127) / 128));
    cfg.blockDim = dim3(128);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, combine_splits_kernel<T, D>, a);
}

// ---------------------------------------------------------------------------------------------
// host side: tensor maps and launch
// ---------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static std::atomic<EncodeTiledFn> cached{nullptr};
    EncodeTiledFn fn = cached.load(std::memory_order_acquire);
    if (fn == nullptr) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
            cached.store(fn, std::memory_order_release);
        }
    }
    return fn;
}

// What a tensor map is made from.  Encoding one costs the driver about a microsecond, four of
// them are needed per call and a decoder calls with the same few buffers again and again, so
// each host thread keeps the maps it has built in a direct-mapped table keyed by these fields.
// A map stays valid for as long as its key describes the tensor: it holds an address and a
// shape, nothing that dies with the allocation.
struct MapKey {
    const void *base;
    int64_t stride_n, stride_h, stride_z;
    int32_t rows, H, Z, D, bf16, box_rows;
    bool operator==(const MapKey &o) const {
        return base == o.base && stride_n == o.stride_n && stride_h == o.stride_h && stride_z == o.stride_z &&
               rows == o.rows && H == o.H && Z == o.Z && D == o.D && bf16 == o.bf16 && box_rows == o.box_rows;
    }
};
struct MapSlot {
    alignas(64) CUtensorMap map;
    MapKey key;
    bool used = false;
};
constexpr int kMapSlots = 1024;

inline MapSlot *map_table() {
    thread_local std::unique_ptr<MapSlot[]> table;
    if (!table) table.reset(new (std::nothrow) MapSlot[kMapSlots]);
    return table.get();
}

// rank-4 map (columns, rows, heads, batch) with 64-column x box_rows boxes, 128-byte swizzle
inline bool make_map(CUtensorMap *map, const void *base, bool bf16, int D, int rows, int H, int Z,
                     int64_t stride_n, int64_t stride_h, int64_t stride_z, int box_rows = 32) {
    const MapKey key{base, stride_n, stride_h, stride_z, rows, H, Z, D, bf16 ? 1 : 0, box_rows};
    MapSlot *table = map_table();
    MapSlot *slot = nullptr;
    if (table != nullptr) {
        uint64_t hsh = reinterpret_cast<uintptr_t>(base) >> 4;
        hsh = (hsh ^ (hsh >> 17) ^ uint64_t(rows) * 0x9E3779B97F4A7C15ull ^ uint64_t(stride_n) * 0xC2B2AE3D27D4EB4Full ^
               uint64_t(H) << 20 ^ uint64_t(Z) << 40 ^ uint64_t(box_rows) << 7) * 0xFF51AFD7ED558CCDull;
        slot = &table[(hsh >> 40) % kMapSlots];
        if (slot->used && slot->key == key) {
            *map = slot->map;
            return true;
        }
    }
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[4] = {cuuint64_t(D), cuuint64_t(rows), cuuint64_t(H), cuuint64_t(Z)};
    const cuuint64_t strides[3] = {cuuint64_t(stride_n) * 2, cuuint64_t(stride_h) * 2, cuuint64_t(stride_z) * 2};
    const cuuint32_t box[4] = {64, cuuint32_t(box_rows), 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    if (fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
           const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (slot != nullptr) {
        slot->map = *map;
        slot->key = key;
        slot->used = true;
    }
    return true;
}

// number of SMs of the current device (cached)
inline int sm_count() {
    static std::atomic<int> cached[kMaxDevices];
    const int slot = current_device_slot();
    if (slot < 0) return 148;
    int n = cached[slot].load(std::memory_order_acquire);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, slot) != cudaSuccess || n <= 0) n = 148;
        cached[slot].store(n, std::memory_order_release);
    }
    return n;
}

template <typename T, int D, int BM, int TN, bool PFX, int NOUT>
cudaError_t launch_tma_pfx(const AttnArgs &a, cudaStream_t stream) {
    using SM = TmaSmem<D, BM, TN>;
    constexpr size_t smem = SM::BYTES;
    constexpr bool bf16 = sizeof(T) == 2 && !std::is_same<T, __half>::value;
    alignas(64) CUtensorMap tq, tk, tv;
    alignas(64) OutMaps<NOUT> to;
    if (!make_map(&tq, a.q, bf16, D, a.n_q, a.H, a.Z, a.qs_n, a.qs_h, a.qs_z) ||
        !make_map(&tk, a.k, bf16, D, a.n_kv, a.H / a.kv_group, a.Z, a.ks_n, a.ks_h, a.ks_z) ||
        !make_map(&tv, a.v, bf16, D, a.n_kv, a.H / a.kv_group, a.Z, a.vs_n, a.vs_h, a.vs_z))
        return cudaErrorNotSupported;
    if (NOUT == 1) {
        if (!make_map(&to.m[0], a.o, bf16, D, a.n_q, a.H, a.Z, a.os_n, a.os_h, a.os_z)) return cudaErrorNotSupported;
    } else {
        if (a.n_out < 1 || a.n_out > NOUT) return cudaErrorInvalidValue;
        for (int p = 0; p < NOUT; ++p)                    // unused entries repeat the last one: never dereferenced
            if (!make_map(&to.m[p], a.o_ranks[p < a.n_out ? p : a.n_out - 1], bf16, D, a.n_q, a.out_H, a.out_Z,
                          a.os_n, a.os_h, a.os_z))
                return cudaErrorNotSupported;
    }
    // A grid of at most one CTA per SM asks for more than half an SM's shared memory, so that no
    // two of its CTAs can share an SM.  Otherwise they do: a grid launched early (programmatic
    // stream serialisation) is placed while the grid ahead still holds its SMs, lands on whatever
    // slots are free, and the CTAs that end up in pairs finish a microsecond after the rest -
    // which is the whole call's latency (256-node tree, 128 CTAs: 6.52 -> 5.90 us per call).
    constexpr size_t kExclusive = 116 * 1024;
    static_assert(kExclusive >= smem || smem > 114 * 1024, "the padded size must cover the kernel's own need");
    static DeviceOnce configured;
    const cudaError_t ce = configured.run([&] {
        return cudaFuncSetAttribute(attn_tma_kernel<T, D, BM, TN, PFX, NOUT>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem > kExclusive ? smem : kExclusive));
    });
    if (ce != cudaSuccess) return ce;
    if (a.n_splits < 1 || (long long)a.Z * a.n_splits > 65535) return cudaErrorInvalidValue;
    // Grid order (see the kernel): a grid of more than one but at most eight CTAs per SM runs a few
    // waves, and how the last one ends decides its time: heads fastest, the long blocks first
    // (1024-node random trees, 512 CTAs: 27.0 -> 24.4 us per call; seeds 1, 5, 9: -8, -16, -7 %).
    // Larger grids keep blocks fastest (64 batched trees and the deep tree lose 3 % the other way).
    const long long ctas = (long long)a.nb * a.H * a.Z * a.n_splits;
    AttnArgs a2 = a;
    a2.heads_first = (TN == 64 && ctas > sm_count() && ctas <= 8LL * sm_count() && a.nb > 1) ? 1 : 0;
    dim3 grid(a.nb, a.H, a.Z * a.n_splits), block(BM * 2);
    if (a2.heads_first) grid = dim3(a.H, a.nb, a.Z * a.n_splits);
    const size_t launch_smem = (ctas <= sm_count() && !a.skip_prefix && smem < kExclusive) ? kExclusive : smem;
    // Programmatic stream serialisation: the grid may become resident while the kernel ahead of
    // it in the stream drains (it waits for that kernel before touching global memory).  Worth
    // about 2 % on back-to-back layers.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = launch_smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.skip_prefix ? 0 : 1;                 // beside the prefix kernel an early, waiting grid would hold the SMs it needs
    return cudaLaunchKernelEx(&cfg, attn_tma_kernel<T, D, BM, TN, PFX, NOUT>, a2, tq, tk, tv, to);
}

template <typename T, int D, int BM, int TN>
cudaError_t launch_tma_inst(const AttnArgs &a, cudaStream_t stream) {
    if (a.n_out > 0) {                                    // attention + delivery to every rank; no shared prefix there
        if (a.prefix > 0 || a.skip_prefix || a.n_splits != 1) return cudaErrorNotSupported;
        return launch_tma_pfx<T, D, BM, TN, false, kMaxRanks>(a, stream);
    }
    // the prefix instantiation also writes partial results (skip_prefix), with or without prefix rows
    return (a.prefix > 0 || a.skip_prefix) ? launch_tma_pfx<T, D, BM, TN, true, 1>(a, stream)
                                           : launch_tma_pfx<T, D, BM, TN, false, 1>(a, stream);
}

// tile_cols: 32, 64, or 0 = by grid size: 64-column tiles up to about eight CTAs per SM (measured:
// 128 and 512 CTAs are faster with 64, 4096 CTAs equal, 8192 CTAs 20 % faster with 32)
template <typename T, int D>
cudaError_t launch_tma_d(const AttnArgs &a, int tile_cols, cudaStream_t stream) {
    if (tile_cols == 0) {
        const long long ctas = (long long)a.nb * a.H * a.Z * a.n_splits;
        tile_cols = ctas <= 8LL * sm_count() ? 64 : 32;
    }
    if (tile_cols == 64) {
        switch (a.bm) {
            case 32: return launch_tma_inst<T, D, 32, 64>(a, stream);
            case 64: return launch_tma_inst<T, D, 64, 64>(a, stream);
            case 128: return launch_tma_inst<T, D, 128, 64>(a, stream);
        }
    } else {
        switch (a.bm) {
            case 32: return launch_tma_inst<T, D, 32, 32>(a, stream);
            case 64: return launch_tma_inst<T, D, 64, 32>(a, stream);
            case 128: return launch_tma_inst<T, D, 128, 32>(a, stream);
        }
    }
    return cudaErrorNotSupported;
}

}  // namespace fst
