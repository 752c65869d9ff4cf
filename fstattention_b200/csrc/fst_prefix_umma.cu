// Dense attention over the shared prefix on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// The prefix part of the reference kernel (fstattention.py:113-136) is plain dense attention:
// every query row attends to every prefix row.  That is the one place on this path where the
// tiles are large and dense, so it gets its own kernel: one CTA per (128 query rows, head,
// batch element, run of prefix rows).  Per 128-row K/V tile t
//     S(t) = Q K(t)^T       tcgen05.mma  M=128 N=128 K=16 x D/16, both operands K-major in shared memory
//     P(t) = softmax part   one thread per query row (TMEM lane = row, so no shuffles): tcgen05.ld
//                           of S, probabilities against a lazily moved reference point, P written
//                           to shared memory in the 128-byte-swizzled K-major layout
//     O_g += P(t) V(t)      tcgen05.mma  A = P, B = V (MN-major: rows of V are the K index)
// Tensor memory holds two S buffers and two accumulators O_0, O_1 (4 x 128 columns).  K/V tiles
// arrive by TMA (128-row x 64-column boxes, 128-byte swizzle) into two stages each.  Head
// dimension D is 64 or 128: one or two 64-column halves per Q / K / V tile.
//
// Ten warps.  Warps 0-3 and 4-7 are two softmax groups; group g takes the tiles with t & 1 == g
// and keeps its own reference point, row sums, P buffer and accumulator O_g, so the groups never
// wait for one another and one group's barrier waits and tensor-memory latencies hide behind the
// other's exponentials.  Warp 8 loads K and its lane 0 issues S(t); warp 9 loads V and its lane 0
// issues O_g += P V.  All hand-offs are mbarriers (TMA completion, tcgen05.commit, or arrivals by
// the 128 threads of a group); every barrier indexed by t & 1 completes once per two tiles, so a
// waiter can never fall two phases behind.  At the end the groups' results are merged through
// shared memory and written as one partial result per run (normalised rows in fp32 plus base-2
// log-sum-exp) in the layout the tree kernel writes; combine_splits_kernel merges the runs.
//
// PAGED = true reads the prefix rows from a page pool through a block table (a KV cache): a
// tile is 128 / page_size pages and lane j of the loading warp requests page j.
//
// Every wait is bounded in time (mbar_wait): on expiry the kernel records FST_DEV_TIMEOUT, stops
// issuing, frees its tensor memory and returns.

#include "fst_attention_tma.cuh"

namespace fst {

namespace umma {

constexpr int QM = 128;                // query rows per CTA (MMA M)
constexpr int KN = 128;                // K/V rows per tile (MMA N of the first product)
constexpr int HALF = QM * 128;         // bytes of one 64-column half of a 128-row tile
constexpr int TILE_P = 2 * HALF;       // bytes of a P tile (128 x 128 fp16)

// Shared-memory map for head dimension D (64 or 128): a Q / K / V tile is 128 rows of D columns,
// D / 64 halves.  Q | P x 2 (double buffered) | K x 2 stages | V x 2 stages | barriers.
template <int D>
struct Geo {
    static constexpr int TILE = (D / 64) * HALF;
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_P = OFF_Q + TILE;
    static constexpr int OFF_K = OFF_P + 2 * TILE_P;
    static constexpr int OFF_V = OFF_K + 2 * TILE;
    static constexpr int OFF_BAR = OFF_V + 2 * TILE;
    static constexpr int SMEM_BYTES = OFF_BAR + 128 + 1024;   // + barriers, TMEM address, 1 KB alignment slack
};

// shared-memory matrix descriptor: 128-byte swizzle, 8-row groups 1 KB apart
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= uint64_t((addr >> 4) & 0x3fff);                 // start address
    d |= uint64_t((lbo_bytes >> 4) & 0x3fff) << 16;      // leading byte offset
    d |= uint64_t((1024 >> 4) & 0x3fff) << 32;           // stride byte offset
    d |= uint64_t(1) << 46;                              // descriptor version (Blackwell)
    d |= uint64_t(2) << 61;                              // SWIZZLE_128B
    return d;
}

// instruction descriptor: f32 accumulate, M=128, N=n, A K-major, B K- or MN-major
__device__ __forceinline__ uint32_t instr_desc(bool bf16, bool b_mn_major, int n) {
    const uint32_t fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (uint32_t(b_mn_major) << 16) |
           (uint32_t(n >> 3) << 17) | (uint32_t(QM >> 4) << 24);
}

__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        bool accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(uint32_t(accumulate)) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
// asynchronous: the registers are valid after tmem_ld_wait()
__device__ __forceinline__ void tmem_ld32(uint32_t (&r)[32], uint32_t taddr) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32"
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15,"
                 " %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
// The loaded registers pass through the wait as read-write operands, so that no use of them can
// be scheduled ahead of it.
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;\n"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                   "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                   "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0],"
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16,"
                 " %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

}  // namespace umma

// Arguments of the prefix kernel beyond AttnArgs: where this launch's partial results start.
struct PrefixArgs {
    int n_runs;          // runs of prefix rows (CTAs per query tile, head, batch element)
    int first_slot;      // partial-result slot of run 0 (slot 0 belongs to the tree kernel)
    // paged prefix: K/V rows live in pages of page_size rows; block_table[z][i] is the page
    // holding rows [i * page_size, (i + 1) * page_size) of batch element z, prefix_lens[z] its
    // number of prefix rows (AttnArgs::prefix is then the largest of them)
    const int32_t *block_table;
    const int32_t *prefix_lens;
    int table_stride, page_size, n_pages;
};

constexpr int PFX_SOFTMAX = 256;       // eight softmax warps: two groups of 128, one thread per query row each
constexpr int PFX_THREADS = PFX_SOFTMAX + 64;   // + two issuing warps

template <typename T, int D, bool PAGED>
__global__ void __launch_bounds__(PFX_THREADS, 1)
prefix_umma_kernel(const AttnArgs a, const PrefixArgs pa, const __grid_constant__ CUtensorMap tm_q,
                   const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
    using namespace umma;
    using MT = MmaTraits<T>;
    using G = Geo<D>;
    constexpr bool BF16 = !std::is_same<T, __half>::value;
    constexpr int DH = D / 64;                            // 64-column halves of a Q / K / V tile
    constexpr int TILE = G::TILE, OFF_Q = G::OFF_Q, OFF_P = G::OFF_P, OFF_K = G::OFF_K, OFF_V = G::OFF_V,
                  OFF_BAR = G::OFF_BAR;

    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");   // the merge kernel may take its place
    extern __shared__ unsigned char smem_raw[];
    const uint32_t s_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char *smem = smem_raw + (s_base - smem_u32(smem_raw));
    const int qt = blockIdx.x, h = blockIdx.y, hk = h / a.kv_group;   // query tile, head, K/V head
    const int z = blockIdx.z / pa.n_runs, run = blockIdx.z - z * pa.n_runs;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int n_q = a.n_q;
    // prefix rows of my batch element (paged: every batch element has its own count)
    const int prefix = PAGED ? min(__ldg(pa.prefix_lens + z), a.prefix) : a.prefix;

    // my run of prefix rows, in whole tiles; the runs are cut from the largest prefix
    const int tiles_total = (a.prefix + KN - 1) / KN, per = (tiles_total + pa.n_runs - 1) / pa.n_runs;
    const int t_lo = min(run * per, tiles_total), t_hi = min(t_lo + per, tiles_total);
    const int p_lo = t_lo * KN, p_end = min(prefix, t_hi * KN);
    const int nt = p_end > p_lo ? (p_end - p_lo + KN - 1) / KN : 0;

    // barriers: Q, K[2], V[2] (TMA), S[2] (S product landed in its buffer), O[2] (O += P V done, per P buffer),
    // P[2] (all softmax threads are through with S(t) and have written P(t)).  Every barrier that is
    // indexed by t & 1 completes once per two tiles, so a waiter can never fall two phases behind.
    const uint32_t bar_q = s_base + OFF_BAR, bar_k = bar_q + 8, bar_v = bar_q + 24, bar_s = bar_q + 40,
                   bar_o = bar_q + 56, bar_p = bar_q + 72;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + OFF_BAR + 112);

    // Loads are issued by whole warps (8: K, 9: V).  Contiguous prefix: lane 0 requests the two
    // boxes of a tile.  Paged: a tile is KN / page_size pages, one pair of boxes each, and lane j
    // takes page j - it reads that page's number from the block table (my_page) a tile before
    // it requests the boxes, so the table's latency is off the path, and a single thread is
    // not left to issue sixteen copies one after the other.  Pages past the end of my batch
    // element's prefix repeat its last page: finite values under columns the softmax masks.
    const int lane = tid & 31;
    const int ps = PAGED ? pa.page_size : KN, npt = KN / ps;
    const int32_t *table = PAGED ? pa.block_table + size_t(z) * pa.table_stride : nullptr;
    const int last_page = PAGED ? max(prefix - 1, 0) / ps : 0;
    auto my_page = [&](int t) -> int {
        if (!PAGED || lane >= npt) return 0;
        return __ldg(table + min((p_lo + t * KN) / ps + lane, last_page));
    };
    auto warp_load = [&](uint32_t dst, const CUtensorMap *map, uint32_t bar, int t, int page) {
        if (lane == 0) mbar_arrive_expect_tx(bar, TILE);
        if (PAGED) __syncwarp();                          // (contiguous: only lane 0 ever comes here)
        if (PAGED) {
            if (lane < npt) {
                if (unsigned(page) >= unsigned(pa.n_pages))       // the boxes then read as zeros
                    report(a.status, FST_DEV_INDEX_RANGE, z, (p_lo + t * KN) / ps + lane);
#pragma unroll
                for (int hf = 0; hf < DH; ++hf)
                    tma_load_4d(dst + lane * ps * 128 + hf * HALF, map, hf * 64, 0, hk, page, bar);
            }
        } else if (lane == 0) {
#pragma unroll
            for (int hf = 0; hf < DH; ++hf) tma_load_4d(dst + hf * HALF, map, hf * 64, p_lo + t * KN, hk, z, bar);
        }
    };
    auto load_k = [&](int t, int page) { warp_load(s_base + OFF_K + (t & 1) * TILE, &tm_k, bar_k + (t & 1) * 8, t, page); };
    auto load_v = [&](int t, int page) { warp_load(s_base + OFF_V + (t & 1) * TILE, &tm_v, bar_v + (t & 1) * 8, t, page); };
    // Warp 8 sets the barriers up and sends the first loads off before the CTA-wide sync, so that
    // they are under way while warp 9 allocates tensor memory.
    if (warp == 8) {
        if (lane == 0) {
            mbar_init(bar_q, 1);
            for (int i = 0; i < 2; ++i) {
                mbar_init(bar_k + i * 8, 1);
                mbar_init(bar_v + i * 8, 1);
                mbar_init(bar_s + i * 8, 1);
                mbar_init(bar_o + i * 8, 1);
                mbar_init(bar_p + i * 8, PFX_SOFTMAX / 2);
            }
            asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        }
        __syncwarp();
        if (nt > 0 && (PAGED || lane == 0)) {
            if (lane == 0) {
                mbar_arrive_expect_tx(bar_q, TILE);
#pragma unroll
                for (int hf = 0; hf < DH; ++hf)
                    tma_load_4d(s_base + OFF_Q + hf * HALF, &tm_q, hf * 64, qt * QM, h, z, bar_q);
            }
            const int page0 = my_page(0), page1 = nt > 1 ? my_page(1) : 0;
            load_k(0, page0);
            load_v(0, page0);
            if (nt > 1) {
                load_k(1, page1);
                load_v(1, page1);
            }
        }
    }
    if (warp == 9) {                                      // tensor memory: two S buffers and two accumulators, 128 columns each
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s0 = tmem_base, tmem_o = tmem_base + 256;   // S(t) at tmem_s0 + (t & 1) * 128, O_g at tmem_o + g * 128

    if (warp >= 8) {
        // ====== two issuing warps: 8 loads K and issues S = Q K^T, 9 loads V and issues O += P V ======
        // Lane 0 waits and issues the products; the whole warp takes part in the loads.
        const uint32_t idesc_s = instr_desc(BF16, false, KN), idesc_pv = instr_desc(BF16, true, D);
        bool alive = true;
        if (warp == 8 && nt > 0 && (PAGED || lane == 0)) {     // contiguous: lane 0 alone
            // descriptors of the tiles' first 16-wide step; a step further on adds its byte offset / 16
            const uint64_t dq = smem_desc(s_base + OFF_Q, 16), dk = smem_desc(s_base + OFF_K, 16);
            int page = nt > 2 ? my_page(2) : 0;           // my page of the tile to be requested next
            if (lane == 0) alive = mbar_wait(bar_q, 0, a.status, qt) && alive;
#pragma unroll 1
            for (int t = 0; t < nt; ++t) {                // S(t) = Q K(t)^T into S buffer t & 1
                const int st = t & 1;
                if (lane == 0 && alive) {
                    // the buffer is free when the softmax warps are through with tile t-2
                    if (t > 1) alive = mbar_wait(bar_p + st * 8, ((t >> 1) - 1) & 1, a.status, qt) && alive;
                    alive = mbar_wait(bar_k + st * 8, (t >> 1) & 1, a.status, qt) && alive;
                    if (alive) {
                        umma::fence_after_sync();
                        const uint64_t dks = dk + uint64_t(st * (TILE >> 4));
#pragma unroll
                        for (int ks = 0; ks < D / 16; ++ks) {
                            const uint64_t koff = ((ks >> 2) * HALF + (ks & 3) * 32) >> 4;
                            mma_f16(tmem_s0 + st * 128, dq + koff, dks + koff, idesc_s, ks > 0);
                        }
                        mma_commit(bar_s + st * 8);
                        // K stage st is free as soon as S(t) has been formed
                        if (t + 2 < nt) alive = mbar_wait(bar_s + st * 8, (t >> 1) & 1, a.status, qt) && alive;
                    }
                }
                if (PAGED) alive = __shfl_sync(0xffffffffu, alive, 0);
                if (!alive) break;
                if (t + 2 < nt) {
                    load_k(t + 2, page);
                    if (t + 3 < nt) page = my_page(t + 3);
                }
            }
        } else if (warp == 9 && nt > 0 && (PAGED || lane == 0)) {
            const uint64_t dp = smem_desc(s_base + OFF_P, 16), dv = smem_desc(s_base + OFF_V, HALF);
            int page = nt > 2 ? my_page(2) : 0;
#pragma unroll 1
            for (int t = 0; t < nt; ++t) {                // O_g += P(t) V(t), g = t & 1
                const int st = t & 1;
                if (lane == 0 && alive) {
                    alive = mbar_wait(bar_p + st * 8, (t >> 1) & 1, a.status, qt) && alive;   // P(t) is in shared memory
                    alive = mbar_wait(bar_v + st * 8, (t >> 1) & 1, a.status, qt) && alive;
                    if (alive) {
                        umma::fence_after_sync();
                        const uint64_t dps = dp + uint64_t(st * (TILE_P >> 4)), dvs = dv + uint64_t(st * (TILE >> 4));
#pragma unroll
                        for (int ks = 0; ks < KN / 16; ++ks) {    // 16 prefix rows per step
                            const uint64_t aoff = ((ks >> 2) * HALF + (ks & 3) * 32) >> 4;
                            mma_f16(tmem_o + st * 128, dps + aoff, dvs + uint64_t((ks * 16 * 128) >> 4), idesc_pv,
                                    t > 1 || ks > 0);
                        }
                        mma_commit(bar_o + st * 8);
                        // V stage st is free once that product has read it
                        if (t + 2 < nt) alive = mbar_wait(bar_o + st * 8, (t >> 1) & 1, a.status, qt) && alive;
                    }
                }
                if (PAGED) alive = __shfl_sync(0xffffffffu, alive, 0);
                if (!alive) break;
                if (t + 2 < nt) {
                    load_v(t + 2, page);
                    if (t + 3 < nt) page = my_page(t + 3);
                }
            }
        }
    } else {
        // ============ softmax: two groups of 128 threads, one thread per query row, alternating tiles ============
        // Group g owns the tiles with t & 1 == g: S buffer g, P buffer g and the accumulator O_g,
        // with its own reference point and row sum, so the groups never wait for one another and
        // one group's waits and tensor-memory latencies hide behind the other's exponentials.
        const int r = tid & 127, g = tid >> 7;            // my query row (TMEM lane r) and group
        const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
        const uint32_t tmem_s = tmem_s0 + g * 128, tmem_og = tmem_o + g * 128;
        unsigned char *prow = smem + OFF_P + g * TILE_P + r * 128; // my row of P buffer g
        const float c2 = a.scale_log2;
        float m_ref = -INFINITY, l = 0.f;                 // reference point of the exponent, row sum
        bool alive = true;
        float mx = -INFINITY, l_tile = 0.f, mu = 0.f;     // results / parameter of a sweep

        // One sweep over my row of S: row maximum, and (WRITE) probabilities against the reference
        // point into my row of P plus their sum.  MASK: columns >= cols are -inf.  S is read 32
        // columns at a time, the next load in flight while the current one is processed.
        auto sweep = [&](auto write_c, auto mask_c, int cols) {
            constexpr bool WRITE = decltype(write_c)::value, MASK = decltype(mask_c)::value;
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY}, l4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t ra[32], rb[32];
            tmem_ld32(ra, tmem_s + lane_base);
            tmem_ld_wait(ra);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t (&cur)[32] = (c & 1) ? rb : ra;
                uint32_t (&nxt)[32] = (c & 1) ? ra : rb;
                if (c < 3) tmem_ld32(nxt, tmem_s + lane_base + (c + 1) * 32);
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float s0 = __uint_as_float(cur[i]), s1 = __uint_as_float(cur[i + 1]);
                    if (MASK) {
                        if (c * 32 + i >= cols) s0 = -INFINITY;
                        if (c * 32 + i + 1 >= cols) s1 = -INFINITY;
                    }
                    mx4[(i >> 1) & 3] = fmaxf(mx4[(i >> 1) & 3], fmaxf(s0, s1));   // four independent chains
                    if (WRITE) {
                        const float p0 = fast_exp2(fmaf(s0, c2, -mu)), p1 = fast_exp2(fmaf(s1, c2, -mu));
                        l4[(i >> 1) & 3] += p0 + p1;
                        packed[i >> 1] = MT::pack(p0, p1);
                    }
                }
                if (WRITE) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {      // four 16-byte chunks of my row, swizzled
                        const int chunk = c * 4 + q4;
                        *reinterpret_cast<uint4 *>(prow + (chunk >> 3) * HALF + (((chunk & 7) ^ (r & 7)) << 4)) =
                            make_uint4(packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
                    }
                }
                if (c < 3) tmem_ld_wait(nxt);
            }
            mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            l_tile = (l4[0] + l4[1]) + (l4[2] + l4[3]);
        };
        const std::true_type yes{};
        const std::false_type no{};

        int n_mine = 0;                                   // tiles my group has taken
#pragma unroll 1
        for (int t = g; t < nt; t += 2, ++n_mine) {
            alive = mbar_wait(bar_s + g * 8, n_mine & 1, a.status, qt) && alive;
            // P buffer g and O_g belong to the tensor core until O_g += P V of my previous tile is done
            if (n_mine > 0) alive = mbar_wait(bar_o + g * 8, (n_mine - 1) & 1, a.status, qt) && alive;
            umma::fence_after_sync();
            const int cols = min(KN, p_end - (p_lo + t * KN));       // valid columns of this tile
            const bool full = cols == KN;

            // Probabilities are formed against the current reference point while the row maximum
            // is tracked (one pass over S).  Only if a row of my warp has outgrown its reference
            // by more than 2^8 (always on the first tile) is the reference moved, O_g rescaled,
            // and the tile done again.
            if (n_mine == 0) {
                // first tile: the maximum of the first 32 columns is reference enough to start
                // with (should a later column outgrow it by 2^8 the tile is redone below)
                uint32_t f[32];
                tmem_ld32(f, tmem_s + lane_base);
                tmem_ld_wait(f);
                mx = -INFINITY;
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (i < cols) mx = fmaxf(mx, __uint_as_float(f[i]));
            }
#pragma unroll 1
            for (int pass = 0; pass < 2; ++pass) {
                if (pass == 1 || n_mine == 0) {
                    const bool up = (mx - m_ref) * c2 > 8.f;          // true from -inf
                    if (n_mine > 0) {                     // rescale my row of O_g in tensor memory
                        const float alpha = up ? fast_exp2((m_ref - mx) * c2) : 1.f;
#pragma unroll 1
                        for (int c0 = 0; c0 < D; c0 += 32) {
                            uint32_t o[32];
                            tmem_ld32(o, tmem_og + lane_base + c0);
                            tmem_ld_wait(o);
#pragma unroll
                            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                            tmem_st32(tmem_og + lane_base + c0, o);
                        }
                        l *= alpha;
                    }
                    if (up) m_ref = mx;
                    mu = m_ref == -INFINITY ? 0.f : m_ref * c2;
                }
                if (full) sweep(yes, no, cols);
                else sweep(yes, yes, cols);
                if (!__any_sync(0xffffffffu, (mx - m_ref) * c2 > 8.f)) break;
            }
            l += l_tile;
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // P visible to the tensor core
            umma::fence_before_sync();
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar_p + g * 8) : "memory");
        }

        // ---- epilogue: merge the two groups' results; O / l and the log-sum-exp of every row go to
        // this run's partial-result slot.  Each thread puts its unnormalised row of O_g into shared
        // memory (the K and V stages, free once every product is done; the (exponent, sum) pairs
        // go to the P buffers); then each warp merges and writes whole rows, 512 contiguous bytes
        // per store instruction.
        if (n_mine > 0) alive = mbar_wait(bar_o + g * 8, (n_mine - 1) & 1, a.status, qt) && alive;
        umma::fence_after_sync();
        asm volatile("bar.sync 1, 256;\n" ::: "memory");  // every product of either group is done
        float2 *stats = reinterpret_cast<float2 *>(smem + OFF_P);            // [2][128]
        float *stage = reinterpret_cast<float *>(smem + OFF_K);              // [2][128][128], 16-byte chunks swizzled
        const float my_mu = (n_mine > 0 && alive && m_ref != -INFINITY) ? m_ref * c2 : -INFINITY;
        stats[g * 128 + r] = make_float2(my_mu, l);
        {
            float *srow = stage + (g * 128 + r) * D;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t o[32];
                if (n_mine > 0) {
                    tmem_ld32(o, tmem_og + lane_base + c0);
                    tmem_ld_wait(o);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = 0u;
                }
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    const int chunk = (c0 + i) >> 2;
                    *reinterpret_cast<uint4 *>(srow + ((chunk ^ (r & 7)) << 2)) = make_uint4(o[i], o[i + 1], o[i + 2], o[i + 3]);
                }
            }
        }
        asm volatile("bar.sync 1, 256;\n" ::: "memory");
        const size_t slot = size_t(pa.first_slot + run);
        constexpr int RPW = QM / (PFX_SOFTMAX / 32);      // 16 rows per warp: rows warp * 16 ..
        // lanes 0..15 work out the two groups' weights for one row each; they are handed round by shuffle
        float f0 = 0.f, f1 = 0.f;
        {
            const int rr = warp * RPW + (lane & (RPW - 1));
            const float2 s0 = stats[rr], s1 = stats[128 + rr];
            const float mu_all = fmaxf(s0.x, s1.x);
            const float w0 = s0.x == -INFINITY ? 0.f : fast_exp2(s0.x - mu_all);
            const float w1 = s1.x == -INFINITY ? 0.f : fast_exp2(s1.x - mu_all);
            const float l_all = s0.y * w0 + s1.y * w1;
            const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
            f0 = w0 * inv;
            f1 = w1 * inv;
            const int grow = qt * QM + rr;
            if (lane < RPW && grow < n_q)
                a.part_lse[((slot * a.Z + z) * a.H + h) * n_q + grow] = l_all > 0.f ? mu_all + log2f(l_all) : -INFINITY;
        }
#pragma unroll 4
        for (int i = 0; i < RPW; ++i) {
            const int rr = warp * RPW + i, grow = qt * QM + rr;
            const float g0 = __shfl_sync(0xffffffffu, f0, i), g1 = __shfl_sync(0xffffffffu, f1, i);
            if (lane >= D / 4) continue;                  // a row is D / 4 chunks of four floats
            const int sw = (lane ^ (rr & 7)) << 2;
            const float4 v0 = *reinterpret_cast<const float4 *>(stage + rr * D + sw);
            const float4 v1 = *reinterpret_cast<const float4 *>(stage + (128 + rr) * D + sw);
            if (grow < n_q) {
                const size_t prow_g = ((slot * a.Z + z) * a.H + h) * n_q + grow;
                reinterpret_cast<float4 *>(a.part_o + prow_g * D)[lane] =
                    make_float4(v0.x * g0 + v1.x * g1, v0.y * g0 + v1.y * g1, v0.z * g0 + v1.z * g1, v0.w * g0 + v1.w * g1);
            }
        }
    }

    umma::fence_before_sync();
    __syncthreads();
    if (warp == 9)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512) : "memory");
}

// rank-4 map with 64-column x 128-row boxes (kept in the calling thread's table of maps)
static bool make_map_rows128(CUtensorMap *map, const void *base, bool bf16, int D, int rows, int H, int Z,
                             int64_t stride_n, int64_t stride_h, int64_t stride_z) {
    return make_map(map, base, bf16, D, rows, H, Z, stride_n, stride_h, stride_z, 128);
}

// rank-4 map over a page pool (columns, rows of a page, K/V heads, pages) with 64-column x page boxes
static bool make_map_pool(CUtensorMap *map, bool bf16, int D, const PagedArgs &pg, int H_kv, const void *pool) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[4] = {cuuint64_t(D), cuuint64_t(pg.page_size), cuuint64_t(H_kv), cuuint64_t(pg.n_pages)};
    const cuuint64_t strides[3] = {cuuint64_t(pg.stride_row) * 2, cuuint64_t(pg.stride_head) * 2,
                                   cuuint64_t(pg.stride_page) * 2};
    const cuuint32_t box[4] = {64, cuuint32_t(pg.page_size), 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
              const_cast<void *>(pool), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename T, int D, bool PAGED>
static cudaError_t launch_prefix_t(const AttnArgs &a, const PagedArgs *pg, int n_runs, int first_slot,
                                   cudaStream_t stream) {
    constexpr bool bf16 = !std::is_same<T, __half>::value;
    alignas(64) CUtensorMap tq, tk, tv;
    if (!make_map_rows128(&tq, a.q, bf16, D, a.n_q, a.H, a.Z, a.qs_n, a.qs_h, a.qs_z)) return cudaErrorNotSupported;
    if (PAGED) {
        if (!make_map_pool(&tk, bf16, D, *pg, a.H / a.kv_group, pg->k_pool) ||
            !make_map_pool(&tv, bf16, D, *pg, a.H / a.kv_group, pg->v_pool))
            return cudaErrorNotSupported;
    } else if (!make_map_rows128(&tk, a.k, bf16, D, a.n_kv, a.H / a.kv_group, a.Z, a.ks_n, a.ks_h, a.ks_z) ||
               !make_map_rows128(&tv, a.v, bf16, D, a.n_kv, a.H / a.kv_group, a.Z, a.vs_n, a.vs_h, a.vs_z)) {
        return cudaErrorNotSupported;
    }
    static DeviceOnce configured;
    const cudaError_t ce = configured.run([&] {
        return cudaFuncSetAttribute(prefix_umma_kernel<T, D, PAGED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    umma::Geo<D>::SMEM_BYTES);
    });
    if (ce != cudaSuccess) return ce;
    if ((long long)a.Z * n_runs > 65535) return cudaErrorInvalidValue;
    PrefixArgs pa{n_runs, first_slot, nullptr, nullptr, 0, 0, 0};
    if (PAGED) {
        pa.block_table = pg->block_table;
        pa.prefix_lens = pg->prefix_lens;
        pa.table_stride = pg->table_stride;
        pa.page_size = pg->page_size;
        pa.n_pages = pg->n_pages;
    }
    dim3 grid((a.n_q + umma::QM - 1) / umma::QM, a.H, a.Z * n_runs);
    prefix_umma_kernel<T, D, PAGED><<<grid, PFX_THREADS, umma::Geo<D>::SMEM_BYTES, stream>>>(a, pa, tq, tk, tv);
    return cudaGetLastError();
}

template <bool PAGED>
static cudaError_t launch_prefix_any(const AttnArgs &a, const PagedArgs *pg, int dtype, int n_runs, int first_slot,
                                     cudaStream_t stream) {
    if ((a.D != 64 && a.D != 128) || a.prefix <= 0 || n_runs < 1) return cudaErrorNotSupported;
    if (dtype == FST_F16)
        return a.D == 128 ? launch_prefix_t<__half, 128, PAGED>(a, pg, n_runs, first_slot, stream)
                          : launch_prefix_t<__half, 64, PAGED>(a, pg, n_runs, first_slot, stream);
    if (dtype == FST_BF16)
        return a.D == 128 ? launch_prefix_t<__nv_bfloat16, 128, PAGED>(a, pg, n_runs, first_slot, stream)
                          : launch_prefix_t<__nv_bfloat16, 64, PAGED>(a, pg, n_runs, first_slot, stream);
    return cudaErrorNotSupported;
}

// Partial results of the prefix, split into n_runs runs, into slots first_slot .. first_slot+n_runs-1.
cudaError_t launch_prefix_umma(const AttnArgs &a, int dtype, int n_runs, int first_slot, cudaStream_t stream) {
    return launch_prefix_any<false>(a, nullptr, dtype, n_runs, first_slot, stream);
}

// The same with the prefix rows in a page pool; a.k / a.v are not read.
cudaError_t launch_prefix_umma_paged(const AttnArgs &a, const PagedArgs &pg, int dtype, int n_runs, int first_slot,
                                     cudaStream_t stream) {
    if (pg.page_size != 16 && pg.page_size != 32 && pg.page_size != 64 && pg.page_size != 128)
        return cudaErrorNotSupported;
    return launch_prefix_any<true>(a, &pg, dtype, n_runs, first_slot, stream);
}

}  // namespace fst
