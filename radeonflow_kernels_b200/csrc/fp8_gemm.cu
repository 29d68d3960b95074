// FP8 (e4m3) block-scaled GEMM for sm_100a.
//
//   C[m,n] = bf16( sum_kb a_s[m,kb] * b_s[n/128,kb] * sum_{j<128} A[m,128kb+j] * B[n,128kb+j] )
//
// Replaces the reference's transpose + pipelined MFMA kernel + split-K reduce
// (src/gemm/gemm_launcher.cpp:43-101, src/gemm/gemm_kernel.cpp:334-562, :288-303).
//
// One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer: A [128 x 128 B] and B [BN x 128 B] tiles, 128-byte
//               swizzle, into a STAGES-deep shared-memory ring (mbarrier tx counts)
//   warps 1, 2  MMA issuers, alternating K blocks: per 128-deep K block, 4 x
//               tcgen05.mma.kind::f8f6f4 (K = 32 each) into one of 512/BN TMEM
//               accumulator buffers, then ONE tcgen05.commit that publishes the
//               buffer (the epilogue, which observes it, frees the smem stage)
//   warps 4..   epilogue: tcgen05.ld the K block's fp32 partial sums, scale by
//               the exact fp32 product a_s*b_s and add into a register
//               accumulator (packed fma.rn.f32x2) while the next K blocks' MMAs run
//               in the other TMEM buffers; finally round to bf16 (or store fp32
//               split-K slices)
//
// The scales are arbitrary fp32 numbers, so the hardware block-scaled MMA
// (ue8m0 scales) cannot be used; promotion is one FMA per element per K block,
// exactly the ratio of the reference's `frag_r += s * frag_c`
// (src/gemm/gemm_kernel.cpp:173-207).
#include "ptx.cuh"
#include "fp8_gemm.h"

#include <cstdio>
#include <cstdlib>

namespace rf {

#ifdef RF_WAIT_STATS
// Debug build only: cycles each role spent inside its barrier waits, summed over CTAs.
__device__ unsigned long long g_wait_stats[12];
#define RF_STAT_BEGIN() const long long _t0 = clock64()
#define RF_STAT_END(acc) (acc) += clock64() - _t0
#define RF_STAT_FLUSH(idx, acc) atomicAdd(&g_wait_stats[idx], (unsigned long long)(acc))
#else
#define RF_STAT_BEGIN()
#define RF_STAT_END(acc)
#define RF_STAT_FLUSH(idx, acc)
#endif

// RF_EPI_WIDE=1 selects an experimental epilogue inner loop (64 staging registers reloaded in place, the
// accumulator buffer handed back after two load latencies).  Measured on B200 it is not faster: built without
// spills it needs the K loop un-unrolled and runs 6144 x 4608 x 7168 in 191 us against 178 us for the default.
#ifndef RF_EPI_WIDE
#define RF_EPI_WIDE 0
#endif

namespace {

constexpr int BM = 128;
constexpr int BK = 128;          // one scale block, one 128-byte swizzle row of fp8
constexpr int UMMA_K = 32;       // K per tcgen05.mma for 8-bit operands
constexpr int NUM_NON_EPI_WARPS = 4;

// TWO_CTA: the tile is 256 x BN per CTA PAIR (2-CTA cluster): each CTA loads its own 128 rows of A and
// half of the B rows, the leader CTA issues cta_group::2 MMAs (M = 256) whose accumulator rows
// 0-127 / 128-255 land in the two CTAs' TMEM.  Per SM and K block this moves 32 KB through shared
// memory each way instead of 48 KB; measured, it is still slower than the 1-CTA 128 x 256 tile (the
// epilogue's promotion work, not shared memory, bounds both), so it is selectable but not the default.
// MN_MAJOR: operands stored [k][m] and [k][n] (M / N contiguous), the reference's physical layout
// (src/gemm/gemm_kernel_legacy.cpp:264-268); consumed directly as MN-major UMMA operands, so the
// reference's transpose pass (src/gemm/gemm_launcher.cpp:55-56) has no counterpart here.
// SLABS: store slabs per epilogue warp.  With two, the second 64-column chunk of a tile is staged while the
// TMA is still reading the first; worth its 32 KB of shared memory (one pipeline stage fewer) only when K is
// short and the per-tile store is a large share of the tile's time.
template <int BN, int STAGES, bool TWO_CTA = false, bool MN_MAJOR = false, int SLABS = 1>
struct GemmCfg {
    static constexpr int kBN = BN;
    static constexpr int kStages = STAGES;
    static constexpr bool kTwoCta = TWO_CTA;
    static constexpr bool kMnMajor = MN_MAJOR;
    static_assert(!(TWO_CTA && MN_MAJOR), "the CTA-pair configuration is K-major only");
    static constexpr int kBRows = TWO_CTA ? BN / 2 : BN;       // rows of B this CTA loads per K block
    static constexpr int kEpiGroups = 2;                       // column groups, 4 warps each
    static constexpr int kColsPerThread = BN / kEpiGroups;     // 64 or 128: one scale block at most
    static constexpr int kEpiWarps = 4 * kEpiGroups;
    static constexpr int kThreads = 32 * (NUM_NON_EPI_WARPS + kEpiWarps);   // 384
    static constexpr int kABytes = BM * BK;
    static constexpr int kBBytes = kBRows * BK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemBufs = 512 / BN;                // accumulator buffers in flight
    static constexpr int kTmemCols = kTmemBufs * BN;          // all 512 TMEM columns
    // full / empty / peer-full per stage, full / empty per accumulator buffer, the two stream-K barriers, the
    // TMEM address slot (16 bytes)
    static constexpr int kBarBytes = (3 * STAGES + 2 * kTmemBufs + 2) * 8 + 16;
    static constexpr int kSlabBytes = 32 * 128;               // one slab: 32 rows x 128 B, swizzled
    static constexpr int kSlabs = SLABS;                      // slabs per epilogue warp
    static_assert(SLABS == 1 || SLABS == 2, "one or two store slabs per warp");
    static constexpr int kSmemBytes =
        STAGES * kStageBytes + kEpiWarps * kSlabs * kSlabBytes + kBarBytes + 1024;       // + alignment slack
    // The epilogue (64 or 128 accumulators per thread plus staging) wants more than the 168 registers a
    // 384-thread CTA starts with, the producer warpgroup far fewer: registers are rebalanced after set-up
    // (128 * kRegsLo + 256 * kRegsHi <= 64512, the CTA's allocation at 168 per thread).  The split is chosen by
    // measurement on the 18-shape sweep.
    static constexpr bool kRebalanceRegs = true;
#if defined(RF_REGS_LO) && defined(RF_REGS_HI)
    static constexpr int kRegsLo = RF_REGS_LO, kRegsHi = RF_REGS_HI;
#elif RF_EPI_WIDE
    static constexpr int kRegsLo = kColsPerThread > 64 ? 40 : 104;
    static constexpr int kRegsHi = kColsPerThread > 64 ? 232 : 200;
#else
    // (56 / 224 for the row-major one-slab configurations, 120 / 192 for the others; 88 / 208 and 72 / 216 run the
    // sweep 17 % and 27 % slower: ptxas allocates the K loop differently at every split)
    static constexpr bool kWideSplit = !TWO_CTA && !MN_MAJOR && SLABS == 1;
    static constexpr int kRegsLo = kWideSplit ? 56 : 120, kRegsHi = kWideSplit ? 224 : 192;
#endif
    static_assert(128 * kRegsLo + 256 * kRegsHi <= 64512 && kRegsLo % 8 == 0 && kRegsHi % 8 == 0, "register split");
    static_assert(kColsPerThread == 64 || kColsPerThread == 128, "epilogue handles 64 or 128 columns per thread");
    static_assert(kTmemCols == 512, "TMEM columns: power of two, at most 512");
    static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

struct TileCoord {
    int m_blk, n_blk;
};

// Tile number -> tile.  Consecutive tiles walk down M inside a band of GROUP_M row blocks before moving to
// the next column block, so the CTAs that run concurrently share B tiles (and A bands) in L2.
__device__ __forceinline__ TileCoord decode_tile(int tile, int tiles_m, int tiles_n) {
    // (This runs once per tile in every role, on the epilogue's critical path between two tiles: one integer
    // division, and shifts for the full bands.  Measured: the earlier form with five divisions, together with two
    // 64-bit divisions for the K range, cost the epilogue about 1400 cycles per tile, the present one 600.)
    constexpr int GROUP_M = 8;
    TileCoord t;
    const int group = GROUP_M * tiles_n;
    const int band = tile / group;
    const int first_m = band * GROUP_M;
    const int band_rows = min(GROUP_M, tiles_m - first_m);
    const int in_band = tile - band * group;
    if (band_rows == GROUP_M) {
        t.m_blk = first_m + (in_band & (GROUP_M - 1));
        t.n_blk = in_band >> 3;
    } else {
        t.n_blk = in_band / band_rows;
        t.m_blk = first_m + in_band - t.n_blk * band_rows;
    }
    return t;
}

// One stretch of work of a CTA: K blocks [kb0, kb1) of work item `item` = tile * splits + K-slice number.
struct Piece {
    int item, kb0, kb1;
};

// First K-block unit of CTA j's share of the stream-K region (`total` units over `n_units` CTAs).
__host__ __device__ __forceinline__ int sk_share_begin(long long total, int j, int n_units) {
    return (int)(total * j / n_units);
}

// Contributors of the tile whose first unit is `base` and whose owner is CTA `unit`: the CTAs j < unit whose
// share overlaps [base, owner's first unit).  sk_first_contributor gives the lowest candidate; candidates with an
// empty share or one that ends at or below `base` contribute nothing.
__host__ __device__ __forceinline__ int sk_first_contributor(long long total, int unit, int n_units, int base) {
    int j = unit - 1;
    while (j > 0 && sk_share_begin(total, j, n_units) > base) --j;
    return j < 0 ? 0 : j;
}
__host__ __device__ __forceinline__ bool sk_contributes(long long total, int j, int n_units, int base) {
    const int hi = sk_share_begin(total, j + 1, n_units);
    return hi > base && hi > sk_share_begin(total, j, n_units);
}

// First tile of the stream-K region.
__host__ __device__ __forceinline__ int sk_tile0(const GemmParams& p) { return p.tiles_m * p.tiles_n - p.sk_tiles; }

// The sequence of pieces a CTA works through; producer, MMA issuers and epilogue each walk their own copy.
//
// Plain launches: work items unit, unit + n_units, ... (a work item is a tile, or one K slice of a tile; the K
// slices of one tile are adjacent).
// Stream-K launches (p.sk_tiles > 0): the LAST p.sk_tiles tiles form a region whose K blocks, numbered
// tile-major, are cut into n_units equal contiguous shares, so that no SM idles in a ragged last wave.  A CTA
// takes its share from the TOP down (so a tile that continues in the next CTA's share is started first and
// the tile it finishes for the previous CTA comes last) and then its plain tiles.  A share boundary inside a
// tile makes the lower CTA a contributor (it leaves its fp32 partial sums in its scratch slot and raises its
// flag at the very beginning of its run) and the upper CTA, which holds the tile's last K block, the owner
// (it adds the slots of the contributors, all of LOWER block index and long finished with them, and stores
// the tile).  Waiting only ever goes to lower block indices, which are scheduled no later than the waiter.
template <bool STREAM_K>
struct WorkWalker;

// Plain launches.  (One register of state: the epilogue's register budget is tight and its allocation fragile.)
template <>
struct WorkWalker<false> {
    int w;                     // the work item drawn last
    __host__ __device__ __forceinline__ WorkWalker(const GemmParams&, int unit, int n_units, int) { w = unit - n_units; }
    __host__ __device__ __forceinline__ bool next(Piece& pc, const GemmParams& p, int n_units, int kb_total) {
        w += n_units;
        if (w >= p.tiles_m * p.tiles_n * p.splits) return false;
        pc.item = w;
        if (p.splits == 1) {
            pc.kb0 = 0;
            pc.kb1 = kb_total;
        } else {
            // (k / 128 < 2^24 and splits <= 64: the products fit 32 bits)
            const int split = w % p.splits;
            pc.kb0 = kb_total * split / p.splits;
            pc.kb1 = kb_total * (split + 1) / p.splits;
        }
        return true;
    }
};

// Stream-K launches (p.splits == 1, so a work item is a tile).
template <>
struct WorkWalker<true> {
    int u_lo, u_hi;            // stream-K units of this CTA not yet done: [u_lo, u_hi), taken from the top
    int w;                     // next plain tile
    __host__ __device__ __forceinline__ WorkWalker(const GemmParams& p, int unit, int n_units, int kb_total) {
        const long long total = (long long)p.sk_tiles * kb_total;
        u_lo = sk_share_begin(total, unit, n_units);
        u_hi = sk_share_begin(total, unit + 1, n_units);
        w = unit;
    }
    __host__ __device__ __forceinline__ bool next(Piece& pc, const GemmParams& p, int n_units, int kb_total) {
        if (u_hi > u_lo) {
            const int t = (u_hi - 1) / kb_total;
            const int base = t * kb_total;
            const int lo = u_lo > base ? u_lo : base;
            pc.item = sk_tile0(p) + t;
            pc.kb0 = lo - base;
            pc.kb1 = u_hi - base;
            u_hi = lo;
            return true;
        }
        if (w < sk_tile0(p)) {
            pc.item = w;
            pc.kb0 = 0;
            pc.kb1 = kb_total;
            w += n_units;
            return true;
        }
        return false;
    }
};

// STREAM_K: the instantiation that stream-K launches (p.sk_tiles > 0) run; plain launches run the other one, which
// contains none of the stream-K code.
template <class Cfg, bool STREAM_K = false>
__global__ void __launch_bounds__(Cfg::kThreads, 1)
fp8_gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                const __grid_constant__ CUtensorMap tma_c, const __grid_constant__ CUtensorMap tma_p,
                const __grid_constant__ GemmDestMaps dests, const GemmParams p) {
    constexpr int BN = Cfg::kBN;
    constexpr int STAGES = Cfg::kStages;
    constexpr int CPT = Cfg::kColsPerThread;
    constexpr int NBUF = Cfg::kTmemBufs;

    extern __shared__ uint8_t smem_raw[];
    // 128-byte-swizzled tiles need 1024-byte alignment.
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t slab_base = smem_base + STAGES * Cfg::kStageBytes;
    const uint32_t bar_base = slab_base + Cfg::kEpiWarps * Cfg::kSlabs * Cfg::kSlabBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tmem_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
    auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + NBUF + b); };
    auto peer_full_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 2 * NBUF + s); };   // leader only
    // stream-K: "this CTA's partial sums are stored" (8 epilogue warps -> warp 3) and "the partial sums this CTA's
    // owner piece needs have arrived" (warp 3 -> epilogue warps); each is used at most once per launch
    const uint32_t sk_stored_bar = bar_base + 8u * (3 * STAGES + 2 * NBUF);
    const uint32_t sk_ready_bar = sk_stored_bar + 8u;
    const uint32_t tmem_slot = bar_base + 8u * (3 * STAGES + 2 * NBUF + 2);
    uint32_t* tmem_slot_ptr =
        reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    constexpr bool TWO = Cfg::kTwoCta;
    // The next kernel in the stream may be scheduled onto SMs as this grid's CTAs leave them; it blocks in
    // its own griddep_wait() until this grid has completed.
    griddep_launch_dependents();
#ifdef RF_SINGLE_ISSUE
    constexpr bool kDualIssue = false;
#else
    constexpr bool kDualIssue = NBUF % 2 == 0;
#endif
    const uint32_t cta_rank = TWO ? cluster_ctarank() : 0u;      // 0 = leader of the pair
    const int unit = TWO ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;          // work-loop index
    const int unit_stride = TWO ? (int)(gridDim.x >> 1) : (int)gridDim.x;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tma_a);
        tma_prefetch_desc(&tma_b);
        tma_prefetch_desc(p.splits == 1 ? &tma_c : &tma_p);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int s = 0; s < STAGES; ++s) mbar_init(peer_full_bar(s), 1);
        if (STREAM_K) {
            mbar_init(sk_stored_bar, Cfg::kEpiWarps);
            mbar_init(sk_ready_bar, 1);
        }
        for (int b = 0; b < NBUF; ++b) {
            mbar_init(tmem_full_bar(b), 1);
            // in a CTA pair the leader's barrier collects the epilogue warps of both CTAs
            mbar_init(tmem_empty_bar(b), TWO ? 2 * Cfg::kEpiWarps : Cfg::kEpiWarps);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        if (TWO) {
            tmem_alloc_2cta(tmem_slot, Cfg::kTmemCols);
            tmem_relinquish_2cta();
        } else {
            tmem_alloc(tmem_slot, Cfg::kTmemCols);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (TWO) cluster_sync_all();     // both CTAs' barriers exist before any remote arrive or multicast commit
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot_ptr);
    // Barriers, TMEM and descriptors are set up; everything below reads or writes global memory that the
    // previous kernel in the stream may still be producing.
    griddep_wait();

    const int kb_total = p.k / BK;

    if (warp < NUM_NON_EPI_WARPS) {
    // Register split after set-up: the 4 producer / MMA warps shrink to kRegsLo, the 8 epilogue warps grow
    // to kRegsHi.
    if (Cfg::kRebalanceRegs) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(Cfg::kRegsLo));
    // Producer and MMA warps keep all 32 lanes in the loops (warp-uniform control
    // flow, so descriptors and addresses live in uniform registers) and elect one
    // lane only for the instructions that must be issued once.
    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        uint32_t it = 0;  // running K-block counter across work items
        bool ok = true;
        long long w_empty = 0; (void)w_empty;
        // e4m3fnuz operands (reference-layout configurations only): an operand that holds +-240 or NaN bytes
        // is read from its converted copy (the conversion pass that ran before this kernel left the flags)
        const CUtensorMap* map_a = &tma_a;
        const CUtensorMap* map_b = &tma_b;
        if (Cfg::kMnMajor && p.fnuz_flags != nullptr) {
            if (p.fnuz_flags[0] != 0) map_a = &dests.m[0];
            if (p.fnuz_flags[1] != 0) map_b = &dests.m[1];
        }
        WorkWalker<STREAM_K> walk(p, unit, unit_stride, kb_total);
        Piece pc;
        while (ok && walk.next(pc, p, unit_stride, kb_total)) {
            const TileCoord t = decode_tile(p.splits == 1 ? pc.item : pc.item / p.splits, p.tiles_m, p.tiles_n);
            // rows of A and of B this CTA fetches (a CTA pair splits both between its two CTAs)
            const int a_row0 = TWO ? (t.m_blk * 2 + (int)cta_rank) * BM : t.m_blk * BM;
            const int b_row0 = t.n_blk * BN + (TWO ? (int)cta_rank * Cfg::kBRows : 0);
            for (int kb = pc.kb0; kb < pc.kb1; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                { RF_STAT_BEGIN();
                ok = __all_sync(0xffffffffu, mbar_wait(empty_bar(s), ph ^ 1, p.status, kErrProducerWait, p.launch_tag));
                RF_STAT_END(w_empty); }
                if (!ok) break;
                if (elect_one()) {
                    mbar_expect_tx(full_bar(s), Cfg::kStageBytes);
                    const uint32_t sa = smem_base + s * Cfg::kStageBytes;
                    if (Cfg::kMnMajor) {
                        // boxes of 128 K-rows x 128 bytes of M (or N); B needs one box per 128 columns
                        tma_load_2d(sa, map_a, full_bar(s), a_row0, kb * BK);
#pragma unroll
                        for (int j = 0; j < BN / 128; ++j)
                            tma_load_2d(sa + Cfg::kABytes + j * (BK * 128), map_b, full_bar(s), b_row0 + 128 * j,
                                        kb * BK);
                    } else {
                        tma_load_2d(sa, &tma_a, full_bar(s), kb * BK, a_row0);
                        tma_load_2d(sa + Cfg::kABytes, &tma_b, full_bar(s), kb * BK, b_row0);
                    }
                }
                __syncwarp();
            }
        }
        if (lane == 0) { RF_STAT_FLUSH(0, w_empty); }
    } else if (warp == 1 || (kDualIssue && warp == 2)) {
        // ------------------------------------------------------- MMA issuers
        // Issuing one K block (two barrier waits, four MMAs, one commit) is a serial chain of a few
        // hundred cycles in a single thread, about as long as the MMAs take to execute.  Two warps on
        // different schedulers therefore alternate K blocks: even blocks (and the even TMEM buffers)
        // belong to warp 1, odd ones to warp 2.  Blocks are independent (separate accumulator buffers
        // and smem stages), so no ordering between the two issuers is needed.
        const uint32_t my_parity = (uint32_t)(warp - 1);
        constexpr uint32_t idesc = make_idesc(TWO ? 2 * BM : BM, BN, /*e4m3*/ 0, /*e4m3*/ 0,
                                              Cfg::kMnMajor ? 1 : 0, Cfg::kMnMajor ? 1 : 0);
        // descriptor advance per MMA (K = 32): 32 bytes inside the swizzled row for K-major operands,
        // 32 K-rows of 128 bytes for MN-major ones (address field is in 16-byte units)
        constexpr uint32_t kstep = Cfg::kMnMajor ? (UMMA_K * 128) / 16 : UMMA_K / 16;
        uint32_t it = 0;
        bool ok = true;
        long long w_tmem = 0, w_full = 0, w_issue = 0; (void)w_tmem; (void)w_full; (void)w_issue;
        WorkWalker<STREAM_K> walk(p, unit, unit_stride, kb_total);
        Piece pc;
        while (ok && walk.next(pc, p, unit_stride, kb_total)) {
            for (int kb = pc.kb0; kb < pc.kb1; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                const int buf = it % NBUF;
                const uint32_t bph = (it / NBUF) & 1;
                if (kDualIssue && (it & 1u) != my_parity) continue;
                if (TWO && cta_rank != 0) {
                    // Second CTA of the pair: it issues no MMA.  This warp relays "my stage has landed"
                    // to the leader (a TMA load can only signal a barrier of the CTA it writes to).
                    ok = __all_sync(0xffffffffu, mbar_wait(full_bar(s), ph, p.status, kErrMmaWaitFull, p.launch_tag));
                    if (!ok) break;
                    // (no memory ordering needed: the stage was written by the TMA and is read by the
                    // tensor core, both through the async proxy; the barrier flip means the bytes landed)
                    if (elect_one()) mbar_arrive_cluster_relaxed(mapa_cluster(peer_full_bar(s), 0));
                    __syncwarp();
                    continue;
                }
                { RF_STAT_BEGIN();
                ok = __all_sync(0xffffffffu, mbar_wait(tmem_empty_bar(buf), bph ^ 1, p.status, kErrMmaWaitTmem, p.launch_tag));
                RF_STAT_END(w_tmem); }
                if (!ok) break;
                { RF_STAT_BEGIN();
                ok = __all_sync(0xffffffffu, mbar_wait(full_bar(s), ph, p.status, kErrMmaWaitFull, p.launch_tag));
                RF_STAT_END(w_full); }
                if (!ok) break;
                if (TWO) {
                    RF_STAT_BEGIN();
                    ok = __all_sync(0xffffffffu, mbar_wait(peer_full_bar(s), ph, p.status, kErrMmaWaitFull, p.launch_tag));
                    RF_STAT_END(w_full);
                    if (!ok) break;
                }
                tc_fence_after();
                RF_STAT_BEGIN();
                const uint32_t sa = smem_base + s * Cfg::kStageBytes;
                const uint64_t adesc = Cfg::kMnMajor ? smem_desc_mnmajor_sw128(sa, BK * 128, 1024)
                                                     : smem_desc_kmajor_sw128(sa);
                const uint64_t bdesc = Cfg::kMnMajor ? smem_desc_mnmajor_sw128(sa + Cfg::kABytes, BK * 128, 1024)
                                                     : smem_desc_kmajor_sw128(sa + Cfg::kABytes);
                const uint32_t d = tmem_base + buf * BN;
                if (elect_one()) {
#pragma unroll
                    for (int j = 0; j < BK / UMMA_K; ++j) {
                        if (TWO) umma_f8_2cta(d, adesc + kstep * j, bdesc + kstep * j, idesc, j > 0 ? 1u : 0u);
                        else umma_f8(d, adesc + kstep * j, bdesc + kstep * j, idesc, j > 0 ? 1u : 0u);
                    }
                    // One commit per K block (every tcgen05 instruction costs tensor-pipe
                    // issue time): it publishes the accumulator buffer, and the epilogue,
                    // which observes it, releases the smem stage on the MMA warp's behalf.
                    if (TWO) umma_commit_2cta_multicast(tmem_full_bar(buf), 0x3);   // same barrier in both CTAs
                    else umma_commit(tmem_full_bar(buf));
                }
                __syncwarp();
                RF_STAT_END(w_issue);
            }
        }
        if (lane == 0) { RF_STAT_FLUSH(1, w_tmem); RF_STAT_FLUSH(2, w_full); RF_STAT_FLUSH(6, w_issue); }
    } else if (STREAM_K && warp == 3) {
        // ------------------------------------------------- stream-K flag keeper
        // The fence that publishes this CTA's partial sums and the acquiring polls on other CTAs' flags cost
        // microseconds; this otherwise idle warp pays them, so the epilogue warps only store, load and pass two
        // shared-memory barriers.  (Memory order: epilogue stores -> mbarrier arrive [release.cta] -> this warp's
        // wait [acquire.cta] -> fence.acq_rel.gpu -> flag store; and on the other side flag load [acquire.gpu]
        // -> mbarrier arrive -> epilogue wait -> loads.  Both chains are causality-ordered.)
        const unsigned long long token = p.sk_token;
        unsigned long long* sk_flags = reinterpret_cast<unsigned long long*>(
            reinterpret_cast<char*>(p.partial) + (size_t)unit_stride * (BM * BN * sizeof(float)));
        const long long total = (long long)p.sk_tiles * kb_total;
        const int u_lo = sk_share_begin(total, unit, unit_stride);
        const int u_hi = sk_share_begin(total, unit + 1, unit_stride);
        bool ok = true;
        if (u_hi > u_lo && u_hi % kb_total != 0) {
            // the top of the share stops inside a tile: the first piece leaves partial sums
            ok = __all_sync(0xffffffffu, mbar_wait(sk_stored_bar, 0, p.status, kErrSchedWait, p.launch_tag));
            if (ok) {
                __threadfence();
                if (lane == 0) st_release_gpu_u64(sk_flags + unit, token);
            }
        }
        const int base = u_lo / kb_total * kb_total;       // first unit of the tile the share starts in
        if (ok && u_lo != base && u_hi >= base + kb_total) {
            // the bottom of the share starts inside a tile and reaches that tile's end: the last piece owns the
            // tile.  Its contributors are the CTAs below whose shares overlap the tile.
            for (int j = sk_first_contributor(total, unit, unit_stride, base); j < unit && ok; ++j) {
                if (!sk_contributes(total, j, unit_stride, base)) continue;
                ok = __all_sync(0xffffffffu, flag_wait_u64(sk_flags + j, token, p.status, kErrSchedWait, p.launch_tag));
                // consumed: cleared for the next launch that uses this scratch (a replayed graph carries the
                // same number every time)
                if (ok && lane == 0) sk_flags[j] = 0ull;
            }
            if (ok && lane == 0) mbar_arrive(sk_ready_bar);
        }
    }
    } else {
        // ---------------------------------------------------------- epilogue
        if (Cfg::kRebalanceRegs) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(Cfg::kRegsHi));
        const int ew = warp - NUM_NON_EPI_WARPS;
        const int quad = warp & 3;            // TMEM lane quadrant this warp may access
        const int grp = ew >> 2;              // column group
        const int row_in_tile = quad * 32 + lane;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
        uint32_t it = 0;
        uint32_t n_stores = 0;        // tile-store chunks issued by this warp so far
        bool ok = true;
        long long w_acc = 0, w_total = 0, w_rel = 0; (void)w_acc; (void)w_total; (void)w_rel;
        long long w_skw = 0, w_skf = 0, w_skr = 0; (void)w_skw; (void)w_skf; (void)w_skr;
#ifdef RF_WAIT_STATS
        const long long t_begin = clock64();
#endif
        // (in a CTA pair tmem_empty lives in the leader CTA, the only MMA issuer; both CTAs arrive on it
        // through the cluster window)
        // K-major scale tables have unit stride along K (a compile-time fact the address arithmetic of the
        // prefetch queue depends on); only the reference's [k/128][m] tables stride by m
        const int as_ks = Cfg::kMnMajor ? (int)p.as_k_stride : 1;
        const int bs_ks = Cfg::kMnMajor ? (int)p.bs_k_stride : 1;
        // out_scale (reference-layout configurations only): 1 for e4m3fn bytes.  e4m3fnuz bytes read as
        // e4m3fn are twice their value, so each operand that is consumed unconverted contributes 1/2; an
        // operand read from its converted copy (true values) contributes 1.  A power of two commutes
        // exactly with every rounding of the fp32 accumulation.
        float out_scale = 1.0f;
        if (Cfg::kMnMajor && p.fnuz_flags != nullptr)
            out_scale = (p.fnuz_flags[0] != 0 ? 1.0f : 0.5f) * (p.fnuz_flags[1] != 0 ? 1.0f : 0.5f);
        // Scale loads run PF K blocks ahead of their use so their latency (L2 or HBM) never sits on the
        // per-K-block critical path.  (Requesting a tile's first scales before the previous tile is stored was
        // measured: no gain on long K, 8 % slower on K <= 512.)
#if RF_EPI_WIDE
        constexpr int PF = 3;
#else
        constexpr int PF = 4;
#endif
        float qa[PF], qb[PF];
        int kb0 = 0, kb1 = 0;
        const float* as_row = p.a_scale;
        const float* bs_row = p.b_scale;
        auto begin_piece = [&](const Piece& pc) {
            const TileCoord t = decode_tile(p.splits == 1 ? pc.item : pc.item / p.splits, p.tiles_m, p.tiles_n);
            kb0 = pc.kb0;
            kb1 = pc.kb1;
            const int cta_m_blk = TWO ? t.m_blk * 2 + (int)cta_rank : t.m_blk;
            const int row = cta_m_blk * BM + row_in_tile;
            const int col0 = t.n_blk * BN + grp * CPT;
            as_row = p.a_scale + (long long)(row < p.m ? row : 0) * p.as_row_stride;
            bs_row = p.b_scale + (long long)(col0 < p.n ? (col0 >> 7) : 0) * p.bs_row_stride;
#pragma unroll
            for (int d = 0; d < PF; ++d) {
                const int kk = min(kb0 + d, kb1 - 1);
                qa[d] = __ldg(as_row + kk * as_ks);
                qb[d] = __ldg(bs_row + kk * bs_ks);
            }
        };
        // The next piece is drawn (tile decoded, scale pointers set, first scales requested) in the middle of the
        // current tile's store, between its first and second chunk, where the warp would otherwise wait for the
        // TMA to have read the slab it is about to rewrite (about 240 cycles per chunk, measured).
        WorkWalker<STREAM_K> walk(p, unit, unit_stride, kb_total);
        Piece pc;
        bool have = walk.next(pc, p, unit_stride, kb_total);
        if (have) begin_piece(pc);
        auto advance = [&] {
            have = walk.next(pc, p, unit_stride, kb_total);
            if (have) begin_piece(pc);
        };
        float2 acc[CPT / 2];
        bool zeroed = false;      // the tile store of the previous tile left every accumulator cleared
        while (ok && have) {
            const int cur_item = pc.item;     // `pc` moves on to the next piece during the store
            bool fresh = true;        // the accumulators still have to be cleared
            if (STREAM_K && kb0 > 0 && kb1 == kb_total) {
                // Stream-K owner piece (the tile's last K blocks; always this CTA's last piece of the region):
                // the accumulators start from the partial sums that lower CTAs left in their scratch slots at
                // the very beginning of their runs, added in ascending K order (a fixed order for a given grid,
                // so results do not depend on timing).  The loads are in flight while the pipeline fills.
                { RF_STAT_BEGIN();
                ok = __all_sync(0xffffffffu, mbar_wait(sk_ready_bar, 0, p.status, kErrSchedWait, p.launch_tag));
                RF_STAT_END(w_skf); }
                if (!ok) break;
                RF_STAT_BEGIN();
                const long long total = (long long)p.sk_tiles * kb_total;
                const int base = (pc.item - sk_tile0(p)) * kb_total;      // the tile's first unit
                for (int j = sk_first_contributor(total, unit, unit_stride, base); j < unit; ++j) {
                    if (!sk_contributes(total, j, unit_stride, base)) continue;
                    const float4* src = reinterpret_cast<const float4*>(p.partial) + (size_t)j * (BM * BN / 4) +
                                        ((int)threadIdx.x - 32 * NUM_NON_EPI_WARPS);
                    if (fresh) {
#pragma unroll
                        for (int q = 0; q < CPT / 4; ++q) {
                            const float4 t4 = __ldcg(src + q * (32 * Cfg::kEpiWarps));
                            acc[2 * q] = make_float2(t4.x, t4.y);
                            acc[2 * q + 1] = make_float2(t4.z, t4.w);
                        }
                        fresh = false;
                    } else {
#pragma unroll
                        for (int q0 = 0; q0 < CPT / 4; q0 += 8) {
                            float4 t4[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) t4[i] = __ldcg(src + (q0 + i) * (32 * Cfg::kEpiWarps));
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                acc[2 * (q0 + i)].x += t4[i].x;
                                acc[2 * (q0 + i)].y += t4[i].y;
                                acc[2 * (q0 + i) + 1].x += t4[i].z;
                                acc[2 * (q0 + i) + 1].y += t4[i].w;
                            }
                        }
                    }
                }
                RF_STAT_END(w_skr);
            }
            if (fresh && !zeroed) {
#pragma unroll
                for (int j = 0; j < CPT / 2; ++j) acc[j] = make_float2(0.f, 0.f);
            }
            zeroed = false;
#if RF_EPI_WIDE
            // two 32-column staging buffers, reloaded in place
            float v[2][32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[0][j] = v[1][j] = 0.f;
#endif
#if RF_EPI_WIDE
#pragma unroll 1
#else
#pragma unroll 4
#endif
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                const float s = Cfg::kMnMajor ? qa[0] * qb[0] * out_scale : qa[0] * qb[0];
#pragma unroll
                for (int d = 0; d + 1 < PF; ++d) { qa[d] = qa[d + 1]; qb[d] = qb[d + 1]; }
                {
                    const int kk = min(kb + PF, kb1 - 1);
                    qa[PF - 1] = __ldg(as_row + kk * as_ks);
                    qb[PF - 1] = __ldg(bs_row + kk * bs_ks);
                }
                const float2 s2 = make_float2(s, s);
                const int buf = it % NBUF;
                const uint32_t bph = (it / NBUF) & 1;
                { RF_STAT_BEGIN();
                if (!mbar_wait(tmem_full_bar(buf), bph, p.status, kErrEpilogueWait, p.launch_tag)) { ok = false; break; }
                RF_STAT_END(w_acc); }
                tc_fence_after();
                // The MMAs that wrote this buffer have finished reading their smem stage.
                if (ew == 0 && lane == 0) mbar_arrive(empty_bar(it % STAGES));
                const uint32_t taddr = lane_addr + buf * BN + grp * CPT;
                constexpr int NCH = CPT / 32;
                auto release_buffer = [&] {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (TWO) mbar_arrive_cluster_relaxed(mapa_cluster(tmem_empty_bar(buf), 0));
                        else mbar_arrive(tmem_empty_bar(buf));
                    }
                };
                RF_STAT_BEGIN();
#if RF_EPI_WIDE
                // The first 64 columns are requested together (two loads: one 64-column load would need 64
                // consecutive registers, which costs spills); while their FMAs run, the loads of the next two
                // 32-column chunks are already in flight, so the accumulator buffer is handed back after two
                // load latencies (one, when the thread owns only 64 columns); the last FMAs run after that.
                auto fma_chunk = [&](int c, const float (&x)[32]) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        acc[c * 16 + j] = __ffma2_rn(make_float2(x[2 * j], x[2 * j + 1]), s2, acc[c * 16 + j]);
                };
                tmem_ld32_async_inplace(taddr, v[0]);
                tmem_ld32_async_inplace(taddr + 32, v[1]);
                tmem_ld_fence2(v[0], v[1]);
                if (NCH == 2) {
                    release_buffer();
                    RF_STAT_END(w_rel);
                    fma_chunk(0, v[0]);
                    fma_chunk(1, v[1]);
                } else {
                    fma_chunk(0, v[0]);
                    tmem_ld32_async_inplace(taddr + 64, v[0]);
                    fma_chunk(1, v[1]);
                    tmem_ld32_async_inplace(taddr + 96, v[1]);
                    tmem_ld_fence2(v[0], v[1]);
                    release_buffer();
                    RF_STAT_END(w_rel);
                    fma_chunk(2, v[0]);
                    fma_chunk(3, v[1]);
                }
#else
                // Staging registers: two 32-column buffers (the load of chunk c+1 overlaps the FMAs of
                // chunk c) when a thread owns 64 columns; one buffer when it owns 128, because 128
                // accumulators leave no room for a second one (the other epilogue warp on the same
                // scheduler covers the load latency instead).
                constexpr int NV = CPT > 64 ? 1 : 2;
                float v[NV][32];
                tmem_ld32_async(taddr, v[0]);
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    tmem_ld_fence(v[c % NV]);   // waits for every load issued so far
                    if (NV == 2 && c + 1 < NCH) tmem_ld32_async(taddr + (c + 1) * 32, v[(c + 1) % NV]);
#ifndef RF_LATE_RELEASE
                    if (c + 1 == NCH) { release_buffer(); RF_STAT_END(w_rel); }
#endif
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        acc[c * 16 + j] =
                            __ffma2_rn(make_float2(v[c % NV][2 * j], v[c % NV][2 * j + 1]), s2, acc[c * 16 + j]);
                    if (NV == 1 && c + 1 < NCH) tmem_ld32_async(taddr + (c + 1) * 32, v[0]);
                }
#ifdef RF_LATE_RELEASE
                release_buffer(); RF_STAT_END(w_rel);
#endif
#endif
            }
            if (!ok) break;
            if (STREAM_K && kb1 < kb_total) {
                // Stream-K contributor piece (always this CTA's first piece): the 128 x BN fp32 partial sums go to
                // this CTA's scratch slot, laid out [float4 number][epilogue thread] so that writer and reader,
                // which map threads to elements alike, move whole 512-byte lines.  Warp 3 publishes them.
                RF_STAT_BEGIN();
                float4* dst = reinterpret_cast<float4*>(p.partial) + (size_t)unit * (BM * BN / 4) +
                              ((int)threadIdx.x - 32 * NUM_NON_EPI_WARPS);
#pragma unroll
                for (int q = 0; q < CPT / 4; ++q)
                    __stcg(dst + q * (32 * Cfg::kEpiWarps),
                           make_float4(acc[2 * q].x, acc[2 * q].y, acc[2 * q + 1].x, acc[2 * q + 1].y));
                __syncwarp();
                if (lane == 0) mbar_arrive(sk_stored_bar);
                RF_STAT_END(w_skw);
                advance();
                continue;
            }
            // Tile store: each warp stages its 32 rows x 128 bytes in its own swizzled shared-memory slab, so
            // that global memory is written in whole 128-byte row segments.
            {
                constexpr int SL = Cfg::kSlabs;
                const TileCoord t = decode_tile(p.splits == 1 ? cur_item : cur_item / p.splits, p.tiles_m, p.tiles_n);
                const int cta_m_blk = TWO ? t.m_blk * 2 + (int)cta_rank : t.m_blk;
                const int col0 = t.n_blk * BN + grp * CPT;
                const uint32_t slab0 = slab_base + ew * SL * Cfg::kSlabBytes;
                // (128-wide tiles hold 64 accumulators per thread and store one chunk, or two short fp32 ones:
                // measured, drawing the next piece in between makes them slower, so they draw it afterwards)
                constexpr bool kAdvanceMidStore = CPT == 128;
                constexpr bool kClearInStore = CPT == 128 && SL == 1;
                bool advanced = false;
                const int slab_row0 = cta_m_blk * BM + quad * 32;
                // One lane hands the slab to the TMA, which clips rows >= m / columns >= n.  Consecutive stores of
                // this warp alternate over its kSlabs slabs (n_stores counts them across tiles, so skipped chunks
                // of a ragged tile cannot break the alternation); before a slab is rewritten, the store that last
                // read it (kSlabs commit groups ago) must have finished reading.  (Reading the slab back and
                // writing C with ordinary vector stores was measured: 20 % slower on the short-K shapes.)
                if (p.splits == 1) {
#pragma unroll
                    for (int ch = 0; ch < CPT / 64; ++ch) {
                        if (col0 + ch * 64 >= p.n) break;
                        const uint32_t slab = slab0 + (n_stores % SL) * Cfg::kSlabBytes;
                        ++n_stores;
                        const uint32_t my_row = slab + lane * 128;
                        if (lane == 0) tma_store_wait_read<SL - 1>();
                        __syncwarp();
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const int a0 = ch * 32 + j * 4;
                            st_shared_v4(my_row + ((j ^ (lane & 7)) << 4),
                                         pack_bf16x2(acc[a0 + 0].x, acc[a0 + 0].y), pack_bf16x2(acc[a0 + 1].x, acc[a0 + 1].y),
                                         pack_bf16x2(acc[a0 + 2].x, acc[a0 + 2].y), pack_bf16x2(acc[a0 + 3].x, acc[a0 + 3].y));
                        }
                        // These accumulators are done with: cleared for the next tile here, in the shadow of the
                        // shared-memory stores the fence below waits for.  (Measured: 2 % on the K ~ 2048 shapes
                        // with the four-stage configuration; the two-slab short-K configuration gets 7-10 %
                        // slower with it and keeps clearing at the top of the tile.)
                        if (kClearInStore) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) acc[ch * 32 + j] = make_float2(0.f, 0.f);
                            zeroed = ch + 1 == CPT / 64;      // (every chunk of the thread's columns was stored)
                        }
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            if (p.n_dest <= 1) {
                                tma_store_2d(&tma_c, slab, col0 + ch * 64, slab_row0);
                            } else {
                                // N-split GEMM: the slab goes to every GPU's C (own memory and peers over
                                // NVLink), which is the all-gather of C done by the epilogue itself
                                // (own copy first, then rank+1, rank+2, ...: at any moment the ranks store
                                // into different GPUs)
                                for (int dd = 0; dd < p.n_dest; ++dd) {
                                    int dst = p.dest_first + dd;
                                    if (dst >= p.n_dest) dst -= p.n_dest;
                                    tma_store_2d(&dests.m[dst], slab, p.c_col_offset + col0 + ch * 64, slab_row0);
                                }
                            }
                            tma_store_commit();
                        }
                        if (kAdvanceMidStore && ch == 0) {
                            advance();
                            advanced = true;
                        }
                    }
                } else {
                    const int cur_split = cur_item % p.splits;
#pragma unroll
                    for (int ch = 0; ch < CPT / 32; ++ch) {
                        if (col0 + ch * 32 >= p.n) break;
                        const uint32_t slab = slab0 + (n_stores % SL) * Cfg::kSlabBytes;
                        ++n_stores;
                        const uint32_t my_row = slab + lane * 128;
                        if (lane == 0) tma_store_wait_read<SL - 1>();
                        __syncwarp();
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const int a0 = ch * 16 + j * 2;
                            st_shared_v4(my_row + ((j ^ (lane & 7)) << 4), __float_as_uint(acc[a0].x),
                                         __float_as_uint(acc[a0].y), __float_as_uint(acc[a0 + 1].x),
                                         __float_as_uint(acc[a0 + 1].y));
                        }
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_3d(&tma_p, slab, col0 + ch * 32, slab_row0, cur_split);
                            tma_store_commit();
                        }
                        if (kAdvanceMidStore && ch == 0) {
                            advance();
                            advanced = true;
                        }
                    }
                }
                if (!advanced) advance();
            }
        }
        // Before exit the warp's slab must have been read by its last store.  Waiting for the writes themselves
        // is left to grid completion (stream order, or the next kernel's griddepcontrol.wait), except when the
        // stores go to other GPUs: the barrier that follows an N-split GEMM is taken after the data has landed.
        if (lane == 0) {
            if (p.n_dest > 1) tma_store_wait_all<0>();
            else tma_store_wait_read<0>();
        }
#ifdef RF_WAIT_STATS
        if (warp == NUM_NON_EPI_WARPS && lane == 0) {
            RF_STAT_FLUSH(3, w_acc);
            RF_STAT_FLUSH(4, clock64() - t_begin);
            RF_STAT_FLUSH(5, w_rel);
            RF_STAT_FLUSH(7, w_skw);
            RF_STAT_FLUSH(8, w_skf);
            RF_STAT_FLUSH(9, w_skr);
        }
#endif
    }

    // ------------------------------------------------------------- tear-down
    tc_fence_before();
    __syncthreads();
    if (TWO) cluster_sync_all();     // the peer no longer touches this CTA's barriers, smem or TMEM
    if (warp == 1) {
        tc_fence_after();
        if (TWO) tmem_dealloc_2cta(tmem_base, Cfg::kTmemCols);
        else tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// C = bf16( sum_s partial[s] )  -  split-K fix-up (reference: reduce_kernel,
// src/gemm/gemm_kernel.cpp:288-303).  One float4 per thread per slice.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ c, size_t mn, int splits) {
    griddep_launch_dependents();
    griddep_wait();     // the slices come from the GEMM launched just before
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= mn) return;
    float4 acc = *reinterpret_cast<const float4*>(partial + i);
    for (int s = 1; s < splits; ++s) {
        const float4 v = *reinterpret_cast<const float4*>(partial + (size_t)s * mn + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    uint2 q;
    q.x = pack_bf16x2(acc.x, acc.y);
    q.y = pack_bf16x2(acc.z, acc.w);
    *reinterpret_cast<uint2*>(c + i) = q;
}

// e4m3fnuz -> e4m3fn at equal value, one pass over an operand.
//
// The GEMM reads e4m3fnuz bytes as e4m3fn (twice the value, exactly, folded into the scale product) - except
// that 0x7F / 0xFF (+-240, the largest fnuz magnitudes, present in every block of amax-scaled data) read as
// NaN and 0x80 (the fnuz NaN) reads as -0.  This pass writes, for the whole operand, the e4m3fn byte of the
// SAME value: byte - 8 for exponent fields >= 2; the 15 magnitudes below 2^-6 fall between e4m3fn's
// subnormals and are rounded to nearest-even on that grid (absolute error <= 2^-10); 0x80 becomes the e4m3fn
// NaN.  If the operand holds one of the three special bytes its flag is raised and the GEMM launched next
// on the stream reads the converted copy; otherwise the GEMM uses the original bytes and stays exact.
__global__ void __launch_bounds__(256)
fnuz_convert_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n_vec, int* __restrict__ flag,
                    int* __restrict__ status) {
    __shared__ uint8_t lut[256];
    {
        const uint32_t b = threadIdx.x;
        const uint32_t sign = b & 0x80u, x = b & 0x7Fu;
        uint32_t o;
        if (b == 0x80u) o = 0x7Fu;                                    // NaN stays NaN
        else if (x >= 16u) o = sign | (x - 8u);                       // same value, exponent field one lower
        else o = sign | ((x + ((x >> 1) & 1u)) >> 1);                 // x * 2^-10 on the 2^-9 grid, nearest-even
        lut[b] = (uint8_t)o;
    }
    __syncthreads();
    bool special = false;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 q = __ldg(src + i);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t x = w[j];
            const uint32_t m7f = x & 0x7F7F7F7Fu;
            // a byte equals 0x7F in its low 7 bits  <=>  (m7f + 0x01010101) has bit 7 set in that byte
            const uint32_t is7f = (m7f + 0x01010101u) & 0x80808080u;
            // a byte equals 0x80  <=>  low 7 bits zero and bit 7 set
            const uint32_t low_zero = ~((m7f + 0x7F7F7F7Fu) | 0x7F7F7F7Fu);   // bit 7 set where low 7 bits == 0
            const uint32_t is80 = low_zero & x & 0x80808080u;
            special |= (is7f | is80) != 0;
            o[j] = (uint32_t)lut[x & 0xFFu] | ((uint32_t)lut[(x >> 8) & 0xFFu] << 8) |
                   ((uint32_t)lut[(x >> 16) & 0xFFu] << 16) | ((uint32_t)lut[x >> 24] << 24);
        }
        dst[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    if (special) {
        *flag = 1;
        atomicOr(status + kStatusDiagWord, (int)kDiagFnuzByte);
    }
}

using Cfg128 = GemmCfg<128, 6>;
using Cfg256 = GemmCfg<256, 4>;
using Cfg256ShortK = GemmCfg<256, 3, false, false, 2>;     // K <= 512: tiles of at most four K blocks
using CfgPair = GemmCfg<256, 6, true>;      // 256 x 256 tile per CTA pair
using CfgPair128 = GemmCfg<128, 8, true>;   // 256 x 128 tile per CTA pair: four accumulator buffers in TMEM
using Cfg128Mn = GemmCfg<128, 6, false, true>;
using Cfg256Mn = GemmCfg<256, 4, false, true>;

// Programmatic dependent launch between consecutive GEMM-path kernels of a stream (the launch latency and
// the barrier / TMEM set-up of kernel i+1 overlap the tail of kernel i).  RF_FP8_GEMM_PDL=0 switches it off.
bool overlap_launches() {
    static const bool on = [] {
        const char* e = getenv("RF_FP8_GEMM_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

// Tiles of at most four K blocks spend a large share of their time in the tile store: they get the
// two-slab configuration (RF_FP8_GEMM_SHORTK=0 keeps the ordinary one).
bool short_k_config(const GemmParams& p) {
    static const bool on = [] {
        const char* e = getenv("RF_FP8_GEMM_SHORTK");
        return !(e && e[0] == '0');
    }();
    return on && p.splits == 1 && p.k <= 4 * BK;
}

template <class Cfg, bool STREAM_K = false>
cudaError_t launch_cfg(const CUtensorMap& tma_a, const CUtensorMap& tma_b, const CUtensorMap& tma_c,
                       const CUtensorMap& tma_p, const GemmDestMaps& dests, const GemmParams& p, int num_sms,
                       cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = fp8_gemm_kernel<Cfg, STREAM_K>;
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    const int total = p.tiles_m * p.tiles_n * p.splits;
    if (!Cfg::kTwoCta) {
        // a stream-K launch shares K blocks out over exactly num_sms CTAs, whatever the tile count
        const int grid = (total < num_sms && p.sk_tiles == 0) ? total : num_sms;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid, 1, 1);
        cfg.blockDim = dim3(Cfg::kThreads, 1, 1);
        cfg.dynamicSmemBytes = Cfg::kSmemBytes;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = overlap_launches() ? 1 : 0;
        return cudaLaunchKernelEx(&cfg, kernel, tma_a, tma_b, tma_c, tma_p, dests, p);
    }
    // CTA pairs: clusters of 2 along x, one pair per work item at most
    const int pairs = total < num_sms / 2 ? total : num_sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(Cfg::kThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, tma_a, tma_b, tma_c, tma_p, dests, p);
}

}  // namespace

namespace {
template <bool STREAM_K>
int walk_pieces(const GemmParams& p, int unit, int n_units, int* out, int max_pieces) {
    const int kb_total = p.k / BK;
    WorkWalker<STREAM_K> walk(p, unit, n_units, kb_total);
    Piece pc;
    int n = 0;
    while (walk.next(pc, p, n_units, kb_total)) {
        if (n < max_pieces) {
            out[4 * n + 0] = pc.item / p.splits;
            out[4 * n + 1] = pc.item % p.splits;
            out[4 * n + 2] = pc.kb0;
            out[4 * n + 3] = pc.kb1;
        }
        ++n;
    }
    return n;
}
}  // namespace

int fp8_gemm_walk_pieces(const GemmParams& p, int unit, int n_units, int* out, int max_pieces) {
    return p.sk_tiles > 0 ? walk_pieces<true>(p, unit, n_units, out, max_pieces)
                          : walk_pieces<false>(p, unit, n_units, out, max_pieces);
}

#ifdef RF_WAIT_STATS
extern "C" void rf_debug_wait_stats(unsigned long long* out8, int reset) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out8, g_wait_stats, sizeof(unsigned long long) * 12);
    if (reset) {
        unsigned long long z[12] = {};
        cudaMemcpyToSymbol(g_wait_stats, z, sizeof(z));
    }
}
#endif

cudaError_t fp8_fnuz_convert_launch(const void* src, void* dst, size_t n_bytes, int* flag, int* status, int num_sms,
                                    cudaStream_t stream) {
    const size_t n_vec = n_bytes / 16;
    cudaError_t e = cudaMemsetAsync(flag, 0, sizeof(int), stream);
    if (e != cudaSuccess || n_vec == 0) return e;
    size_t blocks = (n_vec + 255) / 256;
    if (blocks > (size_t)num_sms * 8) blocks = (size_t)num_sms * 8;
    fnuz_convert_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst),
                                                             n_vec, flag, status);
    return cudaGetLastError();
}

namespace {
template <class Cfg, bool STREAM_K = false>
cudaError_t prepare_cfg() {
    return cudaFuncSetAttribute(fp8_gemm_kernel<Cfg, STREAM_K>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                Cfg::kSmemBytes);
}
}  // namespace

cudaError_t fp8_gemm_prepare_device() {
    cudaError_t e;
    if ((e = prepare_cfg<Cfg128>()) != cudaSuccess) return e;
    if ((e = prepare_cfg<Cfg256>()) != cudaSuccess) return e;
    if ((e = prepare_cfg<Cfg128, true>()) != cudaSuccess) return e;
    if ((e = prepare_cfg<Cfg256, true>()) != cudaSuccess) return e;
    if ((e = prepare_cfg<Cfg256ShortK>()) != cudaSuccess) return e;
    if ((e = prepare_cfg<CfgPair>()) != cudaSuccess) return e;
    if ((e = prepare_cfg<CfgPair128>()) != cudaSuccess) return e;
    if ((e = prepare_cfg<Cfg128Mn>()) != cudaSuccess) return e;
    if ((e = prepare_cfg<Cfg256Mn>()) != cudaSuccess) return e;
    // the split-K fix-up takes no attribute; querying it loads the function now, not at its first launch
    cudaFuncAttributes fa;
    return cudaFuncGetAttributes(&fa, splitk_reduce_kernel);
}

cudaError_t fp8_gemm_launch(const CUtensorMap& tma_a, const CUtensorMap& tma_b, const CUtensorMap& tma_c,
                            const CUtensorMap& tma_p, const GemmDestMaps* dests, const GemmParams& p, int block_n,
                            int num_sms, cudaStream_t stream, bool mn_major) {
    GemmDestMaps local;
    if (!dests) {
        for (int i = 0; i < 8; ++i) local.m[i] = tma_c;
        dests = &local;
    }
    // block_n: 128 / 256 = one-CTA tiles of that width; 512 / 384 = the CTA-pair configurations (256 x 256 and
    // 256 x 128 per pair)
    if (p.sk_tiles > 0) {
        // stream-K: row-major operands, one destination, the one-CTA tiles
        if (mn_major || gemm_is_pair(block_n) || p.splits != 1 || p.n_dest > 1) return cudaErrorInvalidValue;
        return block_n == 256 ? launch_cfg<Cfg256, true>(tma_a, tma_b, tma_c, tma_p, *dests, p, num_sms, stream)
                              : launch_cfg<Cfg128, true>(tma_a, tma_b, tma_c, tma_p, *dests, p, num_sms, stream);
    }
    cudaError_t e = mn_major
                        ? (block_n == 256 ? launch_cfg<Cfg256Mn>(tma_a, tma_b, tma_c, tma_p, *dests, p, num_sms, stream)
                                          : launch_cfg<Cfg128Mn>(tma_a, tma_b, tma_c, tma_p, *dests, p, num_sms, stream))
                    : block_n == 512 ? launch_cfg<CfgPair>(tma_a, tma_b, tma_c, tma_p, *dests, p, num_sms, stream)
                    : block_n == 384 ? launch_cfg<CfgPair128>(tma_a, tma_b, tma_c, tma_p, *dests, p, num_sms, stream)
                    : block_n == 256
                        ? (short_k_config(p) ? launch_cfg<Cfg256ShortK>(tma_a, tma_b, tma_c, tma_p, *dests, p, num_sms, stream)
                                             : launch_cfg<Cfg256>(tma_a, tma_b, tma_c, tma_p, *dests, p, num_sms, stream))
                        : launch_cfg<Cfg128>(tma_a, tma_b, tma_c, tma_p, *dests, p, num_sms, stream);
    if (e != cudaSuccess) return e;
    if (p.splits > 1) {
        const size_t mn = (size_t)p.m * p.n;
        const unsigned blocks = (unsigned)((mn / 4 + 255) / 256);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(blocks, 1, 1);
        cfg.blockDim = dim3(256, 1, 1);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = overlap_launches() ? 1 : 0;
        e = cudaLaunchKernelEx(&cfg, splitk_reduce_kernel, (const float*)p.partial, (__nv_bfloat16*)p.c, mn,
                               (int)p.splits);
    }
    return e;
}

}  // namespace rf
