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
//   warp 1      MMA issuer: per 128-deep K block, 4 x tcgen05.mma.kind::f8f6f4
//               (K = 32 each) into one of 512/BN TMEM accumulator buffers, then
//               tcgen05.commit to free the smem stage and publish the buffer
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

namespace rf {

#ifdef RF_WAIT_STATS
// Debug build only: cycles each role spent inside its barrier waits, summed over CTAs.
__device__ unsigned long long g_wait_stats[8];
#define RF_STAT_BEGIN() const long long _t0 = clock64()
#define RF_STAT_END(acc) (acc) += clock64() - _t0
#define RF_STAT_FLUSH(idx, acc) atomicAdd(&g_wait_stats[idx], (unsigned long long)(acc))
#else
#define RF_STAT_BEGIN()
#define RF_STAT_END(acc)
#define RF_STAT_FLUSH(idx, acc)
#endif

namespace {

constexpr int BM = 128;
constexpr int BK = 128;          // one scale block, one 128-byte swizzle row of fp8
constexpr int UMMA_K = 32;       // K per tcgen05.mma for 8-bit operands
constexpr int NUM_NON_EPI_WARPS = 4;

template <int BN, int STAGES>
struct GemmCfg {
    static constexpr int kBN = BN;
    static constexpr int kStages = STAGES;
    static constexpr int kEpiGroups = 2;                       // column groups, 4 warps each
    static constexpr int kColsPerThread = BN / kEpiGroups;     // 64 or 128: one scale block at most
    static constexpr int kEpiWarps = 4 * kEpiGroups;
    static constexpr int kThreads = 32 * (NUM_NON_EPI_WARPS + kEpiWarps);   // 384
    static constexpr int kABytes = BM * BK;
    static constexpr int kBBytes = BN * BK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemBufs = 512 / BN;                // accumulator buffers in flight
    static constexpr int kTmemCols = kTmemBufs * BN;          // all 512 TMEM columns
    static constexpr int kBarBytes = (2 * STAGES + 2 * kTmemBufs) * 8 + 16;
    static constexpr int kSlabBytes = 32 * 128;               // per epilogue warp: 32 rows x 128 B, swizzled
    static constexpr int kSmemBytes =
        STAGES * kStageBytes + kEpiWarps * kSlabBytes + kBarBytes + 1024;       // + alignment slack
    // 128 accumulators per thread need more than the 168 registers a 384-thread
    // CTA starts with: the producer warpgroup gives registers to the epilogue.
    static constexpr bool kRebalanceRegs = kColsPerThread > 64;
    static_assert(kColsPerThread == 64 || kColsPerThread == 128, "epilogue handles 64 or 128 columns per thread");
    static_assert(kTmemCols == 512, "TMEM columns: power of two, at most 512");
    static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

struct TileCoord {
    int m_blk, n_blk, split;
};

// Work item -> tile.  Consecutive work items walk down M inside a band of
// GROUP_M row blocks before moving to the next column block, so the CTAs that
// run concurrently share B tiles (and A bands) in L2.  K slices of one tile are
// adjacent.
__device__ __forceinline__ TileCoord decode_work(int w, int tiles_m, int tiles_n, int splits) {
    constexpr int GROUP_M = 8;
    TileCoord t;
    t.split = w % splits;
    int tile = w / splits;
    int band = tile / (GROUP_M * tiles_n);
    int first_m = band * GROUP_M;
    int band_rows = min(GROUP_M, tiles_m - first_m);
    int in_band = tile - band * GROUP_M * tiles_n;
    t.m_blk = first_m + in_band % band_rows;
    t.n_blk = in_band / band_rows;
    return t;
}

template <class Cfg>
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
    const uint32_t bar_base = slab_base + Cfg::kEpiWarps * Cfg::kSlabBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tmem_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
    auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + NBUF + b); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 2 * NBUF);
    uint32_t* tmem_slot_ptr =
        reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tma_a);
        tma_prefetch_desc(&tma_b);
        tma_prefetch_desc(p.splits == 1 ? &tma_c : &tma_p);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < NBUF; ++b) {
            mbar_init(tmem_full_bar(b), 1);
            mbar_init(tmem_empty_bar(b), Cfg::kEpiWarps);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot_ptr);

    const int total_work = p.tiles_m * p.tiles_n * p.splits;
    const int kb_total = p.k / BK;

    if (warp < NUM_NON_EPI_WARPS) {
    if (Cfg::kRebalanceRegs) asm volatile("setmaxnreg.dec.sync.aligned.u32 72;\n");
    // Producer and MMA warps keep all 32 lanes in the loops (warp-uniform control
    // flow, so descriptors and addresses live in uniform registers) and elect one
    // lane only for the instructions that must be issued once.
    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        uint32_t it = 0;  // running K-block counter across work items
        bool ok = true;
        long long w_empty = 0; (void)w_empty;
        for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
            const TileCoord t = decode_work(w, p.tiles_m, p.tiles_n, p.splits);
            const int kb0 = (int)((long long)kb_total * t.split / p.splits);
            const int kb1 = (int)((long long)kb_total * (t.split + 1) / p.splits);
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                { RF_STAT_BEGIN();
                ok = __all_sync(0xffffffffu, mbar_wait(empty_bar(s), ph ^ 1, p.status, kErrProducerWait));
                RF_STAT_END(w_empty); }
                if (!ok) break;
                if (elect_one()) {
                    mbar_expect_tx(full_bar(s), Cfg::kStageBytes);
                    const uint32_t sa = smem_base + s * Cfg::kStageBytes;
                    tma_load_2d(sa, &tma_a, full_bar(s), kb * BK, t.m_blk * BM);
                    tma_load_2d(sa + Cfg::kABytes, &tma_b, full_bar(s), kb * BK, t.n_blk * BN);
                }
                __syncwarp();
            }
        }
        if (lane == 0) { RF_STAT_FLUSH(0, w_empty); }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        constexpr uint32_t idesc = make_idesc(BM, BN, /*e4m3*/ 0, /*e4m3*/ 0, 0, 0);
        uint32_t it = 0;
        bool ok = true;
        long long w_tmem = 0, w_full = 0; (void)w_tmem; (void)w_full;
        for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
            const TileCoord t = decode_work(w, p.tiles_m, p.tiles_n, p.splits);
            const int kb0 = (int)((long long)kb_total * t.split / p.splits);
            const int kb1 = (int)((long long)kb_total * (t.split + 1) / p.splits);
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                const int buf = it % NBUF;
                const uint32_t bph = (it / NBUF) & 1;
                { RF_STAT_BEGIN();
                ok = __all_sync(0xffffffffu, mbar_wait(tmem_empty_bar(buf), bph ^ 1, p.status, kErrMmaWaitTmem));
                RF_STAT_END(w_tmem); }
                if (!ok) break;
                { RF_STAT_BEGIN();
                ok = __all_sync(0xffffffffu, mbar_wait(full_bar(s), ph, p.status, kErrMmaWaitFull));
                RF_STAT_END(w_full); }
                if (!ok) break;
                tc_fence_after();
                const uint32_t sa = smem_base + s * Cfg::kStageBytes;
                const uint64_t adesc = smem_desc_kmajor_sw128(sa);
                const uint64_t bdesc = smem_desc_kmajor_sw128(sa + Cfg::kABytes);
                const uint32_t d = tmem_base + buf * BN;
                if (elect_one()) {
#pragma unroll
                    for (int j = 0; j < BK / UMMA_K; ++j) {
                        // +32 bytes along K inside the swizzled row = +2 in the (addr >> 4) field
                        umma_f8(d, adesc + 2 * j, bdesc + 2 * j, idesc, j > 0 ? 1u : 0u);
                    }
                    // One commit per K block (every tcgen05 instruction costs tensor-pipe
                    // issue time): it publishes the accumulator buffer, and the epilogue,
                    // which observes it, releases the smem stage on the MMA warp's behalf.
                    umma_commit(tmem_full_bar(buf));
                }
                __syncwarp();
            }
        }
        if (lane == 0) { RF_STAT_FLUSH(1, w_tmem); RF_STAT_FLUSH(2, w_full); }
    }
    } else {
        // ---------------------------------------------------------- epilogue
        if (Cfg::kRebalanceRegs) asm volatile("setmaxnreg.inc.sync.aligned.u32 216;\n");
        const int ew = warp - NUM_NON_EPI_WARPS;
        const int quad = warp & 3;            // TMEM lane quadrant this warp may access
        const int grp = ew >> 2;              // column group
        const int row_in_tile = quad * 32 + lane;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
        const int kbs = p.k / BK;
        uint32_t it = 0;
        bool ok = true;
        long long w_acc = 0, w_total = 0; (void)w_acc; (void)w_total;
#ifdef RF_WAIT_STATS
        const long long t_begin = clock64();
#endif
        for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
            const TileCoord t = decode_work(w, p.tiles_m, p.tiles_n, p.splits);
            const int kb0 = (int)((long long)kb_total * t.split / p.splits);
            const int kb1 = (int)((long long)kb_total * (t.split + 1) / p.splits);
            const int row = t.m_blk * BM + row_in_tile;
            const int col0 = t.n_blk * BN + grp * CPT;
            const bool row_ok = row < p.m;
            const int nb = col0 >> 7;
            const bool nb_ok = col0 < p.n;
            const float* as_row = p.a_scale + (size_t)(row_ok ? row : 0) * kbs;
            const float* bs_row = p.b_scale + (size_t)(nb_ok ? nb : 0) * kbs;

            float2 acc[CPT / 2];
#pragma unroll
            for (int j = 0; j < CPT / 2; ++j) acc[j] = make_float2(0.f, 0.f);

            // Scale loads run PF K blocks ahead of their use so their latency
            // (L2 or HBM) never sits on the per-K-block critical path.
            constexpr int PF = 4;
            float qa[PF], qb[PF];
#pragma unroll
            for (int d = 0; d < PF; ++d) {
                const int kk = min(kb0 + d, kb1 - 1);
                qa[d] = __ldg(as_row + kk);
                qb[d] = __ldg(bs_row + kk);
            }
#pragma unroll 4
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                const float s = qa[0] * qb[0];
#pragma unroll
                for (int d = 0; d + 1 < PF; ++d) { qa[d] = qa[d + 1]; qb[d] = qb[d + 1]; }
                {
                    const int kk = min(kb + PF, kb1 - 1);
                    qa[PF - 1] = __ldg(as_row + kk);
                    qb[PF - 1] = __ldg(bs_row + kk);
                }
                const float2 s2 = make_float2(s, s);
                const int buf = it % NBUF;
                const uint32_t bph = (it / NBUF) & 1;
                { RF_STAT_BEGIN();
                if (!mbar_wait(tmem_full_bar(buf), bph, p.status, kErrEpilogueWait)) { ok = false; break; }
                RF_STAT_END(w_acc); }
                tc_fence_after();
                // The MMAs that wrote this buffer have finished reading their smem stage.
                if (ew == 0 && lane == 0) mbar_arrive(empty_bar(it % STAGES));
                const uint32_t taddr = lane_addr + buf * BN + grp * CPT;
                constexpr int NCH = CPT / 32;
                float v[2][32];
                tmem_ld32_async(taddr, v[0]);
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    tmem_ld_fence(v[c & 1]);   // waits for every load issued so far
                    if (c + 1 < NCH) {
                        tmem_ld32_async(taddr + (c + 1) * 32, v[(c + 1) & 1]);   // overlaps the FMAs below
                    } else {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tmem_empty_bar(buf));
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        acc[c * 16 + j] =
                            __ffma2_rn(make_float2(v[c & 1][2 * j], v[c & 1][2 * j + 1]), s2, acc[c * 16 + j]);
                }
            }
            if (!ok) break;

            // Tile store: each warp stages its 32 rows x 128 bytes in its own swizzled
            // shared-memory slab and one lane hands the slab to the TMA, which writes
            // full 128-byte row segments and clips rows >= m / columns >= n.
            {
                const uint32_t slab = slab_base + ew * Cfg::kSlabBytes;
                const uint32_t my_row = slab + lane * 128;
                const int slab_row0 = t.m_blk * BM + quad * 32;
                if (p.splits == 1) {
#pragma unroll
                    for (int ch = 0; ch < CPT / 64; ++ch) {
                        if (col0 + ch * 64 >= p.n) break;
                        if (lane == 0) tma_store_wait_read<0>();   // previous store has drained the slab
                        __syncwarp();
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const int a0 = ch * 32 + j * 4;
                            st_shared_v4(my_row + ((j ^ (lane & 7)) << 4),
                                         pack_bf16x2(acc[a0 + 0].x, acc[a0 + 0].y), pack_bf16x2(acc[a0 + 1].x, acc[a0 + 1].y),
                                         pack_bf16x2(acc[a0 + 2].x, acc[a0 + 2].y), pack_bf16x2(acc[a0 + 3].x, acc[a0 + 3].y));
                        }
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            if (p.n_dest <= 1) {
                                tma_store_2d(&tma_c, slab, col0 + ch * 64, slab_row0);
                            } else {
                                // N-split GEMM: the slab goes to every GPU's C (own memory and peers over
                                // NVLink), which is the all-gather of C done by the epilogue itself
                                for (int dd = 0; dd < p.n_dest; ++dd)
                                    tma_store_2d(&dests.m[dd], slab, p.c_col_offset + col0 + ch * 64, slab_row0);
                            }
                            tma_store_commit();
                        }
                    }
                } else {
#pragma unroll
                    for (int ch = 0; ch < CPT / 32; ++ch) {
                        if (col0 + ch * 32 >= p.n) break;
                        if (lane == 0) tma_store_wait_read<0>();
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
                            tma_store_3d(&tma_p, slab, col0 + ch * 32, slab_row0, t.split);
                            tma_store_commit();
                        }
                    }
                }
            }
        }
        if (lane == 0) tma_store_wait_all<0>();   // all of this warp's stores are complete before exit
#ifdef RF_WAIT_STATS
        if (warp == NUM_NON_EPI_WARPS && lane == 0) {
            RF_STAT_FLUSH(3, w_acc);
            RF_STAT_FLUSH(4, clock64() - t_begin);
        }
#endif
    }

    // ------------------------------------------------------------- tear-down
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// C = bf16( sum_s partial[s] )  -  split-K fix-up (reference: reduce_kernel,
// src/gemm/gemm_kernel.cpp:288-303).  One float4 per thread per slice.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ c, size_t mn, int splits) {
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

using Cfg128 = GemmCfg<128, 6>;
using Cfg256 = GemmCfg<256, 4>;

template <class Cfg>
cudaError_t launch_cfg(const CUtensorMap& tma_a, const CUtensorMap& tma_b, const CUtensorMap& tma_c,
                       const CUtensorMap& tma_p, const GemmDestMaps& dests, const GemmParams& p, int num_sms,
                       cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = fp8_gemm_kernel<Cfg>;
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    const int total = p.tiles_m * p.tiles_n * p.splits;
    const int grid = total < num_sms ? total : num_sms;
    kernel<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(tma_a, tma_b, tma_c, tma_p, dests, p);
    return cudaGetLastError();
}

}  // namespace

#ifdef RF_WAIT_STATS
extern "C" void rf_debug_wait_stats(unsigned long long* out8, int reset) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out8, g_wait_stats, sizeof(unsigned long long) * 8);
    if (reset) {
        unsigned long long z[8] = {};
        cudaMemcpyToSymbol(g_wait_stats, z, sizeof(z));
    }
}
#endif

cudaError_t fp8_gemm_prepare_device() {
    cudaError_t e = cudaFuncSetAttribute(fp8_gemm_kernel<Cfg128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg128::kSmemBytes);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(fp8_gemm_kernel<Cfg256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                Cfg256::kSmemBytes);
}

cudaError_t fp8_gemm_launch(const CUtensorMap& tma_a, const CUtensorMap& tma_b, const CUtensorMap& tma_c,
                            const CUtensorMap& tma_p, const GemmDestMaps* dests, const GemmParams& p, int block_n,
                            int num_sms, cudaStream_t stream) {
    GemmDestMaps local;
    if (!dests) {
        for (int i = 0; i < 8; ++i) local.m[i] = tma_c;
        dests = &local;
    }
    cudaError_t e = block_n == 256 ? launch_cfg<Cfg256>(tma_a, tma_b, tma_c, tma_p, *dests, p, num_sms, stream)
                                   : launch_cfg<Cfg128>(tma_a, tma_b, tma_c, tma_p, *dests, p, num_sms, stream);
    if (e != cudaSuccess) return e;
    if (p.splits > 1) {
        const size_t mn = (size_t)p.m * p.n;
        const unsigned blocks = (unsigned)((mn / 4 + 255) / 256);
        splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(p.partial, p.c, mn, p.splits);
        e = cudaGetLastError();
    }
    return e;
}

}  // namespace rf
