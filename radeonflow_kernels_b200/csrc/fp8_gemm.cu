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
//               (K = 32 each) into one of two TMEM accumulator buffers, then
//               tcgen05.commit to free the smem stage and publish the buffer
//   warps 4..   epilogue: tcgen05.ld the K block's fp32 partial sums, scale by
//               the exact fp32 product a_s*b_s and add into a register
//               accumulator while the next K block's MMAs run in the other
//               TMEM buffer; finally round to bf16 (or store fp32 split-K slices)
//
// The scales are arbitrary fp32 numbers, so the hardware block-scaled MMA
// (ue8m0 scales) cannot be used; promotion is one FMA per element per K block,
// exactly the ratio of the reference's `frag_r += s * frag_c`
// (src/gemm/gemm_kernel.cpp:173-207).
#include "ptx.cuh"
#include "fp8_gemm.h"

#include <cstdio>

namespace rf {

namespace {

constexpr int BM = 128;
constexpr int BK = 128;          // one scale block, one 128-byte swizzle row of fp8
constexpr int UMMA_K = 32;       // K per tcgen05.mma for 8-bit operands
constexpr int NUM_NON_EPI_WARPS = 4;

template <int BN, int STAGES, int EPI_GROUPS>
struct GemmCfg {
    static constexpr int kBN = BN;
    static constexpr int kStages = STAGES;
    static constexpr int kEpiGroups = EPI_GROUPS;              // column groups, 4 warps each
    static constexpr int kColsPerThread = BN / EPI_GROUPS;
    static constexpr int kEpiWarps = 4 * EPI_GROUPS;
    static constexpr int kThreads = 32 * (NUM_NON_EPI_WARPS + kEpiWarps);
    static constexpr int kABytes = BM * BK;
    static constexpr int kBBytes = BN * BK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemCols = 2 * BN;                  // two accumulator buffers
    static constexpr int kBarBytes = (2 * STAGES + 4) * 8 + 16;
    static constexpr int kSmemBytes = STAGES * kStageBytes + kBarBytes + 1024;  // + alignment slack
    static_assert(kColsPerThread % 32 == 0, "epilogue loads 32 columns at a time");
    static_assert(kColsPerThread <= 128, "a thread's columns must share one 128-wide scale block");
    static_assert(kTmemCols == 256 || kTmemCols == 512 || kTmemCols == 128, "TMEM columns: power of two");
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
                const GemmParams p) {
    constexpr int BN = Cfg::kBN;
    constexpr int STAGES = Cfg::kStages;
    constexpr int CPT = Cfg::kColsPerThread;

    extern __shared__ uint8_t smem_raw[];
    // 128-byte-swizzled tiles need 1024-byte alignment.
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + STAGES * Cfg::kStageBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tmem_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
    auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);
    uint32_t* tmem_slot_ptr =
        reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tma_a);
        tma_prefetch_desc(&tma_b);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
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

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;  // running K-block counter across work items
            bool ok = true;
            for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
                const TileCoord t = decode_work(w, p.tiles_m, p.tiles_n, p.splits);
                const int kb0 = (int)((long long)kb_total * t.split / p.splits);
                const int kb1 = (int)((long long)kb_total * (t.split + 1) / p.splits);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(empty_bar(s), ph ^ 1, p.status, kErrProducerWait)) { ok = false; break; }
                    mbar_expect_tx(full_bar(s), Cfg::kStageBytes);
                    const uint32_t sa = smem_base + s * Cfg::kStageBytes;
                    tma_load_2d(sa, &tma_a, full_bar(s), kb * BK, t.m_blk * BM);
                    tma_load_2d(sa + Cfg::kABytes, &tma_b, full_bar(s), kb * BK, t.n_blk * BN);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN, /*e4m3*/ 0, /*e4m3*/ 0, 0, 0);
            uint32_t it = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
                const TileCoord t = decode_work(w, p.tiles_m, p.tiles_n, p.splits);
                const int kb0 = (int)((long long)kb_total * t.split / p.splits);
                const int kb1 = (int)((long long)kb_total * (t.split + 1) / p.splits);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    const int buf = it & 1;
                    const uint32_t bph = (it >> 1) & 1;
                    if (!mbar_wait(tmem_empty_bar(buf), bph ^ 1, p.status, kErrMmaWaitTmem)) { ok = false; break; }
                    if (!mbar_wait(full_bar(s), ph, p.status, kErrMmaWaitFull)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_base + s * Cfg::kStageBytes;
                    const uint64_t adesc = smem_desc_kmajor_sw128(sa);
                    const uint64_t bdesc = smem_desc_kmajor_sw128(sa + Cfg::kABytes);
                    const uint32_t d = tmem_base + buf * BN;
#pragma unroll
                    for (int j = 0; j < BK / UMMA_K; ++j) {
                        // +32 bytes along K inside the swizzled row = +2 in the (addr >> 4) field
                        umma_f8(d, adesc + 2 * j, bdesc + 2 * j, idesc, j > 0 ? 1u : 0u);
                    }
                    umma_commit(empty_bar(s));        // smem stage reusable once the MMAs have read it
                    umma_commit(tmem_full_bar(buf));  // accumulator buffer ready for the epilogue
                }
            }
        }
        __syncwarp();
    } else if (warp >= NUM_NON_EPI_WARPS) {
        // ---------------------------------------------------------- epilogue
        const int ew = warp - NUM_NON_EPI_WARPS;
        const int quad = warp & 3;            // TMEM lane quadrant this warp may access
        const int grp = ew >> 2;              // column group
        const int row_in_tile = quad * 32 + lane;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
        const int kbs = p.k / BK;
        uint32_t it = 0;
        bool ok = true;
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

            float acc[CPT];
#pragma unroll
            for (int j = 0; j < CPT; ++j) acc[j] = 0.f;

            float s_next = __ldg(as_row + kb0) * __ldg(bs_row + kb0);
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                const float s = s_next;
                if (kb + 1 < kb1) s_next = __ldg(as_row + kb + 1) * __ldg(bs_row + kb + 1);
                const int buf = it & 1;
                const uint32_t bph = (it >> 1) & 1;
                if (!mbar_wait(tmem_full_bar(buf), bph, p.status, kErrEpilogueWait)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < CPT / 32; ++c) {
                    float v[32];
                    tmem_ld32(lane_addr + buf * BN + grp * CPT + c * 32, v);
                    if (c == CPT / 32 - 1) {
                        // all of this warp's reads of the buffer are complete
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tmem_empty_bar(buf));
                    }
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[c * 32 + j] = fmaf(s, v[j], acc[c * 32 + j]);
                }
            }
            if (!ok) break;

            if (row_ok) {
                if (p.splits == 1) {
                    __nv_bfloat16* crow = p.c + (size_t)row * p.n + col0;
#pragma unroll
                    for (int j = 0; j < CPT; j += 8) {
                        if (col0 + j < p.n) {
                            uint4 q;
                            q.x = pack_bf16x2(acc[j + 0], acc[j + 1]);
                            q.y = pack_bf16x2(acc[j + 2], acc[j + 3]);
                            q.z = pack_bf16x2(acc[j + 4], acc[j + 5]);
                            q.w = pack_bf16x2(acc[j + 6], acc[j + 7]);
                            *reinterpret_cast<uint4*>(crow + j) = q;
                        }
                    }
                } else {
                    float* prow = p.partial + ((size_t)t.split * p.m + row) * p.n + col0;
#pragma unroll
                    for (int j = 0; j < CPT; j += 4) {
                        if (col0 + j < p.n) {
                            *reinterpret_cast<float4*>(prow + j) =
                                make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
                        }
                    }
                }
            }
        }
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

using Cfg128 = GemmCfg<128, 6, 2>;

}  // namespace

size_t fp8_gemm_smem_bytes() { return Cfg128::kSmemBytes; }
int fp8_gemm_block_n() { return Cfg128::kBN; }

cudaError_t fp8_gemm_launch(const CUtensorMap& tma_a, const CUtensorMap& tma_b, const GemmParams& p, int num_sms,
                            cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = fp8_gemm_kernel<Cfg128>;
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg128::kSmemBytes);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    const int total = p.tiles_m * p.tiles_n * p.splits;
    const int grid = total < num_sms ? total : num_sms;
    kernel<<<grid, Cfg128::kThreads, Cfg128::kSmemBytes, stream>>>(tma_a, tma_b, p);
    cudaError_t e = cudaGetLastError();
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
