// Grouped fp16 GEMM for the MoE layer on sm_100a: per-expert row ranges, no padding rows.
//
// Replaces the hipBLASLt grouped / dense GEMM calls and the separate SwiGLU pass of the reference
// (src/moe/gemm_thirdparty.cpp:65-115, :261-288; src/moe/moe_gemm_pipeline_kernel.cpp:377-405), and
// the PyTorch router matmul (scripts/gen_submission.py:400).
//
// A work item is (128-row tile of one group, block of output columns).  Row tiles come from a
// device-built list (tile_list_kernel), so per-expert counts never visit the host.  One persistent
// CTA per SM, warp-specialised like the FP8 GEMM:
//   warp 0     TMA producer: A tile [128 x 64] fp16 (K-major, 128-byte swizzle) and B as four
//              [64 K-rows x 64 N] boxes of the row-major weight (MN-major operand, 128-byte swizzle);
//              in SwiGLU mode two boxes come from W_gate and two from W_up at the same columns
//              (SwiGLU mode with a row map: warps 2 and 3 gather the A rows from the token matrix with 16-byte
//              cp.async copies into the same swizzled layout, and the TMA loads only B)
//   warp 1     MMA issuer: 4 x tcgen05.mma.kind::f16 (128 x 256 x 16) per stage, accumulating the
//              whole K range in one of two 256-column TMEM buffers; one commit per stage frees the
//              shared-memory stage, one per tile publishes the accumulator
//   warps 4-11 epilogue of the previous tile while the next tile's MMAs run: tcgen05.ld, fp16
//              rounding (SwiGLU: SiLU(fp16 G) * fp16 U), rows past the group's end masked
// Rows of a tile beyond its group's range belong to the next group: they are computed and dropped.
#include "ptx.cuh"
#include "moe_kernels.h"

namespace rf {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;          // MMA N, TMEM columns per accumulator buffer
constexpr int BK = 64;           // 128 bytes of fp16: one swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;        // 16 KB
constexpr int B_BYTES = BN * BK * 2;        // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int B_BOX_BYTES = 64 * BK * 2;    // one [64 K x 64 N] box: 8 KB
constexpr int NUM_NON_EPI_WARPS = 4;
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 32 * (NUM_NON_EPI_WARPS + EPI_WARPS);
constexpr int SLAB_BYTES = 32 * 128;
constexpr int NBUF = 2;
constexpr int GATHER_THREADS = 64;   // warps 2 and 3
constexpr int GATHER_LAG = 2;        // cp.async groups a gather thread keeps in flight
constexpr int TMEM_COLS = NBUF * BN;
constexpr int BAR_BYTES = (2 * STAGES + 2 * NBUF) * 8 + 16;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_WARPS * SLAB_BYTES + BAR_BYTES + 1024;

__device__ __forceinline__ float silu_fp16_rounded(float g) {
    // SiLU evaluated in fp32 on an fp16 input, result rounded to fp16 (scripts/problems/moe/reference.py:23)
    const float s = g / (1.0f + __expf(-g));
    return __half2float(__float2half_rn(s));
}

// Work item -> (row tile, column block).  Items walk one chunk (up to kMoeChunkTiles row tiles of one
// group, built by tile_list_kernel) for one column block, then the next column block of the same chunk:
// the CTAs running at the same time share that group's weight column block, and the chunk's A tiles stay
// in L2 across all column blocks.  The chunk of work item w is the chunk of tile w / nbn, because the
// chunks before it hold exactly (first tile of the chunk) * nbn items.
__device__ __forceinline__ void decode_item(int w, const int* __restrict__ tile_chunk, int nbn, int* tile, int* nb) {
    const int info = __ldg(tile_chunk + w / nbn);
    const int first = info >> 8;
    const int rows = info & 0xff;
    const int r = w - first * nbn;
    *nb = r / rows;
    *tile = first + r % rows;
}

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1)
moe_gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_out,
                const MoeGemmParams p) {
    constexpr bool SWIGLU = MODE == kMoeGemmSwiglu;
    constexpr bool ROUTER = MODE == kMoeGemmRouter;
    constexpr int TILE_N = SWIGLU ? 128 : 256;     // output columns per work item

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t slab_base = smem_base + STAGES * STAGE_BYTES;
    const uint32_t bar_base = slab_base + EPI_WARPS * SLAB_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tmem_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
    auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + NBUF + b); };
    const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 2 * NBUF);
    uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // gathered A rows: the stage is full when the TMA's B bytes have landed AND every gather thread has arrived
    const bool gather = SWIGLU && p.gather_map != nullptr;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tma_a);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), gather ? 1 + GATHER_THREADS : 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < NBUF; ++b) {
            mbar_init(tmem_full_bar(b), 1);
            mbar_init(tmem_empty_bar(b), EPI_WARPS);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot_ptr);

    const int n_tiles = __ldg(p.tile_count);
    const int nbn = (p.n_out + TILE_N - 1) / TILE_N;
    const int total_work = n_tiles * nbn;
    const int k_steps = p.k / BK;

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        uint32_t it = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
            int tile, nb_i;
            decode_item(w, p.tile_chunk, nbn, &tile, &nb_i);
            const int n0 = nb_i * TILE_N;
            const int row0 = __ldg(p.tile_row0 + tile);
            const int grp = __ldg(p.tile_group + tile);
            const CUtensorMap* mb = p.b_maps + grp;
            const CUtensorMap* mb2 = SWIGLU ? p.b2_maps + grp : mb;
            for (int ks = 0; ks < k_steps; ++ks, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                ok = __all_sync(0xffffffffu, mbar_wait(empty_bar(s), ph ^ 1, p.status, kErrProducerWait, p.launch_tag));
                if (!ok) break;
                if (elect_one()) {
                    mbar_expect_tx(full_bar(s), gather ? B_BYTES : STAGE_BYTES);
                    const uint32_t sa = smem_base + s * STAGE_BYTES;
                    const uint32_t sb = sa + A_BYTES;
                    if (!gather) tma_load_2d(sa, &tma_a, full_bar(s), ks * BK, row0);
                    if (ROUTER) {
                        // B [N, K] row-major: one box of 256 rows (N) x 64 K
                        tma_load_2d(sb, mb, full_bar(s), ks * BK, n0);
                    } else if (SWIGLU) {
                        tma_load_2d(sb + 0 * B_BOX_BYTES, mb, full_bar(s), n0, ks * BK);
                        tma_load_2d(sb + 1 * B_BOX_BYTES, mb, full_bar(s), n0 + 64, ks * BK);
                        tma_load_2d(sb + 2 * B_BOX_BYTES, mb2, full_bar(s), n0, ks * BK);
                        tma_load_2d(sb + 3 * B_BOX_BYTES, mb2, full_bar(s), n0 + 64, ks * BK);
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            tma_load_2d(sb + j * B_BOX_BYTES, mb, full_bar(s), n0 + 64 * j, ks * BK);
                    }
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        constexpr uint32_t idesc = make_idesc(BM, BN, /*f16*/ 0, /*f16*/ 0, 0, ROUTER ? 0 : 1);
        uint32_t it = 0, tcount = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x, ++tcount) {
            const int buf = tcount & 1;
            const uint32_t bph = (tcount >> 1) & 1;
            ok = __all_sync(0xffffffffu, mbar_wait(tmem_empty_bar(buf), bph ^ 1, p.status, kErrMmaWaitTmem, p.launch_tag));
            if (!ok) break;
            const uint32_t d = tmem_base + buf * BN;
            for (int ks = 0; ks < k_steps; ++ks, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                ok = __all_sync(0xffffffffu, mbar_wait(full_bar(s), ph, p.status, kErrMmaWaitFull, p.launch_tag));
                if (!ok) break;
                tc_fence_after();
                const uint32_t sa = smem_base + s * STAGE_BYTES;
                const uint64_t adesc = smem_desc_kmajor_sw128(sa);
                const uint64_t bdesc = ROUTER ? smem_desc_kmajor_sw128(sa + A_BYTES)
                                              : smem_desc_mnmajor_sw128(sa + A_BYTES, B_BOX_BYTES, 1024);
                if (elect_one()) {
#pragma unroll
                    for (int j = 0; j < BK / UMMA_K; ++j) {
                        // A and K-major B: +32 bytes along K; MN-major B: +16 K-rows = +2048 bytes
                        const uint64_t bd = bdesc + (ROUTER ? 2 * j : 128 * j);
                        umma_f16(d, adesc + 2 * j, bd, idesc, (ks > 0 || j > 0) ? 1u : 0u);
                    }
                    umma_commit(empty_bar(s));
                    if (ks == k_steps - 1) umma_commit(tmem_full_bar(buf));
                }
                __syncwarp();
            }
        }
    } else if (warp < NUM_NON_EPI_WARPS) {
        // ------------------------------------------------- A-row gather (warps 2, 3)
        // 8 lanes per 128-byte row segment, so every copy instruction of a warp reads four whole 128-byte
        // segments of four token rows and writes four whole rows of the swizzled tile.  A thread keeps
        // GATHER_LAG groups in flight; when a group has landed it makes the bytes visible to the tensor core's
        // proxy and arrives on the stage's barrier.
        if (gather) {
            const int tg = threadIdx.x - 64;            // 0..63
            const int c8 = tg & 7, rsub = tg >> 3;      // 16-byte piece of the segment; row within a group of 8
            const __half* xsrc = static_cast<const __half*>(p.gather_src);
            uint32_t it = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
                int tile, nb_i;
                decode_item(w, p.tile_chunk, nbn, &tile, &nb_i);
                const int row0 = __ldg(p.tile_row0 + tile);
                int tok[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int r = min(row0 + i * 8 + rsub, p.gather_rows - 1);
                    tok[i] = __ldg(p.gather_map + r) % p.gather_mod;
                }
                for (int ks = 0; ks < k_steps; ++ks) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(empty_bar(s), ph ^ 1, p.status, kErrProducerWait, p.launch_tag)) { ok = false; break; }
                    const uint32_t sa = smem_base + s * STAGE_BYTES;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int r = i * 8 + rsub;     // r & 7 == rsub
                        cp_async_16(sa + r * 128 + ((c8 ^ rsub) << 4),
                                    xsrc + (size_t)tok[i] * p.k + ks * BK + c8 * 8);
                    }
                    cp_async_commit();
                    ++it;
                    if (it > GATHER_LAG) {
                        cp_async_wait<GATHER_LAG>();
                        fence_proxy_async_smem();
                        mbar_arrive(full_bar((it - 1 - GATHER_LAG) % STAGES));
                    }
                }
            }
            // drain: the last groups, oldest first (also after a wait gave up: no copy may outlive the CTA)
            cp_async_wait<1>();
            if (ok && it >= 2) { fence_proxy_async_smem(); mbar_arrive(full_bar((it - 2) % STAGES)); }
            cp_async_wait<0>();
            if (ok && it >= 1) { fence_proxy_async_smem(); mbar_arrive(full_bar((it - 1) % STAGES)); }
        }
    } else {
        // ---------------------------------------------------------- epilogue
        const int ew = warp - NUM_NON_EPI_WARPS;
        const int quad = warp & 3;
        const int grp_c = ew >> 2;                         // column group 0/1
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
        const uint32_t slab = slab_base + ew * SLAB_BYTES;
        const uint32_t my_row = slab + lane * 128;
        __half* out = static_cast<__half*>(p.out);
        uint32_t tcount = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x, ++tcount) {
            int tile, nb_i;
            decode_item(w, p.tile_chunk, nbn, &tile, &nb_i);
            const int n0 = nb_i * TILE_N;
            const int row0 = __ldg(p.tile_row0 + tile);
            const int grp = __ldg(p.tile_group + tile);
            const int row_end = __ldg(p.group_offsets + grp + 1);
            const int buf = tcount & 1;
            const uint32_t bph = (tcount >> 1) & 1;
            if (!mbar_wait(tmem_full_bar(buf), bph, p.status, kErrEpilogueWait, p.launch_tag)) { ok = false; break; }
            tc_fence_after();

            const int slab_row0 = row0 + quad * 32;
            const int rows_valid = row_end - slab_row0;          // <= 0: nothing to store
            const bool full_slab = rows_valid >= 32;
            const bool my_row_ok = lane < rows_valid;
            const uint32_t tbase = lane_addr + buf * BN;
            // scatter mode: this thread's row goes to a row of another (or this) GPU's matrix
            const bool scatter = MODE == kMoeGemmPlain && p.scatter_meta != nullptr;
            __half* scatter_row = nullptr;
            if (scatter && my_row_ok) {
                const int meta = __ldg(p.scatter_meta + slab_row0 + lane);
                scatter_row = static_cast<__half*>(pick_peer(p.scatter_dst, meta >> kEpMetaSlotBits)) +
                              (size_t)(meta & ((1 << kEpMetaSlotBits) - 1)) * p.n_out;
            }

            // 64 output columns (one 128-byte slab row) per iteration
            constexpr int OUT_COLS = SWIGLU ? 64 : 128;          // per epilogue warp
#pragma unroll 1
            for (int c64 = 0; c64 < OUT_COLS; c64 += 64) {
                const int out_col = n0 + grp_c * OUT_COLS + c64;
                uint32_t packed[32];                              // 64 fp16 values of this thread's row
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float v[32];
                    if (SWIGLU) {
                        float u[32];
                        tmem_ld32_async(tbase + grp_c * 64 + c64 + h * 32, v);          // gate columns
                        tmem_ld32_async(tbase + 128 + grp_c * 64 + c64 + h * 32, u);    // up columns
                        tmem_ld_fence(v);
                        tmem_ld_fence(u);
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float g16 = __half2float(__float2half_rn(v[j]));
                            const float u16 = __half2float(__float2half_rn(u[j]));
                            v[j] = silu_fp16_rounded(g16) * u16;
                        }
                    } else {
                        tmem_ld32_async(tbase + grp_c * 128 + c64 + h * 32, v);
                        tmem_ld_fence(v);
                        if (ROUTER && p.bias != nullptr) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const int col = out_col + h * 32 + j;
                                v[j] += col < p.n_out ? __ldg(p.bias + col) : 0.f;
                            }
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) packed[h * 16 + j] = pack_f16x2(v[2 * j], v[2 * j + 1]);
                }
                if (out_col >= p.n_out || rows_valid <= 0) continue;
                if (scatter) {
                    // Through the warp's slab, so that every store instruction writes four whole 128-byte
                    // row segments (8 lanes each) instead of 32 scattered 16-byte pieces: over NVLink the
                    // payload per transaction decides the bandwidth.
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        st_shared_v4(my_row + ((j ^ (lane & 7)) << 4), packed[4 * j], packed[4 * j + 1],
                                     packed[4 * j + 2], packed[4 * j + 3]);
                    __syncwarp();
                    const int c = lane & 7;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int r = 4 * i + (lane >> 3);
                        const unsigned long long base =
                            __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(scatter_row), r);
                        const uint4 v = ld_shared_v4(slab + r * 128 + ((c ^ (r & 7)) << 4));
                        if (r < rows_valid)
                            *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(base) + out_col + 8 * c) = v;
                    }
                } else if (p.tma_store && full_slab) {
                    if (lane == 0) tma_store_wait_read<0>();
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        st_shared_v4(my_row + ((j ^ (lane & 7)) << 4), packed[4 * j], packed[4 * j + 1],
                                     packed[4 * j + 2], packed[4 * j + 3]);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&tma_out, slab, out_col, slab_row0);
                        tma_store_commit();
                    }
                } else if (my_row_ok) {
                    __half* orow = out + (size_t)(slab_row0 + lane) * p.n_out + out_col;
                    if (out_col + 64 <= p.n_out && (p.n_out % 8) == 0) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            *reinterpret_cast<uint4*>(orow + 8 * j) =
                                make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                    } else {
                        // ragged column tail (router with few experts): element stores, fully unrolled
                        // so `packed` stays in registers
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const __half2 hv = *reinterpret_cast<const __half2*>(&packed[j]);
                            if (out_col + 2 * j < p.n_out) orow[2 * j] = __low2half(hv);
                            if (out_col + 2 * j + 1 < p.n_out) orow[2 * j + 1] = __high2half(hv);
                        }
                    }
                }
            }
            // every TMEM read of this buffer by this warp has completed (loads are fenced above)
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tmem_empty_bar(buf));
        }
        if (lane == 0) tma_store_wait_read<0>();   // the slab has been read; the writes complete with the grid
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int MODE>
cudaError_t launch_mode(const CUtensorMap& tma_a, const CUtensorMap& tma_out, const MoeGemmParams& p, int num_sms,
                        cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kernel = moe_gemm_kernel<MODE>;
    if (dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    kernel<<<num_sms, THREADS, SMEM_BYTES, stream>>>(tma_a, tma_out, p);
    return cudaGetLastError();
}

}  // namespace

int moe_gemm_tile_n(int mode) { return mode == kMoeGemmSwiglu ? 128 : 256; }

cudaError_t moe_gemm_launch(int mode, const CUtensorMap& tma_a, const CUtensorMap& tma_out, const MoeGemmParams& p,
                            int num_sms, cudaStream_t stream) {
    switch (mode) {
        case kMoeGemmPlain: return launch_mode<kMoeGemmPlain>(tma_a, tma_out, p, num_sms, stream);
        case kMoeGemmSwiglu: return launch_mode<kMoeGemmSwiglu>(tma_a, tma_out, p, num_sms, stream);
        case kMoeGemmRouter: return launch_mode<kMoeGemmRouter>(tma_a, tma_out, p, num_sms, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace rf
