// C-ABI entry points of the FP8 block-scaled GEMM (declared in include/rf_b200.h).
#include "../../include/rf_b200.h"
#include "fp8_gemm.h"
#include "host_util.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace {

constexpr int kBlockK = 128;
constexpr int kMaxSplits = 64;     // K slices per GEMM (the kernel's 32-bit K-range arithmetic relies on it)

bool shape_ok(int m, int n, int k) { return m > 0 && n > 0 && k > 0 && (n % 64) == 0 && (k % kBlockK) == 0; }

// Tuning knob for experiments: RF_FP8_GEMM_BN=128|256|384|512 forces the tile configuration (512 / 384 = CTA
// pairs with 256 x 256 / 256 x 128 tiles).
int forced_block_n() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("RF_FP8_GEMM_BN");
        v = e ? atoi(e) : 0;
        if (v != 128 && v != 256 && v != 384 && v != 512) v = 0;
    }
    return v;
}

// The CTA-pair configuration (cta_group::2, 256 x 256 per 2-CTA cluster) is correct and selectable
// (RF_FP8_GEMM_BN=512, or RF_FP8_GEMM_PAIR=1 to let the planner consider it) but is not chosen by
// default: measured on B200 it runs 6144x4608x7168 at 2.05 PFLOP/s against 2.2 for the one-CTA 128 x 256
// tile, because the per-K-block accumulator hand-off, not shared-memory bandwidth, bounds both.
bool pair_config_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("RF_FP8_GEMM_PAIR");
        v = (e && atoi(e) == 1) ? 1 : 0;
    }
    return v == 1;
}

// splits: K slices (1 = none), or kStreamK: one pass whose ragged last wave is shared out by K blocks.
constexpr int kStreamK = -1;

struct GemmPlan {
    int block_n;
    int splits;
    double cost;
};

// RF_FP8_GEMM_STREAMK=1 makes every automatic plan whose tiles do not fill whole waves a stream-K plan, =0 never
// uses stream-K; unset, the tuned table and the cost model decide.
int streamk_override() {
    static int v = -2;
    if (v == -2) {
        const char* e = getenv("RF_FP8_GEMM_STREAMK");
        v = e ? (atoi(e) != 0 ? 1 : 0) : -1;
    }
    return v;
}

// Tiles of the stream-K region of this launch, 0 = the plan runs as a plain pass.
int streamk_region(int m, int n, int k, int bn, int num_sms) {
    if (rf::gemm_is_pair(bn)) return 0;
    const int tiles = ((m + 127) / 128) * ((n + bn - 1) / bn);
    const int sk = rf::gemm_streamk_tiles(tiles, num_sms);
    // shares shorter than two K blocks are all fix-up and no work
    if (sk > 0 && (long long)sk * (k / kBlockK) < 2LL * num_sms) return 0;
    return sk;
}

// Cost model, in units of one 128-deep K block of a 128 x 128 tile at full tensor rate
// (about 0.14 us): rounds of tiles over the SMs x (K blocks per slice + fixed per-tile cost),
// plus, for split-K, the fp32 slice round trip through HBM and the second launch.
GemmPlan plan_for(int m, int n, int k, int num_sms, int bn, int forced_split) {
    const int tr = rf::gemm_tile_rows(bn), tc = rf::gemm_tile_cols(bn);
    const int tiles = ((m + tr - 1) / tr) * ((n + tc - 1) / tc);
    const int kb = k / kBlockK;
    if (rf::gemm_is_pair(bn)) num_sms /= 2;     // work items go to CTA pairs
    // relative time of one K block of one work item, from in-kernel cycle counts
    // (128 x 128: ~620 cycles, 128 x 256: ~790, CTA pair 256 x 256: ~925)
    const double tile_w = bn == 512 ? 1.5 : (bn == 256 ? 1.25 : (bn == 384 ? 0.8 : 1.0));
    GemmPlan best{bn, 1, 1e30};
    for (int s = 1; s <= 8; ++s) {
        if (forced_split > 0 && s != forced_split) continue;
        if (forced_split <= 0 && s > 1 && (kb / s < 4 || tiles >= num_sms)) break;
        if (s > kb) break;
        const int rounds = (tiles * s + num_sms - 1) / num_sms;
        const int kb_per = (kb + s - 1) / s;
        double cost = (double)rounds * (kb_per * tile_w + 4.0);
        if (s > 1) {
            const double bytes = 8.0 * s * (double)m * n + 2.0 * (double)m * n;
            cost += (bytes / 6.0e12 + 2.5e-6) / 0.14e-6;
        }
        if (cost < best.cost) best = GemmPlan{bn, s, cost};
    }
    if (best.cost > 1e29) best = GemmPlan{bn, forced_split > kb ? kb : (forced_split > 0 ? forced_split : 1), 0};
    return best;
}

GemmPlan choose_plan_inner(int m, int n, int k, int num_sms, int forced_split) {
    const int fb = forced_block_n();
    if (fb) return plan_for(m, n, k, num_sms, fb, forced_split);
    // a measured entry for this exact shape beats the model (the caller's explicit split still wins)
    int tbn = 0, tsplits = 0;
    if (forced_split <= 0 && rf::tuned_plan_lookup(m, n, k, &tbn, &tsplits)) return GemmPlan{tbn, tsplits, 0.0};
    GemmPlan p128 = plan_for(m, n, k, num_sms, 128, forced_split);
    GemmPlan p256 = plan_for(m, n, k, num_sms, 256, forced_split);
    // Wide tiles halve the A traffic and the MMA instruction count per FLOP; prefer them unless
    // they cost noticeably more rounds (ragged N such as 576, or too few tiles).
    GemmPlan best = p256.cost <= p128.cost * 1.02 ? p256 : p128;
    if (pair_config_enabled()) {
        GemmPlan pp = plan_for(m, n, k, num_sms, 512, forced_split);
        if (pp.cost < best.cost) best = pp;
    }
    // Stream-K instead of a plain single pass, in K blocks of the chosen tile: a plain pass takes
    // rounds x (kb + per-tile cost), a stream-K pass the even share of all K blocks plus its fixed cost (slot
    // write, slot read, one more piece per CTA: 7-11 us measured on B200, about 18 K blocks of a 128 x 256 tile).
    // That pays when a long-K shape has just over a whole number of waves (160 tiles of 56 K blocks: 2 x 56
    // against 60.5 + 18); none of the 18 benchmark shapes is such a shape.
    if (forced_split == 0 && best.splits == 1 && !rf::gemm_is_pair(best.block_n) &&
        streamk_region(m, n, k, best.block_n, num_sms) > 0) {
        const int kb = k / kBlockK;
        const int tiles = ((m + 127) / 128) * ((n + best.block_n - 1) / best.block_n);
        const int rounds = (tiles + num_sms - 1) / num_sms;
        const double plain = (double)rounds * (kb + 3.0);
        const double shared = (double)tiles * kb / num_sms + 3.0 * (tiles / num_sms + 1) + 18.0;
        if (shared < plain) best.splits = kStreamK;
    }
    return best;
}

// forced_split: > 0 = that many K slices, kStreamK = stream-K, 0 = the library's choice.
GemmPlan choose_plan(int m, int n, int k, int num_sms, int forced_split) {
    GemmPlan plan = choose_plan_inner(m, n, k, num_sms, forced_split == kStreamK ? 1 : forced_split);
    if (forced_split == kStreamK) plan.splits = kStreamK;
    if (forced_split == 0) {
        const int ov = streamk_override();
        if (ov == 1) {
            if (plan.splits != kStreamK) plan = GemmPlan{forced_block_n() ? plan.block_n : 256, kStreamK, 0.0};
        } else if (ov == 0 && plan.splits == kStreamK) {
            plan.splits = 1;
        }
    }
    // a stream-K plan that has no ragged wave to share out is a plain pass
    if (plan.splits == kStreamK && streamk_region(m, n, k, plan.block_n, num_sms) == 0) plan.splits = 1;
    return plan;
}

// `dest_c` / `n_dest` / `dest_n` / `col_offset`: when n_dest > 1 the [m, n] result is written at column
// `col_offset` of each of the n_dest row-major [m, dest_n] matrices in dest_c (N-split GEMM) and `c` is unused.
int gemm_impl(const void* a, const void* b, const float* as, const float* bs, void* c, int m, int n, int k,
              int split_k, void* workspace, size_t workspace_bytes, bool own_workspace, cudaStream_t stream,
              void* const* dest_c = nullptr, int n_dest = 1, int dest_n = 0, int col_offset = 0,
              bool mn_major = false, bool fnuz = false) {
    if (!shape_ok(m, n, k)) return RF_ERR_BAD_SHAPE;
    if (mn_major && (m % 16) != 0) return RF_ERR_BAD_SHAPE;     // [k][m] rows must be 16-byte multiples for TMA
    if (n_dest > 1) {
        if (!dest_c || n_dest > 8 || dest_n < col_offset + n || dest_n % 8 != 0 || col_offset % 64 != 0)
            return RF_ERR_BAD_SHAPE;
        for (int i = 0; i < n_dest; ++i)
            if (!dest_c[i] || ((uintptr_t)dest_c[i] & 15)) return RF_ERR_NULL_POINTER;
        c = dest_c[0];
        split_k = 1;
    }
    if (!a || !b || !as || !bs || !c) return RF_ERR_NULL_POINTER;
    if (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15) return RF_ERR_MISALIGNED;
    if (((uintptr_t)as | (uintptr_t)bs) & 3) return RF_ERR_MISALIGNED;
    rf::DeviceState* st = rf::device_state();
    if (!st) return RF_ERR_CUDA;

    const int kb = k / kBlockK;
    if (split_k > kb) split_k = kb;
    if (split_k > kMaxSplits) split_k = kMaxSplits;
    if (split_k < kStreamK) return RF_ERR_BAD_SHAPE;
    GemmPlan plan = choose_plan(m, n, k, st->num_sms, split_k);
    if (mn_major && rf::gemm_is_pair(plan.block_n)) plan = plan_for(m, n, k, st->num_sms, 256, split_k > 0 ? split_k : 0);
    // stream-K serves the row-major single-destination GEMM; elsewhere such a plan runs as a plain pass
    if (plan.splits == kStreamK && (mn_major || n_dest > 1 || rf::gemm_is_pair(plan.block_n))) plan.splits = 1;
    const int bn = plan.block_n;
    const int sk_tiles = plan.splits == kStreamK ? streamk_region(m, n, k, bn, st->num_sms) : 0;
    const int splits = plan.splits == kStreamK ? 1 : plan.splits;

    float* partial = nullptr;
    if (splits > 1 || sk_tiles > 0) {
        const size_t need = sk_tiles > 0 ? rf::gemm_streamk_bytes(bn, st->num_sms) : (size_t)splits * m * n * sizeof(float);
        if (own_workspace) {
            partial = static_cast<float*>(rf::device_scratch(need));
            if (!partial) return RF_ERR_CUDA;
        } else {
            if (!workspace || workspace_bytes < need) return RF_ERR_WORKSPACE;
            if ((uintptr_t)workspace & 15) return RF_ERR_MISALIGNED;
            partial = static_cast<float*>(workspace);
        }
    }

    CUtensorMap ta, tb;
    if (mn_major) {
        // a [k][m], b [k][n]: boxes of 128 K-rows x 128 bytes of M / N
        if (!rf::encode_tma_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, (uint64_t)k, (uint64_t)m, (uint64_t)m, 128,
                               128, true) ||
            !rf::encode_tma_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, (uint64_t)k, (uint64_t)n, (uint64_t)n, 128,
                               128, true))
            return RF_ERR_CUDA;
    } else {
        if (!rf::encode_tma_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, (uint64_t)m, (uint64_t)k, (uint64_t)k, 128,
                               128, true))
            return RF_ERR_CUDA;
        if (!rf::encode_tma_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, (uint64_t)n, (uint64_t)k, (uint64_t)k,
                               (uint32_t)rf::gemm_b_box_rows(bn), 128, true))
            return RF_ERR_CUDA;
    }

    CUtensorMap tc, tp;
    if (!rf::encode_tma_2d(&tc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, c, (uint64_t)m, (uint64_t)n, (uint64_t)n * 2, 32,
                           64, true))
        return RF_ERR_CUDA;
    if (splits > 1) {
        if (!rf::encode_tma_3d(&tp, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, partial, (uint64_t)n, (uint64_t)m,
                               (uint64_t)splits, 32, 32, true))
            return RF_ERR_CUDA;
    } else {
        tp = tc;
    }

    rf::GemmParams p;
    p.a_scale = as;
    p.b_scale = bs;
    p.c = static_cast<__nv_bfloat16*>(c);
    p.partial = partial;
    p.status = st->status;
    p.launch_tag = rf::next_launch_tag();
    p.m = m; p.n = n; p.k = k;
    p.tiles_m = (m + rf::gemm_tile_rows(bn) - 1) / rf::gemm_tile_rows(bn);
    p.tiles_n = (n + rf::gemm_tile_cols(bn) - 1) / rf::gemm_tile_cols(bn);
    p.splits = splits;
    if (mn_major) {
        p.as_row_stride = 1; p.as_k_stride = m;
        p.bs_row_stride = 1; p.bs_k_stride = (n + 127) / 128;
    } else {
        p.as_row_stride = kb; p.as_k_stride = 1;
        p.bs_row_stride = kb; p.bs_k_stride = 1;
    }
    p.n_dest = n_dest;
    p.c_col_offset = col_offset;
    p.dest_first = (n_dest > 1 && dest_n > 0 && n > 0) ? (col_offset / n) % n_dest : 0;   // = rank for an N-split
    if (sk_tiles > 0) {
        p.sk_tiles = sk_tiles;
        p.sk_token = rf::gemm_streamk_token(rf::next_streamk_epoch());
    }
    rf::GemmDestMaps dests;
    bool use_dests = false;
    if (fnuz) {
        // e4m3fnuz operands: one pass per operand writes the equal-valued e4m3fn bytes into library-owned
        // scratch and flags operands that hold +-240 or NaN bytes; the kernel reads a flagged operand from
        // its converted copy (maps in dests.m[0] / m[1]) and an unflagged one, exactly, from the caller's bytes.
        const size_t a_bytes = (size_t)m * k, b_bytes = (size_t)n * k;
        if (a_bytes % 16 != 0 || b_bytes % 16 != 0) return RF_ERR_BAD_SHAPE;
        const size_t a_pad = (a_bytes + 255) / 256 * 256, b_pad = (b_bytes + 255) / 256 * 256;
        char* conv = static_cast<char*>(rf::device_scratch(a_pad + b_pad + 256, rf::kScratchFnuz));
        if (!conv) return RF_ERR_CUDA;
        int* flags = reinterpret_cast<int*>(conv + a_pad + b_pad);
        if (rf::fp8_fnuz_convert_launch(a, conv, a_bytes, flags, st->status, st->num_sms, stream) != cudaSuccess ||
            rf::fp8_fnuz_convert_launch(b, conv + a_pad, b_bytes, flags + 1, st->status, st->num_sms, stream) !=
                cudaSuccess)
            return RF_ERR_CUDA;
        if (!rf::encode_tma_2d(&dests.m[0], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, conv, (uint64_t)k, (uint64_t)m,
                               (uint64_t)m, 128, 128, true) ||
            !rf::encode_tma_2d(&dests.m[1], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, conv + a_pad, (uint64_t)k, (uint64_t)n,
                               (uint64_t)n, 128, 128, true))
            return RF_ERR_CUDA;
        for (int i = 2; i < 8; ++i) dests.m[i] = dests.m[0];
        p.fnuz_flags = flags;
        use_dests = true;
    }
    if (n_dest > 1) {
        for (int i = 0; i < n_dest; ++i) {
            if (!rf::encode_tma_2d(&dests.m[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dest_c[i], (uint64_t)m,
                                   (uint64_t)dest_n, (uint64_t)dest_n * 2, 32, 64, true))
                return RF_ERR_CUDA;
        }
        for (int i = n_dest; i < 8; ++i) dests.m[i] = dests.m[0];
        use_dests = true;
    }
    cudaError_t e = rf::fp8_gemm_launch(ta, tb, tc, tp, use_dests ? &dests : nullptr, p, bn, st->num_sms, stream,
                                        mn_major);
    if (e != cudaSuccess) {
        fprintf(stderr, "rf_b200: fp8 gemm launch failed: %s\n", cudaGetErrorString(e));
        return RF_ERR_CUDA;
    }
    return RF_OK;
}

}  // namespace

namespace rf {
void fp8_gemm_plan(int m, int n, int k, int num_sms, int split_k, int* block_n, int* splits) {
    const int kb = k / kBlockK;
    if (split_k > kb) split_k = kb;
    if (split_k > kMaxSplits) split_k = kMaxSplits;
    const GemmPlan plan = choose_plan(m, n, k, num_sms, split_k);
    *block_n = plan.block_n;
    *splits = plan.splits;
}
}  // namespace rf

extern "C" {

const char* rf_version(void) { return "rf_b200 0.1 sm_100a"; }

int rf_device_status(int* detail) {
    rf::DeviceState* st = rf::device_state();
    if (!st) return RF_ERR_CUDA;
    int v[2] = {0, 0};
    if (cudaDeviceSynchronize() != cudaSuccess) return RF_ERR_CUDA;
    if (cudaMemcpy(v, st->status, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return RF_ERR_CUDA;
    // word 0: code of an expired wait (1-6); word 1: diagnostic flags (16, 32) that stopped nothing
    if (detail) *detail = v[0] != 0 ? (v[0] & 0xFF) : v[1];
    if (v[0] != 0 || v[1] != 0) {
        cudaMemset(st->status, 0, sizeof(v));
        return RF_ERR_DEVICE_TIMEOUT;
    }
    return RF_OK;
}

int rf_set_wait_limit_ns(unsigned long long limit_ns) {
    rf::DeviceState* st = rf::device_state();
    if (!st) return RF_ERR_CUDA;
    return cudaMemcpy(st->status + rf::kStatusLimitWord, &limit_ns, sizeof(limit_ns), cudaMemcpyHostToDevice) ==
                   cudaSuccess
               ? RF_OK : RF_ERR_CUDA;
}

int rf_fp8_gemm_get_plan(int m, int n, int k, int* block_n, int* split_k) {
    if (!shape_ok(m, n, k)) return RF_ERR_BAD_SHAPE;
    rf::DeviceState* st = rf::device_state();
    const GemmPlan plan = choose_plan(m, n, k, st ? st->num_sms : 148, 0);
    if (block_n) *block_n = plan.block_n;
    if (split_k) *split_k = plan.splits;
    return RF_OK;
}

int rf_fp8_gemm_choose_split(int m, int n, int k) {
    if (!shape_ok(m, n, k)) return 0;
    rf::DeviceState* st = rf::device_state();
    if (!st) return 0;
    return choose_plan(m, n, k, st->num_sms, 0).splits;
}

int rf_fp8_gemm_work_pieces(int m, int n, int k, int block_n, int split_k, int num_sms, int cta, int* pieces,
                            int max_pieces) {
    if (!shape_ok(m, n, k) || (block_n != 128 && block_n != 256) || num_sms < 1 || cta < 0 || !pieces) return -1;
    const int kb = k / kBlockK;
    if (split_k < kStreamK || split_k == 0 || split_k > kb || split_k > kMaxSplits) return -1;
    rf::GemmParams p;
    p.k = k;
    p.tiles_m = (m + 127) / 128;
    p.tiles_n = (n + block_n - 1) / block_n;
    p.splits = split_k == kStreamK ? 1 : split_k;
    p.sk_tiles = split_k == kStreamK ? rf::gemm_streamk_tiles(p.tiles_m * p.tiles_n, num_sms) : 0;
    const int total = p.tiles_m * p.tiles_n * p.splits;
    const int grid = (total < num_sms && p.sk_tiles == 0) ? total : num_sms;
    if (cta >= grid) return 0;
    return rf::fp8_gemm_walk_pieces(p, cta, grid, pieces, max_pieces);
}

size_t rf_fp8_gemm_workspace_bytes(int m, int n, int k, int split_k) {
    if (!shape_ok(m, n, k) || split_k < kStreamK) return 0;
    rf::DeviceState* st = rf::device_state();
    const int num_sms = st ? st->num_sms : 148;      // (no GPU: the answer for a B200)
    const int kb = k / kBlockK;
    if (split_k > kb) split_k = kb;
    if (split_k > kMaxSplits) split_k = kMaxSplits;
    const GemmPlan plan = choose_plan(m, n, k, num_sms, split_k);
    if (plan.splits == kStreamK) return rf::gemm_streamk_bytes(plan.block_n, num_sms);
    return plan.splits > 1 ? (size_t)plan.splits * m * n * sizeof(float) : 0;
}

int rf_fp8_gemm(const void* a, const void* b, const float* as, const float* bs, void* c, int m, int n, int k,
                int split_k, void* workspace, size_t workspace_bytes, rf_stream_t stream) {
    return gemm_impl(a, b, as, bs, c, m, n, k, split_k, workspace, workspace_bytes, false,
                     reinterpret_cast<cudaStream_t>(stream));
}

int rf_fp8_gemm_nsplit(const void* a, const void* b_shard, const float* as, const float* bs_shard,
                       void* const* c_all, int m, int n_total, int k, int rank, int world, rf_stream_t stream) {
    if (world < 1 || world > 8 || rank < 0 || rank >= world || n_total % world != 0) return RF_ERR_BAD_SHAPE;
    const int n_loc = n_total / world;
    if (n_loc % 128 != 0) return RF_ERR_BAD_SHAPE;     // shards must keep whole 128-wide scale blocks
    if (!c_all) return RF_ERR_NULL_POINTER;
    if (world == 1)
        return gemm_impl(a, b_shard, as, bs_shard, c_all[0], m, n_total, k, 1, nullptr, 0, true,
                         reinterpret_cast<cudaStream_t>(stream));
    return gemm_impl(a, b_shard, as, bs_shard, nullptr, m, n_loc, k, 1, nullptr, 0, true,
                     reinterpret_cast<cudaStream_t>(stream), c_all, world, n_total, rank * n_loc);
}

int rf_fp8_gemm_colmajor(const void* a, const void* b, const float* as, const float* bs, void* c, int m, int n,
                         int k, void* workspace, size_t workspace_bytes, rf_stream_t stream) {
    return gemm_impl(a, b, as, bs, c, m, n, k, 0, workspace, workspace_bytes, workspace == nullptr,
                     reinterpret_cast<cudaStream_t>(stream), nullptr, 1, 0, 0, true);
}

int rf_fp8_gemm_colmajor_fnuz(const void* a, const void* b, const float* as, const float* bs, void* c, int m, int n,
                              int k, void* workspace, size_t workspace_bytes, rf_stream_t stream) {
    return gemm_impl(a, b, as, bs, c, m, n, k, 0, workspace, workspace_bytes, workspace == nullptr,
                     reinterpret_cast<cudaStream_t>(stream), nullptr, 1, 0, 0, true, true);
}

void run(void* a, void* b, void* as, void* bs, void* c, int m, int n, int k, PerfMetrics* metrics,
         rf_stream_t stream) {
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (metrics) {
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        cudaEventRecord(e0, s);
    }
    int rc = gemm_impl(a, b, static_cast<const float*>(as), static_cast<const float*>(bs), c, m, n, k, 0, nullptr, 0,
                       true, s);
    if (rc != RF_OK) {
        fprintf(stderr, "Error: fp8 gemm failed (status %d) for M=%d, K=%d, N=%d\n", rc, m, k, n);
        abort();
    }
    if (metrics) {
        cudaEventRecord(e1, s);
        cudaEventSynchronize(e1);
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (metrics->count < 1) metrics->count = 1;
        strncpy(metrics->entries[0].name, "gemm", sizeof(metrics->entries[0].name) - 1);
        metrics->entries[0].time = ms;
        metrics->entries[0].gflops = ms > 0.f ? (float)(2.0 * m * n * k / (ms * 1e-3) / 1e9) : 0.f;
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
    }
}

}  // extern "C"
