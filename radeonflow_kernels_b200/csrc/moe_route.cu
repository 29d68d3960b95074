// MoE routing and data-movement kernels (all HBM/latency bound, no tensor cores):
//   topk_kernel          softmax + k rounds of warp-shuffle arg-max          (src/moe/moe_topk_kernel.cpp:15-150)
//   count/scan/scatter   stable counting sort of (expert, source_row) pairs, replacing the radix sort,
//                        the binary-search offsets and the index half of expand_input
//                        (src/moe/moe.cpp:119-126, src/moe/moe_topk_kernel.cpp:152-172, :199-201)
//   gather_rows_kernel   expanded_seq_input[dest] = x[permuted_rows[dest] % T]  (:174-213)
//   combine_kernel       out[t] = sum_i w * Y[rev[i*T+t]] + shared[t]           (:215-251)
//   tile_list_kernel     per-expert row ranges -> list of 128-row tiles for the grouped GEMM
#include "moe_kernels.h"

#include <cuda_fp16.h>
#include <stdint.h>

namespace rf {

namespace {

// exp(x), x <= 0, as a fixed sequence of fp32 operations with no fused multiply-add, so a CPU
// restatement reproduces it bit for bit: t = max(x,-80)*log2e; n = rint(t); f = t-n; degree-7
// Horner for 2^f; exact scaling by 2^n.
__device__ __forceinline__ float det_exp(float x) {
    x = fmaxf(x, -80.0f);
    const float t = __fmul_rn(x, 1.4426950408889634f);
    const float n = rintf(t);
    const float f = __fsub_rn(t, n);
    float p = 1.5252733804059840e-05f;
    p = __fadd_rn(__fmul_rn(p, f), 0.0001540353039338161f);
    p = __fadd_rn(__fmul_rn(p, f), 0.0013333558146428443f);
    p = __fadd_rn(__fmul_rn(p, f), 0.009618129107628477f);
    p = __fadd_rn(__fmul_rn(p, f), 0.05550410866482158f);
    p = __fadd_rn(__fmul_rn(p, f), 0.2402265069591007f);
    p = __fadd_rn(__fmul_rn(p, f), 0.6931471805599453f);
    p = __fadd_rn(__fmul_rn(p, f), 1.0f);
    return __uint_as_float(__float_as_uint(p) + (static_cast<int>(n) << 23));   // p in [0.7, 1.42], result normal
}

// One warp per token row.  Lane l owns experts [l*VPT, (l+1)*VPT); for E < 32 lanes >= E are idle.
template <int VPT>
__global__ void __launch_bounds__(256)
topk_kernel(const __half* __restrict__ scores, int n_tokens, int n_experts, int top_k, int* __restrict__ out_index,
            __half* __restrict__ out_weight, int* __restrict__ source_rows) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= n_tokens) return;
    const int first = lane * VPT;
    const bool active = first < n_experts;
    const __half* row = scores + (size_t)warp * n_experts;

    float logit[VPT];
    if (active) {
        if (VPT == 8) {
            const uint4 q = *reinterpret_cast<const uint4*>(row + first);
            const __half* h = reinterpret_cast<const __half*>(&q);
#pragma unroll
            for (int j = 0; j < VPT; ++j) logit[j] = __half2float(h[j]);
        } else {
#pragma unroll
            for (int j = 0; j < VPT; ++j) logit[j] = __half2float(row[first + j]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < VPT; ++j) logit[j] = -65504.0f;
    }
    // row maximum (exact in any order; the reference takes it in fp16, same value)
    float mx = logit[0];
#pragma unroll
    for (int j = 1; j < VPT; ++j) mx = fmaxf(mx, logit[j]);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));

    float e[VPT];
    float part = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        e[j] = active ? det_exp(__fsub_rn(logit[j], mx)) : 0.f;
        part = (j == 0) ? e[0] : __fadd_rn(part, e[j]);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, s));
    const float recip = __fdiv_rn(1.0f, part);

    // fp16 probabilities; the selection runs on these (ties are frequent at fp16 resolution)
    float prob[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j)
        prob[j] = active ? __half2float(__float2half_rn(__fmul_rn(e[j], recip))) : -INFINITY;

    for (int k = 0; k < top_k; ++k) {
        float best = prob[0];
        int best_i = first;
#pragma unroll
        for (int j = 1; j < VPT; ++j) {
            if (prob[j] > best) { best = prob[j]; best_i = first + j; }
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, s);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, s);
            if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
        }
        if (lane == 0) {
            const size_t o = (size_t)warp * top_k + k;
            out_index[o] = best_i;
            out_weight[o] = __float2half_rn(best);
            source_rows[o] = k * n_tokens + warp;
        }
        // clear the winner in its owner lane
#pragma unroll
        for (int j = 0; j < VPT; ++j)
            if (first + j == best_i) prob[j] = -INFINITY;
    }
}

constexpr int kSortBlock = 256;
constexpr int kSortItemsPerBlock = 1024;     // 8 warps x 128 consecutive items

// block_counts[e * n_blocks + b] = number of items of block b routed to expert e
__global__ void __launch_bounds__(kSortBlock)
sort_count_kernel(const int* __restrict__ experts, int n_items, int n_experts, int n_blocks,
                  int* __restrict__ block_counts) {
    extern __shared__ int hist[];
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    const int base = blockIdx.x * kSortItemsPerBlock;
    for (int i = threadIdx.x; i < kSortItemsPerBlock; i += blockDim.x) {
        const int g = base + i;
        if (g < n_items) atomicAdd(&hist[experts[g]], 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) block_counts[e * n_blocks + blockIdx.x] = hist[e];
}

// Exclusive scan of block_counts in (expert major, block minor) order, in place; also writes
// first_token_offset[0..E].  One block of 1024 threads; n = E * n_blocks.
__global__ void __launch_bounds__(1024)
sort_scan_kernel(int* __restrict__ block_counts, int n_experts, int n_blocks, int* __restrict__ first_token_offset) {
    __shared__ int warp_sums[32];
    __shared__ int carry;
    const int n = n_experts * n_blocks;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int base = 0; base < n; base += 1024) {
        const int i = base + threadIdx.x;
        const int v = i < n ? block_counts[i] : 0;
        int incl = v;
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, incl, s);
            if (lane >= s) incl += o;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = warp_sums[lane];
#pragma unroll
            for (int s = 1; s < 32; s <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, w, s);
                if (lane >= s) w += o;
            }
            warp_sums[lane] = w;
        }
        __syncthreads();
        const int excl = carry + (warp > 0 ? warp_sums[warp - 1] : 0) + incl - v;
        if (i < n) {
            block_counts[i] = excl;
            if (i % n_blocks == 0) first_token_offset[i / n_blocks] = excl;
        }
        __syncthreads();
        if (threadIdx.x == 1023) carry = excl + v;
        __syncthreads();
    }
    if (threadIdx.x == 0) first_token_offset[n_experts] = carry;
}

// Stable scatter: item g (expert e) goes to block_base[e][b] + (number of earlier items of block b with expert e).
__global__ void __launch_bounds__(kSortBlock)
sort_scatter_kernel(const int* __restrict__ experts, const int* __restrict__ source_rows,
                    const __half* __restrict__ weights, int n_items, int n_experts, int n_blocks,
                    const int* __restrict__ block_base, int* __restrict__ permuted_experts,
                    int* __restrict__ permuted_rows, int* __restrict__ rev_permuted_rows,
                    __half* __restrict__ expanded_softmax) {
    extern __shared__ int smem[];          // [8 warps][E] running offsets
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int* mine = smem + warp * n_experts;
    for (int e = threadIdx.x; e < 8 * n_experts; e += blockDim.x) smem[e] = 0;
    __syncthreads();
    const int wbase = blockIdx.x * kSortItemsPerBlock + warp * 128;
    // pass 1: per-warp counts
    for (int it = 0; it < 4; ++it) {
        const int g = wbase + it * 32 + lane;
        const int e = g < n_items ? experts[g] : -1;
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        if (e >= 0 && (peers & ((1u << lane) - 1)) == 0) mine[e] += __popc(peers);
        __syncwarp();
    }
    __syncthreads();
    // exclusive scan over the 8 warps, per expert, starting from this block's base for the expert
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        int run = block_base[e * n_blocks + blockIdx.x];
        for (int w = 0; w < 8; ++w) {
            const int c = smem[w * n_experts + e];
            smem[w * n_experts + e] = run;
            run += c;
        }
    }
    __syncthreads();
    // pass 2: ranks inside each group of 32 by match_any, groups in order
    for (int it = 0; it < 4; ++it) {
        const int g = wbase + it * 32 + lane;
        const int e = g < n_items ? experts[g] : -1;
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        if (e >= 0) {
            const int pos = mine[e] + __popc(peers & ((1u << lane) - 1));
            const int src = source_rows[g];
            permuted_experts[pos] = e;
            permuted_rows[pos] = src;
            rev_permuted_rows[src] = pos;
            expanded_softmax[pos] = weights[g];
        }
        __syncwarp();
        if (e >= 0 && (peers & ((1u << lane) - 1)) == 0) mine[e] += __popc(peers);
        __syncwarp();
    }
}

// dest row r <- src row (row_map[r] % row_mod); one 16-byte vector per thread-iteration
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ src, const int* __restrict__ row_map, int row_mod, int n_rows,
                   int vec_per_row, uint4* __restrict__ dst) {
    const size_t total = (size_t)n_rows * vec_per_row;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / vec_per_row);
        const int v = (int)(i - (size_t)r * vec_per_row);
        const int s = row_map[r] % row_mod;
        dst[i] = __ldg(src + (size_t)s * vec_per_row + v);
    }
}

// out[t, :] = fp16( sum_i w_i * Y[rev[i*T+t], :] + S[t, :] ), fp32 accumulation in rank order
template <int MAX_K>
__global__ void __launch_bounds__(256)
combine_kernel(const uint4* __restrict__ y, const uint4* __restrict__ shared_out, const int* __restrict__ rev,
               const __half* __restrict__ expanded_softmax, int n_tokens, int top_k, int vec_per_row,
               uint4* __restrict__ out) {
    const int t = blockIdx.x;
    __shared__ int pos_s[MAX_K];
    __shared__ float w_s[MAX_K];
    if (threadIdx.x < top_k) {
        const int pos = rev[threadIdx.x * n_tokens + t];
        pos_s[threadIdx.x] = pos;
        w_s[threadIdx.x] = __half2float(expanded_softmax[pos]);
    }
    __syncthreads();
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        // all k row segments are requested before the first is used
        uint4 qv[MAX_K];
#pragma unroll
        for (int i = 0; i < MAX_K; ++i)
            if (i < top_k) qv[i] = __ldg(y + (size_t)pos_s[i] * vec_per_row + v);
#pragma unroll
        for (int i = 0; i < MAX_K; ++i) {
            if (i >= top_k) continue;
            const uint4 q = qv[i];
            const __half2* h = reinterpret_cast<const __half2*>(&q);
            const float w = w_s[i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(h[j]);
                acc[2 * j] = fmaf(w, f.x, acc[2 * j]);
                acc[2 * j + 1] = fmaf(w, f.y, acc[2 * j + 1]);
            }
        }
        const uint4 sq = __ldg(shared_out + (size_t)t * vec_per_row + v);
        const __half2* sh = reinterpret_cast<const __half2*>(&sq);
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(sh[j]);
            oh[j] = __floats2half2_rn(acc[2 * j] + f.x, acc[2 * j + 1] + f.y);
        }
        out[(size_t)t * vec_per_row + v] = o;
    }
}

// Row ranges [offsets[g], offsets[g+1]) -> list of 128-row tiles: tile_group[i], tile_row0[i];
// tile_count[0] = number of tiles.  One block; groups <= 1024.
// tile_chunk[i] = (first tile of i's chunk << 8) | tiles in the chunk.  A chunk is a run of at most
// kMoeChunkTiles consecutive tiles of ONE group (a group's tiles are split into equal chunks); the grouped
// GEMM walks a chunk column block by column block, so the CTAs that run at the same time share one
// group's weight column block and the chunk's row tiles.
__global__ void __launch_bounds__(1024)
tile_list_kernel(const int* __restrict__ offsets, int n_groups, int* __restrict__ tile_group,
                 int* __restrict__ tile_row0, int* __restrict__ tile_chunk, int* __restrict__ tile_count) {
    __shared__ int warp_sums[32];
    const int g = threadIdx.x;
    const int lane = g & 31, warp = g >> 5;
    int lo = 0, n = 0;
    if (g < n_groups) {
        lo = offsets[g];
        n = (offsets[g + 1] - lo + 127) >> 7;
    }
    int incl = n;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, incl, s);
        if (lane >= s) incl += o;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = warp_sums[lane];
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
            const int o = __shfl_up_sync(0xffffffffu, w, s);
            if (lane >= s) w += o;
        }
        warp_sums[lane] = w;
    }
    __syncthreads();
    const int start = (warp > 0 ? warp_sums[warp - 1] : 0) + incl - n;
    const int n_chunks = (n + kMoeChunkTiles - 1) / kMoeChunkTiles;
    const int base = n_chunks ? n / n_chunks : 0;
    const int rem = n_chunks ? n % n_chunks : 0;          // the first `rem` chunks hold base + 1 tiles
    for (int i = 0; i < n; ++i) {
        tile_group[start + i] = g;
        tile_row0[start + i] = lo + i * 128;
        int c_first, c_size;
        if (i < rem * (base + 1)) {
            c_size = base + 1;
            c_first = (i / c_size) * c_size;
        } else {
            c_size = base;
            c_first = rem * (base + 1) + ((i - rem * (base + 1)) / base) * base;
        }
        tile_chunk[start + i] = ((start + c_first) << 8) | c_size;
    }
    if (g == 1023) tile_count[0] = start + n;
}

__global__ void set_range_kernel(int* dst, int a, int b) {
    dst[0] = a;
    dst[1] = b;
}

}  // namespace

cudaError_t moe_set_range_launch(int* dst, int a, int b, cudaStream_t stream) {
    set_range_kernel<<<1, 1, 0, stream>>>(dst, a, b);
    return cudaGetLastError();
}

cudaError_t moe_topk_launch(const void* scores, int n_tokens, int n_experts, int top_k, void* index, void* weight,
                            void* source_rows, cudaStream_t stream) {
    const int warps_per_block = 8;
    const unsigned grid = (unsigned)((n_tokens + warps_per_block - 1) / warps_per_block);
    const __half* s = static_cast<const __half*>(scores);
    int* oi = static_cast<int*>(index);
    __half* ow = static_cast<__half*>(weight);
    int* sr = static_cast<int*>(source_rows);
    const int vpt = n_experts <= 32 ? 1 : n_experts / 32;
    switch (vpt) {
        case 1: topk_kernel<1><<<grid, 256, 0, stream>>>(s, n_tokens, n_experts, top_k, oi, ow, sr); break;
        case 2: topk_kernel<2><<<grid, 256, 0, stream>>>(s, n_tokens, n_experts, top_k, oi, ow, sr); break;
        case 4: topk_kernel<4><<<grid, 256, 0, stream>>>(s, n_tokens, n_experts, top_k, oi, ow, sr); break;
        case 8: topk_kernel<8><<<grid, 256, 0, stream>>>(s, n_tokens, n_experts, top_k, oi, ow, sr); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

size_t moe_permute_scratch_bytes(int n_items, int n_experts) {
    const int n_blocks = (n_items + kSortItemsPerBlock - 1) / kSortItemsPerBlock;
    return (size_t)n_experts * (n_blocks > 0 ? n_blocks : 1) * sizeof(int);
}

cudaError_t moe_permute_launch(const void* experts, const void* source_rows, const void* weights, int n_items,
                               int n_experts, void* permuted_experts, void* permuted_rows, void* first_token_offset,
                               void* rev_permuted_rows, void* expanded_softmax, void* scratch, cudaStream_t stream) {
    const int n_blocks = (n_items + kSortItemsPerBlock - 1) / kSortItemsPerBlock;
    int* counts = static_cast<int*>(scratch);
    sort_count_kernel<<<n_blocks, kSortBlock, n_experts * sizeof(int), stream>>>(
        static_cast<const int*>(experts), n_items, n_experts, n_blocks, counts);
    sort_scan_kernel<<<1, 1024, 0, stream>>>(counts, n_experts, n_blocks, static_cast<int*>(first_token_offset));
    sort_scatter_kernel<<<n_blocks, kSortBlock, 8 * n_experts * sizeof(int), stream>>>(
        static_cast<const int*>(experts), static_cast<const int*>(source_rows), static_cast<const __half*>(weights),
        n_items, n_experts, n_blocks, counts, static_cast<int*>(permuted_experts), static_cast<int*>(permuted_rows),
        static_cast<int*>(rev_permuted_rows), static_cast<__half*>(expanded_softmax));
    return cudaGetLastError();
}

cudaError_t moe_gather_rows_launch(const void* src, const int* row_map, int row_mod, int n_rows, int row_bytes,
                                   void* dst, int num_sms, cudaStream_t stream) {
    const int vec = row_bytes / 16;
    const size_t total = (size_t)n_rows * vec;
    size_t blocks = (total + 255) / 256;
    const size_t cap = (size_t)num_sms * 16;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) return cudaSuccess;
    gather_rows_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const uint4*>(src), row_map, row_mod, n_rows,
                                                             vec, static_cast<uint4*>(dst));
    return cudaGetLastError();
}

cudaError_t moe_combine_launch(const void* y, const void* shared_out, const int* rev, const void* expanded_softmax,
                               int n_tokens, int top_k, int row_bytes, void* out, cudaStream_t stream) {
    if (n_tokens == 0) return cudaSuccess;
    combine_kernel<8><<<n_tokens, 256, 0, stream>>>(static_cast<const uint4*>(y), static_cast<const uint4*>(shared_out),
                                                   rev, static_cast<const __half*>(expanded_softmax), n_tokens, top_k,
                                                   row_bytes / 16, static_cast<uint4*>(out));
    return cudaGetLastError();
}

cudaError_t moe_tile_list_launch(const int* offsets, int n_groups, int* tile_group, int* tile_row0, int* tile_chunk,
                                 int* tile_count, cudaStream_t stream) {
    tile_list_kernel<<<1, 1024, 0, stream>>>(offsets, n_groups, tile_group, tile_row0, tile_chunk, tile_count);
    return cudaGetLastError();
}

}  // namespace rf
