// Expert-parallel token exchange over NVLink peer memory.  The reference is single-GPU; these kernels
// are the multi-GPU form of its expand_input / reduce_output pair (src/moe/moe_topk_kernel.cpp:174-251):
// the row gather writes straight into the owner GPU's receive buffer (dispatch) and the weighted
// combine reads the expert outputs straight from the owner GPUs (combine).  Only ordinary peer
// loads and stores are used; ordering between GPUs comes from stream-ordered barriers outside.
#include "moe_kernels.h"
#include "ptx.cuh"

#include <cuda_fp16.h>
#include <stdint.h>

namespace rf {

namespace {

__global__ void __launch_bounds__(1024)
ep_layout_kernel(const int* __restrict__ counts_all, int rank, int world, int n_experts, int capacity,
                 int* __restrict__ send_base, int* __restrict__ recv_offsets, int* __restrict__ status) {
    __shared__ int tot[1024];
    const int e = threadIdx.x;
    const int per = n_experts / world;
    int t = 0, before_me = 0;
    if (e < n_experts) {
        // Rows of one expert are ordered by source rank starting at the owner: q, q+1, ... (mod world).
        // The owners then walk their rows, and return the results, towards different GPUs at any moment.
        const int q = e / per;
        const int my_pos = (rank - q + world) % world;
        for (int j = 0; j < world; ++j) {
            int s = q + j;
            if (s >= world) s -= world;
            const int c = counts_all[s * n_experts + e];
            if (j < my_pos) before_me += c;
            t += c;
        }
        tot[e] = t;
    }
    __syncthreads();
    if (e < n_experts) {
        const int owner_first = (e / per) * per;
        int base = 0;
        for (int j = owner_first; j < e; ++j) base += tot[j];
        send_base[e] = base + before_me;
    }
    if (e <= per) {
        int off = 0;
        for (int j = 0; j < e; ++j) off += tot[rank * per + j];
        // Rows beyond the receive capacity are never written by the senders (ep_dispatch_kernel drops them):
        // the expert row ranges are clipped to the capacity and the overflow is reported.
        if (off > capacity) {
            if (e == per) atomicOr(status + kStatusDiagWord, (int)kDiagEpOverflow);
            off = capacity;
        }
        recv_offsets[e] = off;
    }
}

// One row per block iteration: the row's indices are read once (not once per 16 bytes), then the
// block's threads move the row with up to four independent 16-byte loads in flight each before the
// matching peer stores.  Launched as many 256-thread blocks spread over every SM (the SM-partitioned dispatch is
// ep_dispatch_bulk_kernel below).
__global__ void __launch_bounds__(1024)
ep_dispatch_kernel(const uint4* __restrict__ x, const int* __restrict__ permuted_experts,
                   const int* __restrict__ permuted_rows, const int* __restrict__ first_token_offset,
                   const int* __restrict__ send_base, int n_tokens, int n_pairs, int vec_per_row,
                   int experts_per_rank, int rank, int world, int capacity, PeerPtrs recv_x, PeerPtrs recv_meta,
                   int with_meta, int* __restrict__ pair_rank, int* __restrict__ pair_row, uint4* __restrict__ drop_fill,
                   int* __restrict__ status) {
    // Pairs are sorted by expert, hence by destination rank.  Every source starts with a different
    // destination (rank+1, rank+2, ...), so at any moment the senders target different GPUs instead of
    // all writing into the same one.
    const int p0 = __ldg(first_token_offset + ((rank + 1) % world) * experts_per_rank);
    // a group of 256 threads moves one row at a time: one group per block, or four in a 1024-thread block
    const int groups_per_block = blockDim.x >> 8;
    const int tid = threadIdx.x & 255;
    for (int i = blockIdx.x * groups_per_block + (threadIdx.x >> 8); i < n_pairs; i += gridDim.x * groups_per_block) {
        int p = i + p0;
        if (p >= n_pairs) p -= n_pairs;
        const int e = __ldg(permuted_experts + p);
        const int q = e / experts_per_rank;
        const int row = __ldg(send_base + e) + (p - __ldg(first_token_offset + e));
        if (row >= capacity) {
            // the owner's receive buffer is full: the row is dropped (its result will be missing), never
            // written past the allocation on another GPU; -1 marks the pair for the pulling combine, and
            // where results are pushed home the pair's result row is zeroed here instead
            if (drop_fill != nullptr)
                for (int v0 = tid; v0 < vec_per_row; v0 += 256)
                    drop_fill[(size_t)p * vec_per_row + v0] = make_uint4(0u, 0u, 0u, 0u);
            if (tid == 0) {
                pair_rank[p] = -1;
                pair_row[p] = 0;
                atomicOr(status + kStatusDiagWord, (int)kDiagEpOverflow);
            }
            continue;
        }
        const int tok = __ldg(permuted_rows + p) % n_tokens;
        const uint4* src = x + (size_t)tok * vec_per_row;
        uint4* dst = static_cast<uint4*>(pick_peer(recv_x, q)) + (size_t)row * vec_per_row;
        for (int v0 = tid; v0 < vec_per_row; v0 += 4 * 256) {
            uint4 r[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (v0 + j * 256 < vec_per_row) r[j] = __ldg(src + v0 + j * 256);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (v0 + j * 256 < vec_per_row) dst[v0 + j * 256] = r[j];
        }
        if (tid == 0) {
            pair_rank[p] = q;
            pair_row[p] = row;
            if (with_meta) static_cast<int*>(pick_peer(recv_meta, q))[row] = (rank << kEpMetaSlotBits) | p;
        }
    }
}

// The dispatch for the SM partition: a few blocks that own an SM each move the rows with the copy engine instead
// of with loads and stores.  Each of a block's kEpBulkWarps warps owns one row buffer in shared memory and moves
// one row at a time through it: a bulk load of the token row (local HBM -> shared memory, counted on the warp's
// mbarrier), then a bulk store of the buffer into the owner's receive buffer (a peer GPU's memory: posted writes
// over NVLink); the buffer is reloaded once that store has finished reading it.  What an SM keeps in flight is
// bounded by its shared memory (12 rows of 14 KB), about 50 GB/s per SM: 16-24 blocks keep NVLink busy and leave
// the other SMs to the shared expert's GEMMs running beside them.
constexpr int kEpBulkWarps = 12;

__global__ void __launch_bounds__(32 * kEpBulkWarps)
ep_dispatch_bulk_kernel(const uint4* __restrict__ x, const int* __restrict__ permuted_experts,
                        const int* __restrict__ permuted_rows, const int* __restrict__ first_token_offset,
                        const int* __restrict__ send_base, int n_tokens, int n_pairs, int vec_per_row,
                        int experts_per_rank, int rank, int world, int capacity, PeerPtrs recv_x, PeerPtrs recv_meta,
                        int with_meta, int* __restrict__ pair_rank, int* __restrict__ pair_row,
                        uint4* __restrict__ drop_fill, int* __restrict__ status) {
    extern __shared__ __align__(128) uint8_t ep_smem[];
    __shared__ __align__(8) unsigned long long bars[kEpBulkWarps];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t row_bytes = (uint32_t)vec_per_row * 16u;
    const uint32_t buf = smem_u32(ep_smem) + (uint32_t)warp * row_bytes;
    const uint32_t bar = smem_u32(bars) + 8u * warp;
    if (lane == 0) mbar_init(bar, 1);
    mbar_fence_init();
    __syncwarp();
    const int p0 = __ldg(first_token_offset + ((rank + 1) % world) * experts_per_rank);
    const int n_warps = gridDim.x * kEpBulkWarps;
    uint32_t cnt = 0;                 // rows this warp has moved
    for (int i = blockIdx.x * kEpBulkWarps + warp; i < n_pairs; i += n_warps) {
        int p = i + p0;
        if (p >= n_pairs) p -= n_pairs;
        const int e = __ldg(permuted_experts + p);
        const int q = e / experts_per_rank;
        const int row = __ldg(send_base + e) + (p - __ldg(first_token_offset + e));
        if (row >= capacity) {
            // receive buffer full: dropped and reported, as in ep_dispatch_kernel
            if (drop_fill != nullptr)
                for (int v0 = lane; v0 < vec_per_row; v0 += 32)
                    drop_fill[(size_t)p * vec_per_row + v0] = make_uint4(0u, 0u, 0u, 0u);
            if (lane == 0) {
                pair_rank[p] = -1;
                pair_row[p] = 0;
                atomicOr(status + kStatusDiagWord, (int)kDiagEpOverflow);
            }
            continue;
        }
        const int tok = __ldg(permuted_rows + p) % n_tokens;
        if (lane == 0) {
            tma_store_wait_read<0>();         // the previous row's store has finished reading the buffer
            mbar_expect_tx(bar, row_bytes);
            bulk_load(buf, x + (size_t)tok * vec_per_row, row_bytes, bar);
            pair_rank[p] = q;
            pair_row[p] = row;
            if (with_meta) static_cast<int*>(pick_peer(recv_meta, q))[row] = (rank << kEpMetaSlotBits) | p;
        }
        __syncwarp();
        const bool ok = __all_sync(0xffffffffu, mbar_wait(bar, cnt & 1u, status, kErrSchedWait, 0));
        if (!ok) break;
        if (lane == 0) {
            bulk_store(static_cast<uint4*>(pick_peer(recv_x, q)) + (size_t)row * vec_per_row, buf, row_bytes);
            tma_store_commit();
        }
        ++cnt;
    }
    // the rows must have landed before the kernel (and the rendezvous that follows it) completes
    if (lane == 0) tma_store_wait_all<0>();
}

__global__ void __launch_bounds__(256)
ep_combine_kernel(PeerPtrs y, const uint4* __restrict__ shared_out, const int* __restrict__ rev,
                  const __half* __restrict__ weights, const int* __restrict__ pair_rank,
                  const int* __restrict__ pair_row, int n_tokens, int top_k, int vec_per_row, uint4* __restrict__ out) {
    const int t = blockIdx.x;
    __shared__ const uint4* src_s[8];
    __shared__ float w_s[8];
    if (threadIdx.x < top_k) {
        const int p = rev[threadIdx.x * n_tokens + t];
        const int q = pair_rank[p];
        // a pair dropped by the dispatch (receive buffer full) contributes nothing
        src_s[threadIdx.x] = static_cast<const uint4*>(pick_peer(y, q < 0 ? 0 : q)) + (size_t)pair_row[p] * vec_per_row;
        w_s[threadIdx.x] = q < 0 ? 0.f : __half2float(weights[p]);
    }
    __syncthreads();
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        // all k row segments are requested before the first is used: k independent loads in flight
        // per thread (the rows sit in other GPUs' memory, a round trip of microseconds)
        uint4 qv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i < top_k) qv[i] = src_s[i][v];     // peer (or local) load
#pragma unroll
        for (int i = 0; i < 8; ++i) {
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
        uint4 sq = make_uint4(0u, 0u, 0u, 0u);                 // fp16 zeros when the shared expert is added later
        if (shared_out != nullptr) sq = __ldg(shared_out + (size_t)t * vec_per_row + v);
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

// out += add, fp16 rows, fp32 arithmetic (the shared expert's output joins the combined routed output
// when its second GEMM ran concurrently with the combine)
__global__ void __launch_bounds__(256)
add_rows_kernel(uint4* __restrict__ out, const uint4* __restrict__ add, size_t n_vec) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.x * blockDim.x) {
        uint4 a = out[i];
        const uint4 b = __ldg(add + i);
        __half2* ah = reinterpret_cast<__half2*>(&a);
        const __half2* bh = reinterpret_cast<const __half2*>(&b);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 x = __half22float2(ah[j]);
            const float2 y = __half22float2(bh[j]);
            ah[j] = __floats2half2_rn(x.x + y.x, x.y + y.y);
        }
        out[i] = a;
    }
}

// One block.  Threads publish this rank's counts to every peer, then thread s < world raises this
// rank's flag on peer s and waits for peer s's flag here.  Flags only grow (epoch numbers), so a slow
// rank can never be overtaken by two epochs.  The wait is bounded: on expiry the status word is set
// and the kernel returns.
__global__ void __launch_bounds__(256)
ep_rendezvous_kernel(PeerPtrs sync, const int* __restrict__ counts, int n_counts, int from_offsets, int rank,
                     int world, int epoch, int* status) {
    if (counts != nullptr) {
        for (int i = threadIdx.x; i < n_counts * world; i += blockDim.x) {
            const int peer = i / n_counts;
            const int j = i - peer * n_counts;
            int* area = static_cast<int*>(pick_peer(sync, peer));
            // `counts` is either the values themselves or n_counts + 1 ascending offsets (first_token_offset)
            area[8 + rank * n_counts + j] = from_offsets ? counts[j + 1] - counts[j] : counts[j];
        }
    }
    __threadfence_system();          // the counts (and every earlier peer store of this stream) before the flag
    __syncthreads();
    if (threadIdx.x < world) {
        const int peer = threadIdx.x;
        volatile int* theirs = static_cast<int*>(pick_peer(sync, peer)) + rank;
        *theirs = epoch;
        volatile int* mine = static_cast<int*>(pick_peer(sync, rank)) + peer;
        const unsigned long long t0 = globaltimer_ns();
        const unsigned long long limit = wait_limit_ns(status);
        unsigned spins = 0;
        while (*mine < epoch) {
            if ((++spins & 0x3ff) == 0 && globaltimer_ns() - t0 > limit) {
                atomicCAS(status, 0, kErrSchedWait);
                break;
            }
        }
    }
    __threadfence_system();
}

}  // namespace

cudaError_t moe_ep_rendezvous_launch(const PeerPtrs& sync, const int* counts, int n_counts, bool from_offsets,
                                     int rank, int world, int epoch, int* status, cudaStream_t stream) {
    ep_rendezvous_kernel<<<1, 256, 0, stream>>>(sync, counts, n_counts, from_offsets ? 1 : 0, rank, world, epoch,
                                                status);
    return cudaGetLastError();
}

cudaError_t moe_add_rows_launch(void* out, const void* add, size_t n_elems, int num_sms, cudaStream_t stream) {
    const size_t n_vec = n_elems / 8;
    if (n_vec == 0) return cudaSuccess;
    size_t blocks = (n_vec + 255) / 256;
    const size_t cap = (size_t)num_sms * 8;
    if (blocks > cap) blocks = cap;
    add_rows_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<uint4*>(out), static_cast<const uint4*>(add),
                                                         n_vec);
    return cudaGetLastError();
}

cudaError_t moe_ep_layout_launch(const int* counts_all, int rank, int world, int n_experts, int capacity,
                                 int* send_base, int* recv_offsets, int* status, cudaStream_t stream) {
    ep_layout_kernel<<<1, 1024, 0, stream>>>(counts_all, rank, world, n_experts, capacity, send_base, recv_offsets,
                                             status);
    return cudaGetLastError();
}

cudaError_t moe_ep_dispatch_launch(const void* x, const int* permuted_experts, const int* permuted_rows,
                                   const int* first_token_offset, const int* send_base, int n_tokens, int n_pairs,
                                   int row_bytes, int experts_per_rank, int rank, int world, int capacity,
                                   const PeerPtrs& recv_x, const PeerPtrs* recv_meta, int* pair_rank, int* pair_row,
                                   void* drop_fill, int* status, int num_sms, int max_blocks, cudaStream_t stream) {
    const int vec = row_bytes / 16;
    if (n_pairs == 0) return cudaSuccess;
    if (max_blocks > 0) {
        // SM partition.  Rows of which twelve fit an SM's shared memory travel by bulk copies:
        const size_t ring_bytes = (size_t)kEpBulkWarps * row_bytes;
        if (row_bytes % 16 == 0 && ring_bytes <= 200 * 1024) {
            // ask for at least 120 KB so that no CTA of the GEMM running beside the dispatch shares the SM
            const size_t smem = ring_bytes > 120 * 1024 ? ring_bytes : 120 * 1024;
            static bool bulk_attr_set[64] = {};
            int dev = 0;
            cudaGetDevice(&dev);
            if (dev < 64 && !bulk_attr_set[dev]) {
                cudaError_t e = cudaFuncSetAttribute(ep_dispatch_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     200 * 1024);
                if (e != cudaSuccess) return e;
                bulk_attr_set[dev] = true;
            }
            int blocks = max_blocks * kEpBulkWarps < n_pairs ? max_blocks : (n_pairs + kEpBulkWarps - 1) / kEpBulkWarps;
            ep_dispatch_bulk_kernel<<<(unsigned)blocks, 32 * kEpBulkWarps, smem, stream>>>(
                static_cast<const uint4*>(x), permuted_experts, permuted_rows, first_token_offset, send_base, n_tokens,
                n_pairs, vec, experts_per_rank, rank, world, capacity, recv_x, recv_meta ? *recv_meta : recv_x,
                recv_meta ? 1 : 0, pair_rank, pair_row, static_cast<uint4*>(drop_fill), status);
            return cudaGetLastError();
        }
        // (longer rows: no partition; the dispatch below spreads over every SM)
    }
    int blocks = num_sms * 8;
    if (blocks > n_pairs) blocks = n_pairs;
    ep_dispatch_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const uint4*>(x), permuted_experts,
                                                             permuted_rows, first_token_offset, send_base, n_tokens,
                                                             n_pairs, vec, experts_per_rank, rank, world, capacity,
                                                             recv_x, recv_meta ? *recv_meta : recv_x,
                                                             recv_meta ? 1 : 0, pair_rank, pair_row,
                                                             static_cast<uint4*>(drop_fill), status);
    return cudaGetLastError();
}

cudaError_t moe_ep_combine_launch(const PeerPtrs& y, const void* shared_out, const int* rev, const void* weights,
                                  const int* pair_rank, const int* pair_row, int n_tokens, int top_k, int row_bytes,
                                  void* out, cudaStream_t stream) {
    if (n_tokens == 0) return cudaSuccess;
    ep_combine_kernel<<<n_tokens, 256, 0, stream>>>(y, static_cast<const uint4*>(shared_out), rev,
                                                    static_cast<const __half*>(weights), pair_rank, pair_row,
                                                    n_tokens, top_k, row_bytes / 16, static_cast<uint4*>(out));
    return cudaGetLastError();
}

}  // namespace rf
