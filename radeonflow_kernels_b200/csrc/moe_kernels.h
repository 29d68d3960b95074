// Internal interface between the C-ABI layer and the MoE kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>

namespace rf {

// ---- routing / data movement (moe_route.cu)
cudaError_t moe_topk_launch(const void* scores, int n_tokens, int n_experts, int top_k, void* index, void* weight,
                            void* source_rows, cudaStream_t stream);
size_t moe_permute_scratch_bytes(int n_items, int n_experts);
cudaError_t moe_permute_launch(const void* experts, const void* source_rows, const void* weights, int n_items,
                               int n_experts, void* permuted_experts, void* permuted_rows, void* first_token_offset,
                               void* rev_permuted_rows, void* expanded_softmax, void* scratch, cudaStream_t stream);
cudaError_t moe_gather_rows_launch(const void* src, const int* row_map, int row_mod, int n_rows, int row_bytes,
                                   void* dst, int num_sms, cudaStream_t stream);
cudaError_t moe_combine_launch(const void* y, const void* shared_out, const int* rev, const void* expanded_softmax,
                               int n_tokens, int top_k, int row_bytes, void* out, cudaStream_t stream);
// dst[0] = a, dst[1] = b (a one-group offsets array written in stream order)
cudaError_t moe_set_range_launch(int* dst, int a, int b, cudaStream_t stream);
cudaError_t moe_tile_list_launch(const int* offsets, int n_groups, int* tile_group, int* tile_row0, int* tile_chunk,
                                 int* tile_count, cudaStream_t stream);

// ---- expert-parallel exchange over peer memory (moe_ep.cu)
struct PeerPtrs {
    void* p[8];
};
#ifdef __CUDACC__
// One of the (at most 8) peer pointers, selected without indexing the kernel-parameter struct dynamically
// (which would force a copy of the struct into local memory).
__device__ __forceinline__ void* pick_peer(const PeerPtrs& pp, int q) {
    void* r = pp.p[0];
#pragma unroll
    for (int i = 1; i < 8; ++i)
        if (q == i) r = pp.p[i];
    return r;
}
#endif
// counts_all [world][n_experts] (row s = pairs per global expert on source rank s).  Writes
//   send_base[e]      row, inside the owner rank's receive buffer, of this rank's first pair for expert e
//   recv_offsets[j]   j = 0..n_experts/world: row range of local expert j in this rank's receive buffer
// Row ranges are clipped to `capacity` (rows of the receive buffers); an overflow ORs kDiagEpOverflow into
// the diagnostics word of `status`.
cudaError_t moe_ep_layout_launch(const int* counts_all, int rank, int world, int n_experts, int capacity,
                                 int* send_base, int* recv_offsets, int* status, cudaStream_t stream);
// Copies the token row of every local (token, expert) pair into the owner rank's receive buffer
// (peer stores) and records where it went (pair_rank, pair_row).  With `recv_meta` != nullptr it also
// writes, beside every row it sends, the return address of the row's result: (this rank << 28) | p, p = the
// pair's position in this rank's expert-sorted order (kEpMetaSlotBits bits).
// A pair whose destination row is >= `capacity` is not sent: pair_rank = -1, kDiagEpOverflow is raised, and
// with `drop_fill` != nullptr (this rank's fp16 [n_pairs, row] result matrix) its result row is zeroed.
// `max_blocks` > 0 caps the grid (to leave SMs to a GEMM running beside it).
constexpr int kEpMetaSlotBits = 28;
cudaError_t moe_ep_dispatch_launch(const void* x, const int* permuted_experts, const int* permuted_rows,
                                   const int* first_token_offset, const int* send_base, int n_tokens, int n_pairs,
                                   int row_bytes, int experts_per_rank, int rank, int world, int capacity,
                                   const PeerPtrs& recv_x, const PeerPtrs* recv_meta, int* pair_rank, int* pair_row,
                                   void* drop_fill, int* status, int num_sms, int max_blocks, cudaStream_t stream);
// out[t] = fp16(sum_i w_i * Y_{rank_i}[row_i] + shared[t]) with Y rows read from the owner ranks (peer loads).
cudaError_t moe_ep_combine_launch(const PeerPtrs& y, const void* shared_out, const int* rev, const void* weights,
                                  const int* pair_rank, const int* pair_row, int n_tokens, int top_k, int row_bytes,
                                  void* out, cudaStream_t stream);

// out[i] = fp16(out[i] + add[i]) over n_elems fp16 values (n_elems % 8 == 0)
cudaError_t moe_add_rows_launch(void* out, const void* add, size_t n_elems, int num_sms, cudaStream_t stream);

// Cross-GPU rendezvous through peer memory.  `sync` = every rank's sync area (int32): words [0, 8) are
// arrival flags (slot s is written by rank s), words [8, 8 + world * n_counts) an all-gather area.
// Each rank stores `epoch` into its slot on every peer and waits (bounded) until its own slots hold
// `epoch`; with `counts` != nullptr it first publishes its n_counts values into row `rank` of every
// peer's gather area.  One launch per rank, every rank on its own GPU.
// `from_offsets`: `counts` holds n_counts + 1 ascending offsets and their differences are published.
cudaError_t moe_ep_rendezvous_launch(const PeerPtrs& sync, const int* counts, int n_counts, bool from_offsets,
                                     int rank, int world, int epoch, int* status, cudaStream_t stream);

// ---- grouped fp16 GEMM (moe_gemm.cu)
enum MoeGemmMode {
    kMoeGemmPlain = 0,    // out[r, n] = fp16(X[r,:] . W_g[:, n]); W_g is [K, N] row-major (N contiguous)
    kMoeGemmSwiglu = 1,   // out[r, n] = fp16(SiLU(fp16(X.Wa_g)) * fp16(X.Wb_g))
    kMoeGemmRouter = 2,   // out[r, n] = fp16(X[r,:] . W[n,:] + bias[n]); W is [N, K] row-major (K contiguous)
};

// Largest run of row tiles of one group that the grouped GEMM walks together (see tile_list_kernel).
constexpr int kMoeChunkTiles = 16;

struct MoeGemmParams {
    const int* tile_group;      // [n_tiles] group (expert) of each 128-row tile
    const int* tile_row0;       // [n_tiles] first row of the tile
    const int* tile_chunk;      // [n_tiles] (first tile of the tile's chunk << 8) | tiles in the chunk
    const int* tile_count;      // [1]
    const int* group_offsets;   // [n_groups + 1] row range of each group
    const CUtensorMap* b_maps;  // device array, one tensor map per group (first weight)
    const CUtensorMap* b2_maps; // second weight per group (SwiGLU mode), else unused
    const float* bias;          // router mode: optional fp32 [n_out]
    void* out;                  // fp16 [rows, n_out]
    // Plain mode only, optional: row r of the result is stored to row (scatter_meta[r] & slot mask) of the
    // fp16 [*, n_out] matrix scatter_dst.p[scatter_meta[r] >> kEpMetaSlotBits] instead of out[r] (peer stores:
    // the expert outputs travel back to the GPUs that own the tokens from the GEMM's own epilogue).
    const int* scatter_meta;
    PeerPtrs scatter_dst;
    // SwiGLU mode only, optional: row r of the A operand is row (gather_map[min(r, gather_rows - 1)] % gather_mod)
    // of the fp16 [gather_mod, k] matrix gather_src (the token rows, read in place: the row gather of
    // expand_input, src/moe/moe_topk_kernel.cpp:174-213, done by the GEMM's own loader); tma_a is then unused.
    const void* gather_src;
    const int* gather_map;
    int gather_mod;
    int gather_rows;
    int n_out;                  // output columns
    int k;                      // reduction length (multiple of 64)
    int tma_store;              // 1: full 32-row slabs leave through the output tensor map
    int* status;                // device status area (status_words.h)
    int launch_tag;             // tag recorded with an expired wait
};

cudaError_t moe_gemm_launch(int mode, const CUtensorMap& tma_a, const CUtensorMap& tma_out, const MoeGemmParams& p,
                            int num_sms, cudaStream_t stream);
// Output columns covered by one tile in the given mode (256, or 128 for SwiGLU).
int moe_gemm_tile_n(int mode);

}  // namespace rf
