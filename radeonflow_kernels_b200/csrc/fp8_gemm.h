// Internal interface between the C-ABI layer and the FP8 GEMM kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stddef.h>

namespace rf {

struct GemmParams {
    const float* a_scale;   // [m, k/128]
    const float* b_scale;   // [ceil(n/128), k/128]
    __nv_bfloat16* c;       // [m, n]
    float* partial;         // [splits, m, n] fp32 when splits > 1
    int* status;            // device status area (status_words.h)
    int launch_tag;         // tag recorded with an expired wait (host_util: next_launch_tag)
    int m, n, k;
    int tiles_m, tiles_n, splits;
    // Scale addressing: a_scale[row * as_row_stride + kb * as_k_stride] (row-major [m, k/128]: (k/128, 1);
    // the reference's physical layout [k/128][m]: (1, m)); same for b_scale with its block row.
    long long as_row_stride, as_k_stride, bs_row_stride, bs_k_stride;
    int n_dest;             // copies of C to write (1, or the number of GPUs of an N-split GEMM)
    int c_col_offset;       // column of this GEMM's C inside each destination matrix
    // (Measured on B200: with 16 more bytes of kernel parameters the short kernels ran 0.3-0.4 us slower per
    // launch, so the struct stays at 128 bytes.  The two members of the union are never used by one launch.)
    union {
        const int* fnuz_flags;          // nullptr, or two device words left by the e4m3fnuz conversion pass
                                        // (reference-layout entry only): [0] / [1] != 0 = read A / B from the
                                        // converted copy (dests.m[0] / m[1])
        unsigned long long sk_token;    // stream-K: the value of a raised flag in this launch
    };
    int dest_first;         // first destination to store to (N-split: own rank, so ranks target different GPUs)
    // Stream-K (splits == 1, row-major operands, one destination): the last sk_tiles tiles are shared out by K
    // blocks over all CTAs of the grid (which then has exactly num_sms CTAs).  `partial` holds one 128 x block_n
    // fp32 slot per CTA, followed by one 64-bit flag per CTA; a flag is raised when it holds sk_token and is
    // cleared by the CTA that consumes it, so stale contents never pass for a raised flag.
    int sk_tiles;
    GemmParams() : fnuz_flags(nullptr), sk_tiles(0) {}
};
static_assert(sizeof(GemmParams) == 128, "kernel parameter block of the GEMM");

// Output tensor maps of an N-split GEMM: entry d addresses GPU d's full row-major C.
struct GemmDestMaps {
    CUtensorMap m[8];
};

// Tile configurations, named by `block_n`: 128 and 256 are one-CTA tiles 128 x block_n; 512 and 384 are the
// CTA-pair configurations (256 x 256 and 256 x 128 per 2-CTA cluster, each CTA loading 128 rows of A and
// half of the tile's rows of B).
inline bool gemm_is_pair(int block_n) { return block_n == 512 || block_n == 384; }
inline int gemm_tile_rows(int block_n) { return gemm_is_pair(block_n) ? 256 : 128; }
inline int gemm_tile_cols(int block_n) { return block_n == 512 ? 256 : (block_n == 384 ? 128 : block_n); }
inline int gemm_b_box_rows(int block_n) { return block_n == 512 ? 128 : (block_n == 384 ? 64 : block_n); }

// Scratch a stream-K launch needs: per CTA one fp32 tile slot, then one 64-bit flag per CTA.
inline size_t gemm_streamk_slot_bytes(int block_n) { return (size_t)128 * gemm_tile_cols(block_n) * sizeof(float); }
// Value of a raised stream-K flag: a fixed upper half and a per-launch number (never 0).
inline unsigned long long gemm_streamk_token(unsigned epoch) { return 0x5246534B00000000ull | epoch; }
inline size_t gemm_streamk_bytes(int block_n, int num_sms) {
    return (size_t)num_sms * (gemm_streamk_slot_bytes(block_n) + sizeof(unsigned long long));
}
// Tiles of the stream-K region for `tiles` tiles on `num_sms` CTAs: the ragged last wave plus one full wave
// (every CTA then gets between one and two tiles' worth of K blocks), or everything when there is less than
// one wave; 0 when the tiles fill whole waves.
inline int gemm_streamk_tiles(int tiles, int num_sms) {
    const int rem = tiles % num_sms;
    if (rem == 0) return 0;
    return tiles < num_sms ? tiles : rem + num_sms;
}

// Launches the GEMM (and the split-K fix-up when p.splits > 1) on `stream`.
// `block_n` is the configuration the tensor map of B and p.tiles_m / p.tiles_n were built for.
// `tma_c` stores bf16 C boxes of 32 rows x 64 columns; `tma_p` (used when p.splits > 1) stores fp32
// slice boxes of 32 rows x 32 columns into the [splits][m][n] scratch.
// When p.n_dest > 1, `dests` holds p.n_dest maps and replaces tma_c (split-K is not combined with it).
// `mn_major`: A and B are stored [k][m] / [k][n] (the reference's physical layout); their tensor maps then
// have boxes of 128 K-rows x 128 elements of M/N and block_n must be 128 or 256.
cudaError_t fp8_gemm_launch(const CUtensorMap& tma_a, const CUtensorMap& tma_b, const CUtensorMap& tma_c,
                            const CUtensorMap& tma_p, const GemmDestMaps* dests, const GemmParams& p, int block_n,
                            int num_sms, cudaStream_t stream, bool mn_major = false);

// The pieces (tile, K slice, first K block, end K block: four ints each) that CTA `unit` of `n_units` works
// through for launch parameters `p`, in order, computed on the host by the same code the kernel runs (only
// p.k, p.tiles_m, p.tiles_n, p.splits and p.sk_tiles are read).  Returns the number of pieces; at most
// `max_pieces` are written.
int fp8_gemm_walk_pieces(const GemmParams& p, int unit, int n_units, int* out, int max_pieces);

// One pass over `n_bytes` (multiple of 16) of e4m3fnuz data: writes the e4m3fn bytes of equal value to `dst`
// and sets *flag (device word, cleared first) when the operand holds a byte that cannot be consumed as it
// is (0x80, 0x7F, 0xFF); in that case kDiagFnuzByte is also OR-ed into the diagnostics word of `status`.
cudaError_t fp8_fnuz_convert_launch(const void* src, void* dst, size_t n_bytes, int* flag, int* status, int num_sms,
                                    cudaStream_t stream);

// Sets the launch attributes of every GEMM kernel configuration on the current device (normally done
// lazily by the first launch of each configuration).
cudaError_t fp8_gemm_prepare_device();

// The tile width (128 or 256) and K-slice count the library uses for this shape on a device with
// `num_sms` SMs; `split_k` > 0 forces the slice count.
void fp8_gemm_plan(int m, int n, int k, int num_sms, int split_k, int* block_n, int* splits);

// Exact-shape entry of the tuned-plan table (built-in, registered or loaded from a file); false = none.
bool tuned_plan_lookup(int m, int n, int k, int* block_n, int* splits);

}  // namespace rf
