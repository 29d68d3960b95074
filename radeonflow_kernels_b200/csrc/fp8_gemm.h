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
    int* status;            // device status word (0 = ok)
    int m, n, k;
    int tiles_m, tiles_n, splits;
};

// Launches the GEMM (and the split-K fix-up when p.splits > 1) on `stream`.
// `block_n` is the tile width the tensor map of B and p.tiles_n were built for: 128 or 256.
// `tma_c` stores bf16 C boxes of 32 rows x 64 columns; `tma_p` (used when p.splits > 1) stores fp32
// slice boxes of 32 rows x 32 columns into the [splits][m][n] scratch.
cudaError_t fp8_gemm_launch(const CUtensorMap& tma_a, const CUtensorMap& tma_b, const CUtensorMap& tma_c,
                            const CUtensorMap& tma_p, const GemmParams& p, int block_n, int num_sms,
                            cudaStream_t stream);

}  // namespace rf
