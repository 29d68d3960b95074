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

size_t fp8_gemm_smem_bytes();
int fp8_gemm_block_n();

// Launches the GEMM (and the split-K fix-up when p.splits > 1) on `stream`.
cudaError_t fp8_gemm_launch(const CUtensorMap& tma_a, const CUtensorMap& tma_b, const GemmParams& p, int num_sms,
                            cudaStream_t stream);

}  // namespace rf
