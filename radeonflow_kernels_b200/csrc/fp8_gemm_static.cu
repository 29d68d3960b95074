// FP8 block-scaled GEMM for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc on the path where the GEMM runs: code inside a
// CUDA-graph capture or replay loop, a real-time serving thread that may not take the allocator's
// locks or trigger an implicit device synchronisation, and embedders whose memory is fully owned by
// another allocator (an inference server's arena, a framework pool) and who cannot hand this
// library a scratch pointer through their operator interface.  The ordinary entry points either
// grow a library-owned buffer with cudaMalloc (`run`) or need a caller buffer (`rf_fp8_gemm`).
//
// This variant keeps the split-K slices in a fixed array that is part of the loaded module, so the
// memory exists as soon as the library is loaded on a GPU and is never allocated or freed at run time.
// The price is a fixed ceiling and a buffer that every call on the device shares.
#include "../../include/rf_b200.h"
#include "fp8_gemm.h"
#include "host_util.h"

#include <atomic>
#include <cstdio>
#include <mutex>

namespace {

// 16 MiB per GPU that loads the library, held until the process exits.
constexpr size_t kStaticScratchBytes = RF_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) float g_static_scratch[kStaticScratchBytes / sizeof(float)];
// Device status area of this path (same four-word layout as the library's other status area: expired-wait
// code, diagnostic flags, wait limit); zero when the module loads.  rf_fp8_gemm_static_status reads and clears it.
static __device__ __align__(16) int g_static_status[rf::kStatusWords];

struct StaticDevice {
    std::atomic<bool> ready{false};
    float* scratch = nullptr;   // DEVICE address of g_static_scratch on this device
    int* status = nullptr;      // DEVICE address of g_static_status on this device
    int num_sms = 0;
};
StaticDevice g_static_dev[rf::kMaxDevices];
std::mutex g_static_mu;

// Once per device, with that device current.  In host code `g_static_scratch` names a host-side
// shadow of the symbol, not device memory; the address a kernel may use comes from
// cudaGetSymbolAddress and differs per device.
int static_setup(StaticDevice** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= rf::kMaxDevices) return RF_ERR_CUDA;
    StaticDevice* sd = &g_static_dev[dev];
    if (!sd->ready.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_static_mu);
        if (!sd->ready.load(std::memory_order_relaxed)) {
            int major = 0, sms = 0;
            if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
                cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
                return RF_ERR_CUDA;
            if (major != 10) {
                fprintf(stderr, "rf_b200: device %d is not sm_100; this library contains sm_100a code only\n", dev);
                return RF_ERR_UNSUPPORTED;
            }
            void* p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
            if (e != cudaSuccess || !p) {
                fprintf(stderr, "rf_b200: cudaGetSymbolAddress(static scratch) failed: %s\n", cudaGetErrorString(e));
                return RF_ERR_CUDA;
            }
            void* s = nullptr;
            e = cudaGetSymbolAddress(&s, g_static_status);
            if (e != cudaSuccess || !s) {
                fprintf(stderr, "rf_b200: cudaGetSymbolAddress(static status) failed: %s\n", cudaGetErrorString(e));
                return RF_ERR_CUDA;
            }
            if (rf::fp8_gemm_prepare_device() != cudaSuccess) return RF_ERR_CUDA;
            sd->scratch = static_cast<float*>(p);
            sd->status = static_cast<int*>(s);
            sd->num_sms = sms;
            sd->ready.store(true, std::memory_order_release);
        }
    }
    *out = sd;
    return RF_OK;
}

}  // namespace

extern "C" int rf_fp8_gemm_static_scratch(const void* a, const void* b, const float* as, const float* bs, void* c,
                                          int m, int n, int k, int split_k, rf_stream_t stream) {
    if (m <= 0 || n <= 0 || k <= 0 || (n % 64) != 0 || (k % 128) != 0) return RF_ERR_BAD_SHAPE;
    if (!a || !b || !as || !bs || !c) return RF_ERR_NULL_POINTER;
    if (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15) return RF_ERR_MISALIGNED;
    if (((uintptr_t)as | (uintptr_t)bs) & 3) return RF_ERR_MISALIGNED;
    StaticDevice* sd = nullptr;
    int rc = static_setup(&sd);
    if (rc != RF_OK) return rc;

    if (split_k < -1) return RF_ERR_BAD_SHAPE;
    int bn = 128, splits = 1;
    rf::fp8_gemm_plan(m, n, k, sd->num_sms, split_k, &bn, &splits);
    const bool streamk = splits == -1;      // one pass, ragged last wave shared out by K blocks
    size_t need = streamk ? rf::gemm_streamk_bytes(bn, sd->num_sms)
                          : (splits > 1 ? (size_t)splits * m * n * sizeof(float) : 0);
    if (need > kStaticScratchBytes && split_k == 0) {
        // the library's own choice must fit the built-in array: fall back to the plain single pass
        rf::fp8_gemm_plan(m, n, k, sd->num_sms, 1, &bn, &splits);
        need = 0;
    }
    if (need > kStaticScratchBytes) {
        fprintf(stderr,
                "rf_fp8_gemm_static_scratch: %d K slices of a %d x %d result need %zu bytes of scratch, the built-in "
                "array holds %zu; pass a smaller split_k (1 needs none) or use rf_fp8_gemm with your own buffer\n",
                splits, m, n, need, kStaticScratchBytes);
        return RF_ERR_WORKSPACE;
    }

    CUtensorMap ta, tb, tc, tp;
    if (!rf::encode_tma_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, (uint64_t)m, (uint64_t)k, (uint64_t)k, 128, 128,
                           true) ||
        !rf::encode_tma_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b, (uint64_t)n, (uint64_t)k, (uint64_t)k,
                           (uint32_t)rf::gemm_b_box_rows(bn), 128, true) ||
        !rf::encode_tma_2d(&tc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, c, (uint64_t)m, (uint64_t)n, (uint64_t)n * 2, 32,
                           64, true))
        return RF_ERR_CUDA;
    if (splits > 1) {
        if (!rf::encode_tma_3d(&tp, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, sd->scratch, (uint64_t)n, (uint64_t)m,
                               (uint64_t)splits, 32, 32, true))
            return RF_ERR_CUDA;
    } else {
        tp = tc;
    }
    rf::GemmParams p;
    p.a_scale = as;
    p.b_scale = bs;
    p.c = static_cast<__nv_bfloat16*>(c);
    p.partial = splits > 1 ? sd->scratch : nullptr;   // every element of the slices is overwritten: nothing to clear
    p.status = sd->status;
    p.launch_tag = rf::next_launch_tag();
    p.m = m; p.n = n; p.k = k;
    p.tiles_m = (m + rf::gemm_tile_rows(bn) - 1) / rf::gemm_tile_rows(bn);
    p.tiles_n = (n + rf::gemm_tile_cols(bn) - 1) / rf::gemm_tile_cols(bn);
    p.splits = splits > 1 ? splits : 1;
    if (splits == -1) {
        p.partial = sd->scratch;
        p.sk_tiles = rf::gemm_streamk_tiles(p.tiles_m * p.tiles_n, sd->num_sms);
        p.sk_token = rf::gemm_streamk_token(rf::next_streamk_epoch());
    }
    p.as_row_stride = k / 128; p.as_k_stride = 1;
    p.bs_row_stride = k / 128; p.bs_k_stride = 1;
    p.n_dest = 1;
    p.c_col_offset = 0;
    p.dest_first = 0;
    cudaError_t e = rf::fp8_gemm_launch(ta, tb, tc, tp, nullptr, p, bn, sd->num_sms,
                                        reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        fprintf(stderr, "rf_fp8_gemm_static_scratch: launch failed: %s\n", cudaGetErrorString(e));
        return RF_ERR_CUDA;
    }
    return RF_OK;
}

// Reads and clears the status area of the allocation-free path (a copy from and to the symbol's device
// address; no allocation).  Synchronises the device, like rf_device_status.
extern "C" int rf_fp8_gemm_static_status(int* detail) {
    StaticDevice* sd = nullptr;
    int rc = static_setup(&sd);
    if (rc != RF_OK) return rc;
    int v[2] = {0, 0};
    if (cudaDeviceSynchronize() != cudaSuccess) return RF_ERR_CUDA;
    if (cudaMemcpy(v, sd->status, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return RF_ERR_CUDA;
    if (detail) *detail = v[0] != 0 ? (v[0] & 0xFF) : v[1];
    if (v[0] != 0 || v[1] != 0) {
        const int zero[2] = {0, 0};
        if (cudaMemcpy(sd->status, zero, sizeof(zero), cudaMemcpyHostToDevice) != cudaSuccess) return RF_ERR_CUDA;
        return RF_ERR_DEVICE_TIMEOUT;
    }
    return RF_OK;
}
