#include "host_util.h"

#include <cudaTypedefs.h>
#include <atomic>
#include <cstdio>
#include <mutex>

namespace rf {

namespace {
DeviceState g_dev[kMaxDevices];
std::mutex g_mu;
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;

bool load_encode() {
    if (g_encode) return true;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) return false;
    g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    return true;
}
}  // namespace

DeviceState* device_state() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    DeviceState* st = &g_dev[dev];
    if (st->init) return st;
    std::lock_guard<std::mutex> lock(g_mu);
    if (st->init) return st;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return nullptr;
    if (prop.major != 10) {
        fprintf(stderr, "rf_b200: device %d is sm_%d%d; this library contains sm_100a code only\n", dev, prop.major,
                prop.minor);
        return nullptr;
    }
    st->num_sms = prop.multiProcessorCount;
    if (cudaMalloc(&st->status, sizeof(int) * kStatusWords) != cudaSuccess) return nullptr;
    if (cudaMemset(st->status, 0, sizeof(int) * kStatusWords) != cudaSuccess) return nullptr;
    if (!load_encode()) return nullptr;
    st->init = true;
    return st;
}

int next_launch_tag() {
    static std::atomic<unsigned> counter{0};
    return (int)(counter.fetch_add(1, std::memory_order_relaxed) % (unsigned)kStatusTagMask) + 1;
}

unsigned next_streamk_epoch() {
    static std::atomic<unsigned> counter{0};
    unsigned v;
    do v = counter.fetch_add(1, std::memory_order_relaxed) + 1; while (v == 0);
    return v;
}

void* device_scratch(size_t bytes, int slot) {
    DeviceState* st = device_state();
    if (!st || slot < 0 || slot >= kScratchSlots) return nullptr;
    if (bytes <= st->scratch_bytes[slot]) return st->scratch[slot];
    std::lock_guard<std::mutex> lock(g_mu);
    if (bytes <= st->scratch_bytes[slot]) return st->scratch[slot];
    // Work already queued may still use the old buffer.
    if (cudaDeviceSynchronize() != cudaSuccess) return nullptr;
    if (st->scratch[slot]) cudaFree(st->scratch[slot]);
    st->scratch[slot] = nullptr;
    st->scratch_bytes[slot] = 0;
    size_t want = bytes + (bytes >> 2);  // 25 % head-room so slowly growing shapes do not thrash
    if (cudaMalloc(&st->scratch[slot], want) != cudaSuccess) {
        cudaGetLastError();
        if (cudaMalloc(&st->scratch[slot], bytes) != cudaSuccess) return nullptr;
        want = bytes;
    }
    st->scratch_bytes[slot] = want;
    return st->scratch[slot];
}

bool encode_tma_2d(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void* base,
                   uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols,
                   bool swizzle128) {
    if (!load_encode()) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    (void)elem_bytes;
    CUresult r = g_encode(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

bool encode_tma_3d(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void* base, uint64_t d0,
                   uint64_t d1, uint64_t d2, uint32_t b0, uint32_t b1, bool swizzle128) {
    if (!load_encode()) return false;
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {d0 * elem_bytes, d0 * d1 * elem_bytes};
    cuuint32_t box[3] = {b0, b1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = g_encode(map, dtype, 3, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace rf
