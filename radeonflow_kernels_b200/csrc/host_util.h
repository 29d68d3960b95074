// Host-side helpers shared by the C-ABI translation units: per-device state
// (SM count, status word, growable scratch), tensor-map encoding through the
// driver entry point (no link-time dependency on libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "status_words.h"

namespace rf {

constexpr int kMaxDevices = 64;

struct DeviceState {
    bool init = false;
    int num_sms = 0;
    int* status = nullptr;          // device status area: kStatusWords 32-bit words (layout in status_words.h)
    void* scratch[4] = {nullptr, nullptr, nullptr, nullptr};   // library-owned growable buffers, see ScratchSlot
    size_t scratch_bytes[4] = {0, 0, 0, 0};
};


enum ScratchSlot {
    kScratchGemm = 0,      // split-K slices / stream-K slots and flags of the FP8 GEMM
    kScratchMoeAux = 1,    // MoE tile lists and sort counters
    kScratchMoeWork = 2,   // MoE intermediates handed out by initialize_workspace
    kScratchFnuz = 3,      // e4m3fn copies of e4m3fnuz operands (reference-format GEMM entry)
    kScratchSlots = 4,
};

// State of the current device; initialises it on first use (allocates the
// 4-byte status word).  Returns nullptr when a CUDA call fails.
DeviceState* device_state();

// A fresh tag (1 .. kStatusTagMask) for the next kernel launch that records expired waits.
int next_launch_tag();

// A fresh non-zero number for the flags of the next stream-K launch (flags that carry another number are stale).
unsigned next_streamk_epoch();

// Library-owned buffer `slot` of at least `bytes` on the current device (grows by
// freeing and re-allocating; synchronises the device when it grows).
void* device_scratch(size_t bytes, int slot = kScratchGemm);

// 2-D row-major tensor map: `rows` x `cols` elements of `elem_bytes`, row
// pitch `pitch_bytes`; box = box_rows x box_cols; 128-byte swizzle when
// `swizzle128`.  dtype is one of CU_TENSOR_MAP_DATA_TYPE_*.
bool encode_tma_2d(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void* base,
                   uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols,
                   bool swizzle128);

// 3-D tensor map over a dense [d2][d1][d0] array (d0 contiguous); box = {b0, b1, 1}.
bool encode_tma_3d(CUtensorMap* map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void* base, uint64_t d0,
                   uint64_t d1, uint64_t d2, uint32_t b0, uint32_t b1, bool swizzle128);

}  // namespace rf
