// Peer-memory plumbing and the expert-parallel C-ABI entry points (declared in include/rf_b200.h).
// Buffers that other GPUs of the node read or write are plain cudaMalloc allocations exported with
// CUDA IPC handles; one process per GPU opens its peers' handles once at set-up.
#include "../../include/rf_b200.h"
#include "host_util.h"
#include "moe_kernels.h"

#include <cstring>

extern "C" {

int rf_peer_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
    if (!ptr || !handle64 || bytes == 0) return RF_ERR_NULL_POINTER;
    if (!rf::device_state()) return RF_ERR_CUDA;
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); return RF_ERR_CUDA; }
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) { cudaGetLastError(); cudaFree(p); return RF_ERR_CUDA; }
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(handle64, &h, 64);
    *ptr = p;
    return RF_OK;
}

int rf_peer_open(const unsigned char* handle64, void** ptr) {
    if (!ptr || !handle64) return RF_ERR_NULL_POINTER;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return RF_ERR_CUDA; }
    *ptr = p;
    return RF_OK;
}

int rf_peer_close(void* ptr) {
    if (!ptr) return RF_ERR_NULL_POINTER;
    return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? RF_OK : RF_ERR_CUDA;
}

int rf_peer_free(void* ptr) {
    if (!ptr) return RF_ERR_NULL_POINTER;
    return cudaFree(ptr) == cudaSuccess ? RF_OK : RF_ERR_CUDA;
}

int rf_moe_add_rows(void* out, const void* add, int n_rows, int d_hidden, rf_stream_t stream) {
    if (!out || !add) return RF_ERR_NULL_POINTER;
    if (n_rows < 0 || d_hidden <= 0 || d_hidden % 8 != 0) return RF_ERR_BAD_SHAPE;
    rf::DeviceState* st = rf::device_state();
    if (!st) return RF_ERR_CUDA;
    return rf::moe_add_rows_launch(out, add, (size_t)n_rows * d_hidden, st->num_sms,
                                   reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess
               ? RF_OK : RF_ERR_CUDA;
}

int rf_moe_ep_rendezvous(void* const* sync_all, const int* counts_dev, int n_counts, int rank, int world, int epoch,
                         rf_stream_t stream) {
    if (!sync_all) return RF_ERR_NULL_POINTER;
    if (world < 1 || world > 8 || rank < 0 || rank >= world || n_counts < 0 || epoch <= 0) return RF_ERR_BAD_SHAPE;
    rf::DeviceState* st = rf::device_state();
    if (!st) return RF_ERR_CUDA;
    rf::PeerPtrs pp;
    for (int i = 0; i < 8; ++i) pp.p[i] = sync_all[i < world ? i : 0];
    for (int i = 0; i < world; ++i)
        if (!pp.p[i] || ((uintptr_t)pp.p[i] & 15)) return RF_ERR_NULL_POINTER;
    return rf::moe_ep_rendezvous_launch(pp, counts_dev, counts_dev ? n_counts : 0, false, rank, world, epoch,
                                        st->status, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess
               ? RF_OK : RF_ERR_CUDA;
}

int rf_moe_ep_layout(const int* counts_all_dev, int rank, int world, int n_experts, int capacity, int* send_base_dev,
                     int* recv_offsets_dev, rf_stream_t stream) {
    if (!counts_all_dev || !send_base_dev || !recv_offsets_dev) return RF_ERR_NULL_POINTER;
    if (world < 1 || world > 8 || rank < 0 || rank >= world || n_experts < world || n_experts > 1024 ||
        n_experts % world != 0 || capacity < 1)
        return RF_ERR_BAD_SHAPE;
    rf::DeviceState* st = rf::device_state();
    if (!st) return RF_ERR_CUDA;
    return rf::moe_ep_layout_launch(counts_all_dev, rank, world, n_experts, capacity, send_base_dev, recv_offsets_dev,
                                    st->status, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess
               ? RF_OK : RF_ERR_CUDA;
}

int rf_moe_ep_dispatch(const void* x, const int* permuted_experts, const int* permuted_rows,
                       const int* first_token_offset, const int* send_base, int n_tokens, int n_pairs, int d_hidden,
                       int n_experts, int rank, int world, int capacity, void* const* recv_x_all,
                       void* const* recv_meta_all, int* pair_rank, int* pair_row, void* drop_fill, rf_stream_t stream) {
    if (!x || !permuted_experts || !permuted_rows || !first_token_offset || !send_base || !recv_x_all || !pair_rank ||
        !pair_row)
        return RF_ERR_NULL_POINTER;
    if (world < 1 || world > 8 || rank < 0 || rank >= world || n_experts % world != 0 || d_hidden <= 0 ||
        d_hidden % 8 != 0 || n_tokens <= 0 || n_pairs < 0 || capacity < 1)
        return RF_ERR_BAD_SHAPE;
    rf::DeviceState* st = rf::device_state();
    if (!st) return RF_ERR_CUDA;
    rf::PeerPtrs pp;
    for (int i = 0; i < 8; ++i) pp.p[i] = recv_x_all[i < world ? i : 0];
    for (int i = 0; i < world; ++i)
        if (!pp.p[i] || ((uintptr_t)pp.p[i] & 15)) return RF_ERR_NULL_POINTER;
    rf::PeerPtrs pm;
    if (recv_meta_all) {
        if (n_pairs >= (1 << rf::kEpMetaSlotBits)) return RF_ERR_BAD_SHAPE;
        for (int i = 0; i < 8; ++i) pm.p[i] = recv_meta_all[i < world ? i : 0];
        for (int i = 0; i < world; ++i)
            if (!pm.p[i] || ((uintptr_t)pm.p[i] & 3)) return RF_ERR_NULL_POINTER;
    }
    return rf::moe_ep_dispatch_launch(x, permuted_experts, permuted_rows, first_token_offset, send_base, n_tokens,
                                      n_pairs, d_hidden * 2, n_experts / world, rank, world, capacity, pp,
                                      recv_meta_all ? &pm : nullptr, pair_rank, pair_row, drop_fill, st->status,
                                      st->num_sms, 0, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess
               ? RF_OK : RF_ERR_CUDA;
}

int rf_moe_ep_combine(void* const* y_all, const void* shared_fc2_output, const int* rev_permuted_rows,
                      const void* expanded_seq_softmax, const int* pair_rank, const int* pair_row, int n_tokens,
                      int top_k, int d_hidden, int world, void* final_output, rf_stream_t stream) {
    if (!y_all || !rev_permuted_rows || !expanded_seq_softmax || !pair_rank || !pair_row || !final_output)
        return RF_ERR_NULL_POINTER;
    if (world < 1 || world > 8 || top_k < 1 || top_k > 8 || d_hidden <= 0 || d_hidden % 8 != 0 || n_tokens < 0)
        return RF_ERR_BAD_SHAPE;
    rf::PeerPtrs pp;
    for (int i = 0; i < 8; ++i) pp.p[i] = y_all[i < world ? i : 0];
    for (int i = 0; i < world; ++i)
        if (!pp.p[i] || ((uintptr_t)pp.p[i] & 15)) return RF_ERR_NULL_POINTER;
    return rf::moe_ep_combine_launch(pp, shared_fc2_output, rev_permuted_rows, expanded_seq_softmax, pair_rank,
                                     pair_row, n_tokens, top_k, d_hidden * 2, final_output,
                                     reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess
               ? RF_OK : RF_ERR_CUDA;
}

}  // extern "C"
