// Expert-parallel MoE layer as one host object (declared in include/rf_b200.h: rf_moe_ep_*).
//
// The reference sequences its single-GPU layer in C++ (run_topk_impl, src/moe/moe.cpp:129-339); this is the
// same kind of host code for the expert-parallel form: it owns every buffer of a step (the peer-visible
// ones are exported with CUDA IPC), a side stream, the events and the rendezvous epoch, and runs one step
//   router GEMM -> top-k -> stable sort -> rendezvous (pair counts all-gathered) -> layout ->
//   dispatch (side stream)  ||  shared expert (main stream) -> rendezvous -> routed fc1 -> routed fc2
//   (results pushed home from the epilogue, or left for the pulling combine) -> rendezvous -> combine
// with no host synchronisation, no allocation and no collective-library call inside the step.
#include "../../include/rf_b200.h"
#include "host_util.h"
#include "moe_kernels.h"

#include <cuda_fp16.h>

#include <cstdio>
#include <cstring>
#include <new>
#include <vector>

namespace {

constexpr int kPeerBuffers = 4;     // sync area, receive rows, result rows, return addresses
enum PeerBuf { kBufSync = 0, kBufRecvX = 1, kBufY = 2, kBufMeta = 3 };
constexpr int kMaxMarks = 12;

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

struct RfMoeEp {
    RfMoeEpConfig cfg;
    int device = -1;
    int E_loc = 0, n_pairs = 0, capacity = 0, fs = 0;
    bool push = false;
    bool connected = false;
    int epoch = 0;
    // one allocation for the local (non-peer) buffers
    char* local = nullptr;
    __half* scores = nullptr;
    int *idx = nullptr, *source_rows = nullptr, *perm_experts = nullptr, *perm_rows = nullptr, *first = nullptr,
        *rev = nullptr, *pair_rank = nullptr, *pair_row = nullptr, *send_base = nullptr, *recv_offsets = nullptr,
        *single_offsets = nullptr;
    __half *gate_w = nullptr, *exp_w = nullptr, *sh1 = nullptr, *sh2 = nullptr, *h = nullptr;
    void* sort_scratch = nullptr;
    // peer-visible buffers: mine and every rank's mapping
    void* mine[kPeerBuffers] = {nullptr, nullptr, nullptr, nullptr};
    size_t peer_bytes[kPeerBuffers] = {0, 0, 0, 0};
    void* all[kPeerBuffers][8] = {};
    bool opened[kPeerBuffers][8] = {};
    // weights
    const void* router_w = nullptr;
    const float* router_bias = nullptr;
    std::vector<const void*> w_gate, w_up, w_down;
    const void *s_gate = nullptr, *s_up = nullptr, *s_down = nullptr;
    cudaStream_t side = nullptr;
    cudaEvent_t ev_ready = nullptr, ev_sent = nullptr;
    // stage timing (optional)
    bool trace = false;
    cudaEvent_t marks[kMaxMarks] = {};
    int n_marks = 0;
    int dispatch_blocks = 0;     // > 0: dispatch grid cap; the shared expert's GEMMs then leave that many SMs free
};

namespace {

const char* const kMarkNames[kMaxMarks] = {"start",      "route+counts", "dispatch+shared", "barrier1", "routed fc1",
                                           "routed fc2", "barrier2",     "combine",         "",         "",
                                           "",           ""};

void mark(RfMoeEp* ep, cudaStream_t s) {
    if (ep->trace && ep->n_marks < kMaxMarks) cudaEventRecord(ep->marks[ep->n_marks++], s);
}

int rendezvous(RfMoeEp* ep, const int* offsets_or_null, cudaStream_t s) {
    rf::DeviceState* st = rf::device_state();
    if (!st) return RF_ERR_CUDA;
    rf::PeerPtrs pp;
    for (int i = 0; i < 8; ++i) pp.p[i] = ep->all[kBufSync][i < ep->cfg.world ? i : 0];
    ++ep->epoch;
    return rf::moe_ep_rendezvous_launch(pp, offsets_or_null, offsets_or_null ? ep->cfg.n_routed_experts : 0,
                                        offsets_or_null != nullptr, ep->cfg.rank, ep->cfg.world, ep->epoch, st->status,
                                        s) == cudaSuccess
               ? RF_OK : RF_ERR_CUDA;
}

void release(RfMoeEp* ep) {
    if (!ep) return;
    int prev = -1;
    cudaGetDevice(&prev);
    if (ep->device >= 0) cudaSetDevice(ep->device);
    cudaDeviceSynchronize();
    for (int b = 0; b < kPeerBuffers; ++b)
        for (int r = 0; r < 8; ++r)
            if (ep->opened[b][r]) cudaIpcCloseMemHandle(ep->all[b][r]);
    for (int b = 0; b < kPeerBuffers; ++b)
        if (ep->mine[b]) cudaFree(ep->mine[b]);
    if (ep->local) cudaFree(ep->local);
    if (ep->side) cudaStreamDestroy(ep->side);
    if (ep->ev_ready) cudaEventDestroy(ep->ev_ready);
    if (ep->ev_sent) cudaEventDestroy(ep->ev_sent);
    for (int i = 0; i < kMaxMarks; ++i)
        if (ep->marks[i]) cudaEventDestroy(ep->marks[i]);
    if (prev >= 0) cudaSetDevice(prev);
    delete ep;
}

}  // namespace

extern "C" {

int rf_moe_ep_create(const RfMoeEpConfig* c, RfMoeEp** out) {
    if (!c || !out) return RF_ERR_NULL_POINTER;
    *out = nullptr;
    if (c->world < 1 || c->world > 8 || c->rank < 0 || c->rank >= c->world) return RF_ERR_BAD_SHAPE;
    if (c->n_tokens <= 0 || c->d_hidden <= 0 || c->d_hidden % 64 != 0 || c->d_expert <= 0 || c->d_expert % 64 != 0)
        return RF_ERR_BAD_SHAPE;
    const int E = c->n_routed_experts, K = c->n_experts_per_token;
    if (E < 1 || E > 256 || (E & (E - 1)) != 0 || E % c->world != 0 || K < 1 || K > 8 || K > E ||
        c->n_shared_experts < 1)
        return RF_ERR_UNSUPPORTED;
    const long long pairs = (long long)c->n_tokens * K;
    if (pairs >= (1ll << rf::kEpMetaSlotBits) || pairs * c->world > 0x7fffffffll) return RF_ERR_BAD_SHAPE;
    if (c->capacity < 0) return RF_ERR_BAD_SHAPE;
    if (!rf::device_state()) return RF_ERR_CUDA;

    RfMoeEp* ep = new (std::nothrow) RfMoeEp();
    if (!ep) return RF_ERR_CUDA;
    ep->cfg = *c;
    cudaGetDevice(&ep->device);
    ep->E_loc = E / c->world;
    ep->n_pairs = (int)pairs;
    ep->capacity = c->capacity > 0 ? c->capacity : (int)(pairs * c->world);     // default: the worst case
    ep->fs = c->d_expert * c->n_shared_experts;
    ep->push = c->push_results != 0 && c->world > 1;     // on one GPU nothing travels: plain fc2 + gathering combine
    // On 2 to 4 GPUs the dispatch runs by default as 32 copy-engine blocks beside the shared expert's GEMMs
    // (measured: dispatch + shared expert 1.67 -> 1.25 ms on 4 GPUs, 2.90 -> 2.44 ms on 2).  On one GPU, where
    // nothing crosses NVLink, it keeps every SM; on 8 it does too (measured: 3.75 against 3.73 ms per layer with the
    // partition; RF_MOE_EP_OPT_DISPATCH_BLOCKS selects it).
    ep->dispatch_blocks = (c->world > 1 && c->world <= 4) ? 32 : 0;
    ep->w_gate.resize(ep->E_loc);
    ep->w_up.resize(ep->E_loc);
    ep->w_down.resize(ep->E_loc);

    const size_t T = c->n_tokens, d = c->d_hidden, f = c->d_expert, TK = (size_t)pairs, cap = ep->capacity;
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t o = off; off += align_up(bytes, 256); return o; };
    const size_t o_scores = take(T * E * 2), o_idx = take(TK * 4), o_gw = take(TK * 2), o_src = take(TK * 4),
                 o_pe = take(TK * 4), o_pr = take(TK * 4), o_first = take((E + 1) * 4), o_rev = take(TK * 4),
                 o_ew = take(TK * 2), o_prank = take(TK * 4), o_prow = take(TK * 4), o_sb = take(E * 4),
                 o_ro = take((ep->E_loc + 1) * 4), o_so = take(2 * 4), o_sh1 = take(T * ep->fs * 2),
                 o_sh2 = take(T * d * 2), o_h = take(cap * f * 2),
                 o_sort = take(rf_moe_permute_scratch_bytes((int)TK, E) + 16);
    if (cudaMalloc(&ep->local, off) != cudaSuccess) { cudaGetLastError(); release(ep); return RF_ERR_CUDA; }
    char* L = ep->local;
    ep->scores = reinterpret_cast<__half*>(L + o_scores);
    ep->idx = reinterpret_cast<int*>(L + o_idx);
    ep->gate_w = reinterpret_cast<__half*>(L + o_gw);
    ep->source_rows = reinterpret_cast<int*>(L + o_src);
    ep->perm_experts = reinterpret_cast<int*>(L + o_pe);
    ep->perm_rows = reinterpret_cast<int*>(L + o_pr);
    ep->first = reinterpret_cast<int*>(L + o_first);
    ep->rev = reinterpret_cast<int*>(L + o_rev);
    ep->exp_w = reinterpret_cast<__half*>(L + o_ew);
    ep->pair_rank = reinterpret_cast<int*>(L + o_prank);
    ep->pair_row = reinterpret_cast<int*>(L + o_prow);
    ep->send_base = reinterpret_cast<int*>(L + o_sb);
    ep->recv_offsets = reinterpret_cast<int*>(L + o_ro);
    ep->single_offsets = reinterpret_cast<int*>(L + o_so);
    ep->sh1 = reinterpret_cast<__half*>(L + o_sh1);
    ep->sh2 = reinterpret_cast<__half*>(L + o_sh2);
    ep->h = reinterpret_cast<__half*>(L + o_h);
    ep->sort_scratch = L + o_sort;
    const int so[2] = {0, c->n_tokens};
    if (cudaMemcpy(ep->single_offsets, so, sizeof(so), cudaMemcpyHostToDevice) != cudaSuccess) {
        release(ep);
        return RF_ERR_CUDA;
    }

    // peer-visible buffers.  Results: with the push variant one row per LOCAL pair (expert-sorted order),
    // otherwise one row per received row.
    ep->peer_bytes[kBufSync] = 4 * (8 + (size_t)c->world * E);
    ep->peer_bytes[kBufRecvX] = cap * d * 2;
    ep->peer_bytes[kBufY] = (ep->push ? TK : cap) * d * 2;
    ep->peer_bytes[kBufMeta] = 4 * cap;
    for (int b = 0; b < kPeerBuffers; ++b) {
        if (cudaMalloc(&ep->mine[b], align_up(ep->peer_bytes[b], 256)) != cudaSuccess) {
            cudaGetLastError();
            release(ep);
            return RF_ERR_CUDA;
        }
        ep->all[b][c->rank] = ep->mine[b];
    }
    // the flags and the count matrix start at zero, before any rank's first epoch
    if (cudaMemset(ep->mine[kBufSync], 0, ep->peer_bytes[kBufSync]) != cudaSuccess ||
        cudaStreamCreateWithFlags(&ep->side, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&ep->ev_ready, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&ep->ev_sent, cudaEventDisableTiming) != cudaSuccess) {
        release(ep);
        return RF_ERR_CUDA;
    }
    for (int i = 0; i < kMaxMarks; ++i)
        if (cudaEventCreate(&ep->marks[i]) != cudaSuccess) { release(ep); return RF_ERR_CUDA; }
    if (cudaDeviceSynchronize() != cudaSuccess) { release(ep); return RF_ERR_CUDA; }
    ep->connected = c->world == 1;
    *out = ep;
    return RF_OK;
}

int rf_moe_ep_handles(RfMoeEp* ep, unsigned char* handles) {
    if (!ep || !handles) return RF_ERR_NULL_POINTER;
    for (int b = 0; b < kPeerBuffers; ++b) {
        cudaIpcMemHandle_t h;
        if (cudaIpcGetMemHandle(&h, ep->mine[b]) != cudaSuccess) { cudaGetLastError(); return RF_ERR_CUDA; }
        memcpy(handles + 64 * b, &h, 64);
    }
    return RF_OK;
}

int rf_moe_ep_connect(RfMoeEp* ep, const unsigned char* all_handles) {
    if (!ep || !all_handles) return RF_ERR_NULL_POINTER;
    if (ep->connected) return RF_OK;
    for (int r = 0; r < ep->cfg.world; ++r) {
        if (r == ep->cfg.rank) continue;
        for (int b = 0; b < kPeerBuffers; ++b) {
            cudaIpcMemHandle_t h;
            memcpy(&h, all_handles + ((size_t)r * kPeerBuffers + b) * 64, 64);
            void* p = nullptr;
            if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                cudaGetLastError();
                return RF_ERR_CUDA;
            }
            ep->all[b][r] = p;
            ep->opened[b][r] = true;
        }
    }
    ep->connected = true;
    return RF_OK;
}

int rf_moe_ep_set_weights(RfMoeEp* ep, const void* router_weight, const float* router_bias,
                          const void* const* expert_gate, const void* const* expert_up,
                          const void* const* expert_down, const void* shared_gate, const void* shared_up,
                          const void* shared_down) {
    if (!ep || !router_weight || !expert_gate || !expert_up || !expert_down || !shared_gate || !shared_up ||
        !shared_down)
        return RF_ERR_NULL_POINTER;
    for (int j = 0; j < ep->E_loc; ++j) {
        if (!expert_gate[j] || !expert_up[j] || !expert_down[j]) return RF_ERR_NULL_POINTER;
        ep->w_gate[j] = expert_gate[j];
        ep->w_up[j] = expert_up[j];
        ep->w_down[j] = expert_down[j];
    }
    ep->router_w = router_weight;
    ep->router_bias = router_bias;
    ep->s_gate = shared_gate;
    ep->s_up = shared_up;
    ep->s_down = shared_down;
    return RF_OK;
}

int rf_moe_ep_set_option(RfMoeEp* ep, int option, int value) {
    if (!ep) return RF_ERR_NULL_POINTER;
    switch (option) {
        case RF_MOE_EP_OPT_TRACE: ep->trace = value != 0; ep->n_marks = 0; return RF_OK;
        case RF_MOE_EP_OPT_DISPATCH_BLOCKS:
            if (value < 0 || value > 64) return RF_ERR_BAD_SHAPE;
            ep->dispatch_blocks = value;
            return RF_OK;
        default: return RF_ERR_UNSUPPORTED;
    }
}

int rf_moe_ep_forward(RfMoeEp* ep, const void* x, void* out, rf_stream_t stream) {
    if (!ep || !x || !out) return RF_ERR_NULL_POINTER;
    if (!ep->connected || !ep->router_w) return RF_ERR_UNSUPPORTED;
    rf::DeviceState* st = rf::device_state();
    if (!st) return RF_ERR_CUDA;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const RfMoeEpConfig& c = ep->cfg;
    const int T = c.n_tokens, K = c.n_experts_per_token, E = c.n_routed_experts, d = c.d_hidden, f = c.d_expert;
    int rc;
    ep->n_marks = 0;
    mark(ep, s);
    if ((rc = rf_moe_router_gemm(x, ep->router_w, ep->router_bias, T, E, d, ep->scores, stream)) != RF_OK) return rc;
    if ((rc = rf_moe_topk(ep->scores, T, E, K, ep->idx, ep->gate_w, ep->source_rows, stream)) != RF_OK) return rc;
    if ((rc = rf_moe_permute(ep->idx, ep->source_rows, ep->gate_w, T, E, K, ep->perm_experts, ep->perm_rows, ep->first,
                             ep->rev, ep->exp_w, ep->sort_scratch, stream)) != RF_OK)
        return rc;
    // pair counts per global expert (differences of the sorted order's offsets), all-gathered through peer
    // memory; the rendezvous also orders this step after every rank's previous combine
    if ((rc = rendezvous(ep, ep->first, s)) != RF_OK) return rc;
    mark(ep, s);
    const int* counts_all = static_cast<const int*>(ep->mine[kBufSync]) + 8;
    if (rf::moe_ep_layout_launch(counts_all, c.rank, c.world, E, ep->capacity, ep->send_base, ep->recv_offsets,
                                 st->status, s) != cudaSuccess)
        return RF_ERR_CUDA;
    // Dispatch on the side stream; the shared expert, which needs no exchange, on the main stream.
    if (cudaEventRecord(ep->ev_ready, s) != cudaSuccess || cudaStreamWaitEvent(ep->side, ep->ev_ready, 0) != cudaSuccess)
        return RF_ERR_CUDA;
    rf::PeerPtrs px, pm;
    for (int i = 0; i < 8; ++i) {
        px.p[i] = ep->all[kBufRecvX][i < c.world ? i : 0];
        pm.p[i] = ep->all[kBufMeta][i < c.world ? i : 0];
    }
    if (rf::moe_ep_dispatch_launch(x, ep->perm_experts, ep->perm_rows, ep->first, ep->send_base, T, ep->n_pairs, d * 2,
                                   ep->E_loc, c.rank, c.world, ep->capacity, px, ep->push ? &pm : nullptr,
                                   ep->pair_rank, ep->pair_row, ep->push ? ep->mine[kBufY] : nullptr, st->status,
                                   st->num_sms, ep->dispatch_blocks, ep->side) != cudaSuccess)
        return RF_ERR_CUDA;
    if (cudaEventRecord(ep->ev_sent, ep->side) != cudaSuccess) return RF_ERR_CUDA;
    // SM partition: while the dispatch blocks own `dispatch_blocks` SMs, the shared expert's persistent GEMMs
    // run with that many CTAs fewer, so both really run at the same time.
    if (ep->dispatch_blocks > 0) rf_moe_set_grid_limit(st->num_sms - ep->dispatch_blocks);
    const void* sg[1] = {ep->s_gate};
    const void* su[1] = {ep->s_up};
    const void* sd[1] = {ep->s_down};
    rc = rf_moe_grouped_gemm(x, T, sg, su, ep->single_offsets, 1, ep->fs, d, ep->sh1, stream);
    if (rc == RF_OK) rc = rf_moe_grouped_gemm(ep->sh1, T, sd, nullptr, ep->single_offsets, 1, d, ep->fs, ep->sh2, stream);
    rf_moe_set_grid_limit(0);
    if (rc != RF_OK) return rc;
    if (cudaStreamWaitEvent(s, ep->ev_sent, 0) != cudaSuccess) return RF_ERR_CUDA;
    mark(ep, s);
    if ((rc = rendezvous(ep, nullptr, s)) != RF_OK) return rc;          // every rank's dispatch has landed
    mark(ep, s);
    if ((rc = rf_moe_grouped_gemm(ep->mine[kBufRecvX], ep->capacity, ep->w_gate.data(), ep->w_up.data(),
                                  ep->recv_offsets, ep->E_loc, f, d, ep->h, stream)) != RF_OK)
        return rc;
    mark(ep, s);
    if (ep->push) {
        rc = rf_moe_grouped_gemm_scatter(ep->h, ep->capacity, ep->w_down.data(), ep->recv_offsets, ep->E_loc, d, f,
                                         static_cast<const int*>(ep->mine[kBufMeta]), ep->all[kBufY], c.world, stream);
    } else {
        rc = rf_moe_grouped_gemm(ep->h, ep->capacity, ep->w_down.data(), nullptr, ep->recv_offsets, ep->E_loc, d, f,
                                 ep->mine[kBufY], stream);
    }
    if (rc != RF_OK) return rc;
    mark(ep, s);
    if ((rc = rendezvous(ep, nullptr, s)) != RF_OK) return rc;          // every rank's expert outputs are complete
    mark(ep, s);
    if (ep->push) {
        rc = rf_moe_combine(ep->mine[kBufY], ep->sh2, ep->rev, ep->exp_w, T, K, d, out, stream);
    } else {
        rc = rf_moe_ep_combine(ep->all[kBufY], ep->sh2, ep->rev, ep->exp_w, ep->pair_rank, ep->pair_row, T, K, d,
                               c.world, out, stream);
    }
    if (rc != RF_OK) return rc;
    mark(ep, s);
    return RF_OK;
}

int rf_moe_ep_stage_times(RfMoeEp* ep, float* ms, const char** names, int max_stages) {
    if (!ep || !ms) return 0;
    if (ep->n_marks < 2) return 0;
    cudaEventSynchronize(ep->marks[ep->n_marks - 1]);
    int n = 0;
    for (int i = 1; i < ep->n_marks && n < max_stages; ++i, ++n) {
        cudaEventElapsedTime(&ms[n], ep->marks[i - 1], ep->marks[i]);
        if (names) names[n] = kMarkNames[i];
    }
    return n;
}

int rf_moe_ep_buffer(RfMoeEp* ep, int which, void** ptr, size_t* bytes) {
    if (!ep || !ptr || !bytes) return RF_ERR_NULL_POINTER;
    const RfMoeEpConfig& c = ep->cfg;
    const size_t T = c.n_tokens, TK = ep->n_pairs, E = c.n_routed_experts;
    switch (which) {
        case RF_MOE_EP_BUF_SCORES: *ptr = ep->scores; *bytes = T * E * 2; break;
        case RF_MOE_EP_BUF_INDEX: *ptr = ep->idx; *bytes = TK * 4; break;
        case RF_MOE_EP_BUF_COUNTS_ALL:
            *ptr = static_cast<int*>(ep->mine[kBufSync]) + 8;
            *bytes = (size_t)c.world * E * 4;
            break;
        case RF_MOE_EP_BUF_SEND_BASE: *ptr = ep->send_base; *bytes = E * 4; break;
        case RF_MOE_EP_BUF_RECV_OFFSETS: *ptr = ep->recv_offsets; *bytes = (size_t)(ep->E_loc + 1) * 4; break;
        case RF_MOE_EP_BUF_PAIR_RANK: *ptr = ep->pair_rank; *bytes = TK * 4; break;
        default: return RF_ERR_UNSUPPORTED;
    }
    return RF_OK;
}

int rf_moe_ep_disconnect(RfMoeEp* ep) {
    if (!ep) return RF_ERR_NULL_POINTER;
    if (cudaDeviceSynchronize() != cudaSuccess) return RF_ERR_CUDA;
    for (int b = 0; b < kPeerBuffers; ++b)
        for (int r = 0; r < 8; ++r)
            if (ep->opened[b][r]) {
                cudaIpcCloseMemHandle(ep->all[b][r]);
                ep->opened[b][r] = false;
                ep->all[b][r] = nullptr;
            }
    ep->connected = false;
    return RF_OK;
}

int rf_moe_ep_destroy(RfMoeEp* ep) {
    if (!ep) return RF_ERR_NULL_POINTER;
    release(ep);
    return RF_OK;
}

}  // extern "C"
