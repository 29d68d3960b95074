"""ctypes binding of librf_b200.so (the C ABI declared in include/rf_b200.h).

There is no fallback: if the shared library is missing or a symbol cannot be
resolved, importing the binding raises.
"""
import ctypes
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "librf_b200.so")

RF_OK = 0
STATUS_NAMES = {
    0: "RF_OK", 1: "RF_ERR_BAD_SHAPE", 2: "RF_ERR_NULL_POINTER", 3: "RF_ERR_MISALIGNED", 4: "RF_ERR_WORKSPACE",
    5: "RF_ERR_CUDA", 6: "RF_ERR_DEVICE_TIMEOUT", 7: "RF_ERR_UNSUPPORTED", 8: "RF_ERR_COMM",
}


class RfError(RuntimeError):
    def __init__(self, what: str, status: int):
        super().__init__(f"{what}: {STATUS_NAMES.get(status, status)}")
        self.status = status


class PerfMetricEntry(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char * 20), ("time", ctypes.c_float), ("gflops", ctypes.c_float)]


class PerfMetrics(ctypes.Structure):
    _fields_ = [("count", ctypes.c_int), ("entries", PerfMetricEntry * 20)]


class InputParams(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in (
        "batch_size", "seq_len", "d_hidden", "d_expert", "n_routed_experts", "n_experts_per_token",
        "n_shared_experts", "seed")]


_MOE_PTR_FIELDS = (
    "expert_weight_gate_transposed", "expert_weight_up_transposed", "expert_weight_down_transposed",
    "input_seq",
    "shared_expert_weight_gate", "shared_expert_weight_gate_transposed",
    "shared_expert_weight_up", "shared_expert_weight_up_transposed",
    "shared_expert_weight_down", "shared_expert_weight_down_transposed",
    "router_weight", "expert_scores", "seq_experts_index", "seq_experts_softmax", "source_rows",
    "permuted_experts", "permuted_rows", "first_token_offset", "expanded_seq_input", "expanded_seq_softmax",
    "rev_permuted_rows", "expanded_fc1_output", "expanded_fc1_gate_splitk", "expanded_fc1_up_splitk",
    "expanded_fc2_output", "expanded_fc2_splitk", "shared_fc1_output", "shared_fc1_gate_splitk",
    "shared_fc1_up_splitk", "shared_fc2_output", "shared_fc2_splitk", "final_output", "final_output_splitk",
)


class MoEInputRaw(ctypes.Structure):
    _fields_ = (
        [("params", InputParams),
         ("expert_weight_gate", ctypes.POINTER(ctypes.c_void_p)),
         ("expert_weight_up", ctypes.POINTER(ctypes.c_void_p)),
         ("expert_weight_down", ctypes.POINTER(ctypes.c_void_p))]
        + [(n, ctypes.c_void_p) for n in _MOE_PTR_FIELDS]
    )


_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing - build it with `python -m radeonflow_kernels_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        _lib = ctypes.CDLL(LIB_PATH)
        _declare(_lib)
        _declare_ep(_lib)
    return _lib


def _declare(L: ctypes.CDLL) -> None:
    vp, ci, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    L.rf_version.restype = ctypes.c_char_p
    L.rf_version.argtypes = []
    L.rf_device_status.restype = ci
    L.rf_device_status.argtypes = [ctypes.POINTER(ci)]
    L.run.restype = None
    L.run.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ctypes.POINTER(PerfMetrics), vp]
    L.rf_fp8_gemm.restype = ci
    L.rf_fp8_gemm.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, vp, sz, vp]
    L.rf_fp8_gemm_workspace_bytes.restype = sz
    L.rf_fp8_gemm_workspace_bytes.argtypes = [ci, ci, ci, ci]
    L.rf_fp8_gemm_choose_split.restype = ci
    L.rf_fp8_gemm_choose_split.argtypes = [ci, ci, ci]
    L.rf_fp8_gemm_set_plan.restype = ci
    L.rf_fp8_gemm_set_plan.argtypes = [ci, ci, ci, ci, ci]
    L.rf_fp8_gemm_work_pieces.restype = ci
    L.rf_fp8_gemm_work_pieces.argtypes = [ci] * 7 + [ctypes.POINTER(ci), ci]
    L.rf_fp8_gemm_get_plan.restype = ci
    L.rf_fp8_gemm_get_plan.argtypes = [ci, ci, ci, ctypes.POINTER(ci), ctypes.POINTER(ci)]
    L.rf_fp8_gemm_load_plans.restype = ci
    L.rf_fp8_gemm_load_plans.argtypes = [ctypes.c_char_p]
    L.rf_fp8_gemm_colmajor.restype = ci
    L.rf_fp8_gemm_colmajor.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, vp, sz, vp]
    L.rf_fp8_gemm_colmajor_fnuz.restype = ci
    L.rf_fp8_gemm_colmajor_fnuz.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, vp, sz, vp]
    L.rf_fp8_gemm_static_scratch.restype = ci
    L.rf_fp8_gemm_static_scratch.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, vp]
    L.rf_fp8_gemm_static_status.restype = ci
    L.rf_fp8_gemm_static_status.argtypes = [ctypes.POINTER(ci)]
    L.rf_set_wait_limit_ns.restype = ci
    L.rf_set_wait_limit_ns.argtypes = [ctypes.c_ulonglong]
    # ---- MoE
    pm = ctypes.POINTER(PerfMetrics)
    raw = ctypes.POINTER(MoEInputRaw)
    ull = ctypes.c_ulonglong
    pull = ctypes.POINTER(ull)
    L.run_topk.restype = ci
    L.run_topk.argtypes = [raw, vp, pm]
    L.rf_moe_forward.restype = ci
    L.rf_moe_forward.argtypes = [raw, vp, vp, pm]
    L.initialize_workspace.restype = None
    L.initialize_workspace.argtypes = [ctypes.POINTER(vp)]
    L.rf_moe_workspace_bytes.restype = sz
    L.rf_moe_workspace_bytes.argtypes = [ctypes.POINTER(InputParams)]
    L.rf_moe_bind_workspace.restype = ci
    L.rf_moe_bind_workspace.argtypes = [raw, vp, sz]
    L.rf_run_from_python.restype = ci
    L.rf_run_from_python.argtypes = [ci] * 7 + [ull, ull, pull, pull, pull, ull, ull, ull, ull, ull, vp]
    L.rf_moe_topk.restype = ci
    L.rf_moe_topk.argtypes = [vp, ci, ci, ci, vp, vp, vp, vp]
    L.rf_moe_permute_scratch_bytes.restype = sz
    L.rf_moe_permute_scratch_bytes.argtypes = [ci, ci]
    L.rf_moe_permute.restype = ci
    L.rf_moe_permute.argtypes = [vp, vp, vp, ci, ci, ci, vp, vp, vp, vp, vp, vp, vp]
    L.rf_moe_gather_rows.restype = ci
    L.rf_moe_gather_rows.argtypes = [vp, vp, ci, ci, ci, vp, vp]
    L.rf_moe_grouped_gemm.restype = ci
    L.rf_moe_grouped_gemm.argtypes = [vp, ci, ctypes.POINTER(vp), ctypes.POINTER(vp), vp, ci, ci, ci, vp, vp]
    L.rf_moe_router_gemm.restype = ci
    L.rf_moe_router_gemm.argtypes = [vp, vp, vp, ci, ci, ci, vp, vp]
    L.rf_moe_set_fused_gather.restype = ci
    L.rf_moe_set_fused_gather.argtypes = [ci]
    L.rf_moe_set_grid_limit.restype = ci
    L.rf_moe_set_grid_limit.argtypes = [ci]
    L.rf_moe_set_map_cache_sets.restype = ci
    L.rf_moe_set_map_cache_sets.argtypes = [ci]
    L.rf_moe_combine.restype = ci
    L.rf_moe_combine.argtypes = [vp, vp, vp, vp, ci, ci, ci, vp, vp]
    # ---- multi-GPU
    pvp = ctypes.POINTER(vp)
    pub = ctypes.POINTER(ctypes.c_ubyte)
    L.rf_peer_alloc.restype = ci
    L.rf_peer_alloc.argtypes = [sz, pvp, pub]
    L.rf_peer_open.restype = ci
    L.rf_peer_open.argtypes = [pub, pvp]
    L.rf_peer_close.restype = ci
    L.rf_peer_close.argtypes = [vp]
    L.rf_peer_free.restype = ci
    L.rf_peer_free.argtypes = [vp]
    L.rf_fp8_gemm_nsplit.restype = ci
    L.rf_fp8_gemm_nsplit.argtypes = [vp, vp, vp, vp, pvp, ci, ci, ci, ci, ci, vp]
    L.rf_moe_add_rows.restype = ci
    L.rf_moe_add_rows.argtypes = [vp, vp, ci, ci, vp]
    L.rf_moe_ep_rendezvous.restype = ci
    L.rf_moe_ep_rendezvous.argtypes = [pvp, vp, ci, ci, ci, ci, vp]
    L.rf_moe_ep_layout.restype = ci
    L.rf_moe_ep_layout.argtypes = [vp, ci, ci, ci, ci, vp, vp, vp]
    L.rf_moe_ep_dispatch.restype = ci
    L.rf_moe_ep_dispatch.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, pvp, pvp, vp, vp, vp, vp]
    L.rf_moe_grouped_gemm_scatter.restype = ci
    L.rf_moe_grouped_gemm_scatter.argtypes = [vp, ci, pvp, vp, ci, ci, ci, vp, pvp, ci, vp]
    L.rf_moe_ep_combine.restype = ci
    L.rf_moe_ep_combine.argtypes = [pvp, vp, vp, vp, vp, vp, ci, ci, ci, ci, vp, vp]


class RfMoeEpConfig(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in (
        "n_tokens", "d_hidden", "d_expert", "n_routed_experts", "n_experts_per_token", "n_shared_experts",
        "rank", "world", "capacity", "push_results")]


RF_MOE_EP_HANDLE_BYTES = 256
(RF_MOE_EP_BUF_SCORES, RF_MOE_EP_BUF_INDEX, RF_MOE_EP_BUF_COUNTS_ALL, RF_MOE_EP_BUF_SEND_BASE,
 RF_MOE_EP_BUF_RECV_OFFSETS, RF_MOE_EP_BUF_PAIR_RANK) = range(6)
RF_MOE_EP_OPT_TRACE, RF_MOE_EP_OPT_DISPATCH_BLOCKS = 1, 2


def _declare_ep(L: ctypes.CDLL) -> None:
    vp, ci, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    pvp = ctypes.POINTER(vp)
    pub = ctypes.POINTER(ctypes.c_ubyte)
    L.rf_moe_ep_create.restype = ci
    L.rf_moe_ep_create.argtypes = [ctypes.POINTER(RfMoeEpConfig), pvp]
    L.rf_moe_ep_handles.restype = ci
    L.rf_moe_ep_handles.argtypes = [vp, pub]
    L.rf_moe_ep_connect.restype = ci
    L.rf_moe_ep_connect.argtypes = [vp, pub]
    L.rf_moe_ep_set_weights.restype = ci
    L.rf_moe_ep_set_weights.argtypes = [vp, vp, vp, pvp, pvp, pvp, vp, vp, vp]
    L.rf_moe_ep_forward.restype = ci
    L.rf_moe_ep_forward.argtypes = [vp, vp, vp, vp]
    L.rf_moe_ep_set_option.restype = ci
    L.rf_moe_ep_set_option.argtypes = [vp, ci, ci]
    L.rf_moe_ep_stage_times.restype = ci
    L.rf_moe_ep_stage_times.argtypes = [vp, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_char_p), ci]
    L.rf_moe_ep_buffer.restype = ci
    L.rf_moe_ep_buffer.argtypes = [vp, ci, pvp, ctypes.POINTER(sz)]
    L.rf_moe_ep_disconnect.restype = ci
    L.rf_moe_ep_disconnect.argtypes = [vp]
    L.rf_moe_ep_destroy.restype = ci
    L.rf_moe_ep_destroy.argtypes = [vp]


def check(status: int, what: str) -> None:
    if status != RF_OK:
        raise RfError(what, status)
